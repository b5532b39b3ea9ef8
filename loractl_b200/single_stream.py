"""The reference's own trunk block — the mirror of `SingleStreamBlock` and what it is made of in
crates/loractl-core/src/mmdit.rs (`ZRmsNorm` :282-330, RoPE :354-399, `MmditAttention` :540-665,
`SwiGlu` :670-708, `DoubleSharedModulation` :714-727, `SingleStreamBlock` :820-870).

It exists as the caller of the hot path with the REFERENCE's semantics: seven injectable sites per
block (`attn.wq`, `attn.wk`, `attn.wv`, `attn.wo`, `mlp.gate`, `mlp.up`, `mlp.down`) each routed
through `site()`, plus the un-adapted `attn.gate` projection.  With `Plain` bases it is plain
PyTorch f32 math and replays the reference's tiny golden trace on the CPU; after
`into_quantized` every site whose input width is a multiple of the quant block runs through
libloractl_b200 (sites that are not stay `Plain`, crates/loractl-core/src/mmdit.rs:1266-1280).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .adapters import LoraAdapters, LoraSite
from .linear import BaseLinear, QuantLinear, site

MASK_NEG = -3.0e4   # crates/loractl-core/src/mmdit.rs:85
SEQUENCE_PAD = 256  # crates/loractl-core/src/mmdit.rs:92


@dataclass
class MmditConfig:
    """The fields of `MmditConfig` (crates/loractl-core/src/mmdit.rs:95-125) the trunk block uses."""
    features: int
    heads: int
    kvheads: int
    multiplier: int = 4
    theta: float = 1e3

    @staticmethod
    def tiny() -> "MmditConfig":  # mmdit.rs:133-149
        return MmditConfig(features=96, heads=6, kvheads=2, multiplier=4, theta=1e3)

    @property
    def head_dim(self) -> int:
        return self.features // self.heads

    @staticmethod
    def rope_axes(head_dim: int) -> Tuple[int, int, int]:  # mmdit.rs:211-214
        unit = head_dim // 16
        return head_dim - 12 * unit, 6 * unit, 6 * unit

    @staticmethod
    def swiglu_dim(features: int, multiplier: int) -> int:  # mmdit.rs:218-221
        raw = (2 * features // 3) * multiplier
        return -(-raw // 128) * 128


class ZRmsNorm(nn.Module):
    """`x / sqrt(mean(x^2) + 1e-5) * (scale + 1)`, zero-initialised `scale` (mmdit.rs:282-330)."""

    def __init__(self, dim: int):
        super().__init__()
        self.scale = nn.Parameter(torch.zeros(dim), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and not self.scale.requires_grad:
            from .block_ops import zrmsnorm

            return zrmsnorm(x, self.scale)
        xf = x.float()
        var = xf.pow(2).mean(dim=-1, keepdim=True)
        return (xf / (var + 1e-5).sqrt() * (self.scale.float() + 1.0)).to(x.dtype)


def rope_tables(pos: torch.Tensor, head_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """`(cos, sin)`, each `[b, l, head_dim / 2]`, from 3-axis positions `[b, l, 3]` with per-axis
    frequency bands, computed in f64 like the reference (mmdit.rs:354-386)."""
    p = pos.to(torch.float64)
    cols = []
    for axis, dim in enumerate(MmditConfig.rope_axes(head_dim)):
        j = torch.arange(dim // 2, dtype=torch.float64, device=pos.device)
        omega = theta ** (-2.0 * j / dim)
        cols.append(p[..., axis:axis + 1] * omega)
    ang = torch.cat(cols, dim=-1)
    return ang.cos().float(), ang.sin().float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Consecutive-pair rotation on `[b, heads, l, head_dim]` (mmdit.rs:388-399)."""
    b, h, l, hd = x.shape
    pairs = x.reshape(b, h, l, hd // 2, 2)
    x0, x1 = pairs[..., 0], pairs[..., 1]
    c, s = cos.reshape(b, 1, l, hd // 2).to(x.dtype), sin.reshape(b, 1, l, hd // 2).to(x.dtype)
    return torch.stack([c * x0 - s * x1, s * x0 + c * x1], dim=-1).reshape(b, h, l, hd)


def additive_mask(mask: torch.Tensor) -> torch.Tensor:
    """0/1 key mask `[b, l]` -> additive `[b, 1, l, l]`: `MASK_NEG` wherever query (x) key is masked
    (mmdit.rs:1510-1517)."""
    b, l = mask.shape
    outer = mask.reshape(b, 1, l, 1) * mask.reshape(b, 1, 1, l)
    return (1.0 - outer) * MASK_NEG


def _fusable(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.is_cuda and a.dtype == b.dtype and a.dtype in (torch.float32, torch.bfloat16)


def _swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """`silu(gate) * up` (mmdit.rs:695-708): the fused kernel on the GPU, plain tensor ops elsewhere."""
    if _fusable(gate, up):
        from .block_ops import swiglu

        return swiglu(gate, up)
    return F.silu(gate) * up


def _sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """`x * sigmoid(gate)` (mmdit.rs:659-664)."""
    if _fusable(x, gate):
        from .block_ops import sigmoid_gate

        return sigmoid_gate(x, gate)
    return x * torch.sigmoid(gate)


def _plain(d_in: int, d_out: int) -> BaseLinear:
    return BaseLinear.plain(nn.Linear(d_in, d_out, bias=False))


class MmditAttention(nn.Module):
    """Gated-sigmoid GQA attention (mmdit.rs:540-665)."""

    def __init__(self, dim: int, heads: int, kvheads: int):
        super().__init__()
        hd = dim // heads
        self.wq, self.wk, self.wv = _plain(dim, hd * heads), _plain(dim, hd * kvheads), _plain(dim, hd * kvheads)
        self.gate, self.wo = _plain(dim, dim), _plain(dim, dim)
        self.qnorm, self.knorm = ZRmsNorm(hd), ZRmsNorm(hd)
        self.heads, self.kvheads = heads, kvheads

    def forward(self, x, rope, mask4, adapters: Optional[LoraAdapters], prefix: str) -> torch.Tensor:
        b, l, dim = x.shape
        heads, kv = self.heads, self.kvheads
        hd = dim // heads
        split = lambda t, n: t.reshape(b, l, n, hd).transpose(1, 2)
        q = split(site(adapters, f"{prefix}.wq", self.wq, x), heads)
        k = split(site(adapters, f"{prefix}.wk", self.wk, x), kv)
        v = split(site(adapters, f"{prefix}.wv", self.wv, x), kv)
        gate = self.gate(x)  # not an injectable site (mmdit.rs:611)
        q, k = self.qnorm(q), self.knorm(k)
        if rope is not None:
            q, k = apply_rope(q, *rope), apply_rope(k, *rope)
        groups = heads // kv  # GQA: repeat KV heads over their query groups (HF repeat_kv order)
        expand = lambda t: t.reshape(b, kv, 1, l, hd).expand(b, kv, groups, l, hd).reshape(b, heads, l, hd)
        k, v = expand(k), expand(v)
        ctx = F.scaled_dot_product_attention(q, k, v, attn_mask=None if mask4 is None else mask4.to(q.dtype))
        merged = ctx.transpose(1, 2).reshape(b, l, heads * hd)
        return site(adapters, f"{prefix}.wo", self.wo, _sigmoid_gate(merged, gate))


class SwiGlu(nn.Module):
    """`down(silu(gate(x)) * up(x))` (mmdit.rs:670-708)."""

    def __init__(self, features: int, multiplier: int):
        super().__init__()
        inner = MmditConfig.swiglu_dim(features, multiplier)
        self.gate, self.up, self.down = _plain(features, inner), _plain(features, inner), _plain(inner, features)

    def forward(self, x, adapters: Optional[LoraAdapters], prefix: str) -> torch.Tensor:
        gated = _swiglu(site(adapters, f"{prefix}.gate", self.gate, x), site(adapters, f"{prefix}.up", self.up, x))
        return site(adapters, f"{prefix}.down", self.down, gated)


class SingleStreamBlock(nn.Module):
    """One trunk block: modulated pre-norm attention + SwiGLU residuals (mmdit.rs:820-870)."""

    SITES = ("attn.wq", "attn.wk", "attn.wv", "attn.wo", "mlp.gate", "mlp.up", "mlp.down")

    def __init__(self, config: MmditConfig):
        super().__init__()
        self.config = config
        self.mod_lin = nn.Parameter(torch.zeros(6 * config.features), requires_grad=False)  # `blocks.N.mod.lin`
        self.prenorm, self.postnorm = ZRmsNorm(config.features), ZRmsNorm(config.features)
        self.attn = MmditAttention(config.features, config.heads, config.kvheads)
        self.mlp = SwiGlu(config.features, config.multiplier)

    # ---- construction -------------------------------------------------------------------
    @staticmethod
    def from_tensors(config: MmditConfig, tensors: Dict[str, torch.Tensor], prefix: str) -> "SingleStreamBlock":
        """Loads the checkpoint keys of one block (`{prefix}.attn.wq.weight` ... in file layout
        `[d_out, d_in]`, `{prefix}.mod.lin`, the norm scales)."""
        blk = SingleStreamBlock(config)
        get = lambda k: tensors[f"{prefix}.{k}"].detach().to(torch.float32)
        with torch.no_grad():
            blk.mod_lin.copy_(get("mod.lin"))
            blk.prenorm.scale.copy_(get("prenorm.scale"))
            blk.postnorm.scale.copy_(get("postnorm.scale"))
            blk.attn.qnorm.scale.copy_(get("attn.qknorm.qnorm.scale"))
            blk.attn.knorm.scale.copy_(get("attn.qknorm.knorm.scale"))
            for name, base in blk.base_linears():
                base.inner.weight.copy_(get(f"{name}.weight"))
        return blk

    def base_linears(self) -> List[Tuple[str, BaseLinear]]:
        """Every base linear of the block in the reference's order (mmdit.rs:1205-1257)."""
        a, m = self.attn, self.mlp
        return [("attn.wq", a.wq), ("attn.wk", a.wk), ("attn.wv", a.wv), ("attn.gate", a.gate), ("attn.wo", a.wo),
                ("mlp.gate", m.gate), ("mlp.up", m.up), ("mlp.down", m.down)]

    def injectable_sites(self, prefix: str) -> List[LoraSite]:
        sizes = dict((n, b) for n, b in self.base_linears())
        return [LoraSite(f"{prefix}.{n}", sizes[n].d_in, sizes[n].d_out) for n in self.SITES]

    def into_quantized(self, value: int, block: int = 32) -> Tuple[int, int]:
        """`Mmdit::into_quantized` for this block (mmdit.rs:1122-1158,1266-1280): every base linear
        whose input width is a multiple of the quant block becomes `Quant`; the rest stay `Plain`.
        Returns (quantized, left plain)."""
        done = left = 0
        for _, base in self.base_linears():
            lin = base.as_plain()
            if lin.in_features % block != 0:
                left += 1
                continue
            base.inner = QuantLinear.from_linear(lin, value, block=block)
            done += 1
        return done, left

    # ---- forward --------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, tvec: torch.Tensor, rope, mask4: Optional[torch.Tensor],
                adapters: Optional[LoraAdapters] = None, prefix: str = "blocks.0") -> torch.Tensor:
        f = self.config.features
        mod = tvec + self.mod_lin.to(tvec.dtype)  # [b, 1, 6f]
        prescale, preshift, pregate, postscale, postshift, postgate = (mod[..., i * f:(i + 1) * f] for i in range(6))
        attn_in = (prescale + 1.0) * self.prenorm(x) + preshift
        x = x + pregate * self.attn(attn_in, rope, mask4, adapters, f"{prefix}.attn")
        mlp_in = (postscale + 1.0) * self.postnorm(x) + postshift
        return x + postgate * self.mlp(mlp_in, adapters, f"{prefix}.mlp")


def pad_sequence(combined: torch.Tensor, mask: torch.Tensor, pos: torch.Tensor):
    """Zero-pads the combined [text | image] sequence to a multiple of 256 (mask false, positions
    zero), as `prepare_trunk` does (mmdit.rs:1395-1407)."""
    b, full, f = combined.shape
    pad = -(-full // SEQUENCE_PAD) * SEQUENCE_PAD - full
    if pad > 0:
        combined = torch.cat([combined, combined.new_zeros(b, pad, f)], dim=1)
        mask = torch.cat([mask, mask.new_zeros(b, pad)], dim=1)
        pos = torch.cat([pos, pos.new_zeros(b, pad, 3)], dim=1)
    return combined, mask, pos

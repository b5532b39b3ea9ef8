"""GPT-2-shaped decoder as a caller of the hot path — the mirror of crates/loractl-core/src/gpt2.rs
(`Gpt2Config` :66-104, `Attention` :106-177, `Mlp` :179-207, `Block` :209-250, `Gpt2` :266-470,
`site()` :482-492, `causal_mask` :498-506).

The reference's GPT-2 runs its four per-block projections (`attn.c_attn`, `attn.c_proj`,
`mlp.c_fc`, `mlp.c_proj`) through `site()` over PLAIN linears only.  Here each of them is a
`BaseLinear`, so `into_quantized` puts the same model on the quantized frozen-base path, and
`split_qkv=True` replaces the fused `c_attn` by three separate projections `attn.q`, `attn.k`,
`attn.v` (row ranges of the same weight) — the "LoRA on q/k/v/o" text-model benchmark
configuration, whose 768 x 768 sites are the small, bandwidth-bound quantized GEMMs.

Checkpoint layout is HF's: `Conv1D` weights are `[d_in, d_out]` and are transposed into the file
layout `[d_out, d_in]` the quantized path wants; LayerNorm `weight`/`bias`; the output head is tied
to `wte` (gpt2.rs:398-405).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from .adapters import LoraAdapters, LoraSite
from .linear import BaseLinear, QuantLinear, site


@dataclass
class Gpt2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    n_inner: int = 3072
    layer_norm_epsilon: float = 1e-5

    @staticmethod
    def tiny() -> "Gpt2Config":  # gpt2.rs:77-88
        return Gpt2Config(vocab_size=61, n_positions=16, n_embd=32, n_layer=2, n_head=2, n_inner=64)

    @staticmethod
    def gpt2_small() -> "Gpt2Config":  # gpt2.rs:93-103
        return Gpt2Config()


def _plain(d_in: int, d_out: int) -> BaseLinear:
    return BaseLinear.plain(nn.Linear(d_in, d_out, bias=True))


class Attention(nn.Module):
    def __init__(self, config: Gpt2Config, split_qkv: bool):
        super().__init__()
        e = config.n_embd
        self.split_qkv = split_qkv
        if split_qkv:
            self.q, self.k, self.v = _plain(e, e), _plain(e, e), _plain(e, e)
        else:
            self.c_attn = _plain(e, 3 * e)
        self.c_proj = _plain(e, e)

    def forward(self, x, n_head: int, adapters: Optional[LoraAdapters], prefix: str) -> torch.Tensor:
        b, s, e = x.shape
        if self.split_qkv:
            q, k, v = (site(adapters, f"{prefix}.attn.{n}", getattr(self, n), x) for n in ("q", "k", "v"))
        else:
            qkv = site(adapters, f"{prefix}.attn.c_attn", self.c_attn, x)
            q, k, v = qkv[..., :e], qkv[..., e:2 * e], qkv[..., 2 * e:]
        hd = e // n_head
        split = lambda t: t.reshape(b, s, n_head, hd).transpose(1, 2)
        # softmax(q k^T / sqrt(hd) + causal mask) v   (gpt2.rs:158-163,498-506)
        ctx = F.scaled_dot_product_attention(split(q), split(k), split(v), is_causal=True)
        return site(adapters, f"{prefix}.attn.c_proj", self.c_proj, ctx.transpose(1, 2).reshape(b, s, e))


class Mlp(nn.Module):
    def __init__(self, config: Gpt2Config):
        super().__init__()
        self.c_fc, self.c_proj = _plain(config.n_embd, config.n_inner), _plain(config.n_inner, config.n_embd)

    def forward(self, x, adapters: Optional[LoraAdapters], prefix: str) -> torch.Tensor:
        up = site(adapters, f"{prefix}.mlp.c_fc", self.c_fc, x)
        return site(adapters, f"{prefix}.mlp.c_proj", self.c_proj, F.gelu(up, approximate="tanh"))  # gelu_new


class Block(nn.Module):
    def __init__(self, config: Gpt2Config, split_qkv: bool):
        super().__init__()
        self.ln_1 = nn.LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.attn = Attention(config, split_qkv)
        self.ln_2 = nn.LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.mlp = Mlp(config)

    def forward(self, h, n_head: int, adapters: Optional[LoraAdapters], prefix: str) -> torch.Tensor:
        h = h + self.attn(self.ln_1(h), n_head, adapters, prefix)
        return h + self.mlp(self.ln_2(h), adapters, prefix)


class Gpt2(nn.Module):
    def __init__(self, config: Gpt2Config, split_qkv: bool = False):
        super().__init__()
        self.config, self.split_qkv = config, split_qkv
        self.wte = nn.Embedding(config.vocab_size, config.n_embd)
        self.wpe = nn.Embedding(config.n_positions, config.n_embd)
        self.h = nn.ModuleList(Block(config, split_qkv) for _ in range(config.n_layer))
        self.ln_f = nn.LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        for p in self.parameters():  # the base is frozen; only adapters train
            p.requires_grad_(False)

    # ---- construction -------------------------------------------------------------------
    @staticmethod
    def from_hf_tensors(config: Gpt2Config, tensors: Dict[str, torch.Tensor], split_qkv: bool = False) -> "Gpt2":
        m = Gpt2(config, split_qkv)
        get = lambda k: tensors[k].detach().to(torch.float32)
        e = config.n_embd
        with torch.no_grad():
            m.wte.weight.copy_(get("transformer.wte.weight"))
            m.wpe.weight.copy_(get("transformer.wpe.weight"))
            m.ln_f.weight.copy_(get("transformer.ln_f.weight"))
            m.ln_f.bias.copy_(get("transformer.ln_f.bias"))
            for i, blk in enumerate(m.h):
                p = f"transformer.h.{i}"
                for ln in ("ln_1", "ln_2"):
                    getattr(blk, ln).weight.copy_(get(f"{p}.{ln}.weight"))
                    getattr(blk, ln).bias.copy_(get(f"{p}.{ln}.bias"))
                w, bias = get(f"{p}.attn.c_attn.weight").t(), get(f"{p}.attn.c_attn.bias")  # [3e, e], [3e]
                if split_qkv:
                    for j, n in enumerate(("q", "k", "v")):
                        lin = getattr(blk.attn, n).as_plain()
                        lin.weight.copy_(w[j * e:(j + 1) * e])
                        lin.bias.copy_(bias[j * e:(j + 1) * e])
                else:
                    blk.attn.c_attn.as_plain().weight.copy_(w)
                    blk.attn.c_attn.as_plain().bias.copy_(bias)
                for mod, name in ((blk.attn, "attn.c_proj"), (blk.mlp, "mlp.c_fc"), (blk.mlp, "mlp.c_proj")):
                    lin = getattr(mod, name.split(".")[1]).as_plain()
                    lin.weight.copy_(get(f"{p}.{name}.weight").t())
                    lin.bias.copy_(get(f"{p}.{name}.bias"))
        return m

    def base_linears(self):
        """(path, BaseLinear) of every per-block projection, in forward order."""
        out = []
        for i, blk in enumerate(self.h):
            p = f"transformer.h.{i}"
            names = ("q", "k", "v") if self.split_qkv else ("c_attn",)
            out += [(f"{p}.attn.{n}", getattr(blk.attn, n)) for n in names]
            out += [(f"{p}.attn.c_proj", blk.attn.c_proj), (f"{p}.mlp.c_fc", blk.mlp.c_fc),
                    (f"{p}.mlp.c_proj", blk.mlp.c_proj)]
        return out

    def injectable_sites(self) -> List[LoraSite]:
        """gpt2.rs:428-456: every per-block projection with the widths a delta must match."""
        return [LoraSite(path, base.d_in, base.d_out) for path, base in self.base_linears()]

    def into_quantized(self, value: int, block: int = 32):
        """Quantizes every per-block projection whose input width is a multiple of the quant block
        (the rule of crates/loractl-core/src/mmdit.rs:1266-1280 applied to this model); embeddings,
        norms and the tied head stay as they are.  Returns (quantized, left plain)."""
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
    def hidden_states(self, ids: torch.Tensor, adapters: Optional[LoraAdapters] = None,
                      dtype: Optional[torch.dtype] = None):
        """(after_embed, after_block0, after_lnf) — the stages of `Gpt2Trace` (gpt2.rs:252-264)."""
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device).unsqueeze(0).expand(b, s)
        h = self.wte(ids) + self.wpe(pos)
        if dtype is not None:
            h = h.to(dtype)
        after_embed = h
        after_block0 = h
        for i, blk in enumerate(self.h):
            h = blk(h, self.config.n_head, adapters, f"transformer.h.{i}")
            if i == 0:
                after_block0 = h
        return after_embed, after_block0, self.ln_f(h)

    def forward(self, ids: torch.Tensor, adapters: Optional[LoraAdapters] = None,
                dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Logits `[batch, seq, vocab]` through the tied head `h . wte^T` (gpt2.rs:398-405)."""
        after_lnf = self.hidden_states(ids, adapters, dtype)[2]
        return after_lnf @ self.wte.weight.to(after_lnf.dtype).t()


def next_token_loss(logits: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Mean cross-entropy of position t's logits against token t + 1, in f32."""
    v = logits.shape[-1]
    return F.cross_entropy(logits[:, :-1].reshape(-1, v).float(), ids[:, 1:].reshape(-1))

"""Quantized linear + the adapter attach seam — the mirror of
crates/loractl-core/src/mmdit.rs:401-536 (`QuantLinear`, `BaseLinear`, `site`).

Where the reference runs `base.forward(x)` and then `adapters.apply(...)` as separate
tensor ops, a site whose base is quantized is ONE call into libloractl_b200 here
(`lq_linear_fwd` / `lq_linear_bwd`): frozen GEMM, bias, rank-r delta and `alpha/rank`
together, behind a `torch.autograd.Function`.
"""
from __future__ import annotations

from typing import List, Optional, Union

import torch
from torch import nn

from . import quant as Q
from .adapters import LoraAdapters
from .lora import LoraDelta


class QuantLinear(nn.Module):
    """crates/loractl-core/src/mmdit.rs:413-428.  `weight` is the frozen quantized weight in
    file layout `[d_out, d_in]`; `rows` records the row-chunk layout the reference would
    use (quant.rs:102-117) — here chunks are row ranges of one packed buffer, so the forward
    is a single kernel whatever the layout.  `bias` stays f32."""

    def __init__(self, weight: Union[Q.QuantWeight, List[Q.QuantWeight]], bias: Optional[torch.Tensor] = None):
        super().__init__()
        chunks = weight if isinstance(weight, list) else [weight]
        self.rows = [c.d_out for c in chunks]
        self.weight = Q.concat_chunks(chunks)
        self.d_out, self.d_in = self.weight.d_out, self.weight.d_in
        self.bias = None
        if bias is not None:
            self.bias = bias.detach().to(self.weight.device, torch.float32).contiguous()
            self.weight.set_bias(self.bias)

    @staticmethod
    def from_linear(lin: nn.Linear, value: int, chunk_bytes: int = 0, block: int = Q.QUANT_BLOCK) -> "QuantLinear":
        """`Mmdit::into_quantized_chunked` for one site (mmdit.rs:1134-1158,1266-1280).
        torch's `nn.Linear.weight` is already `[d_out, d_in]`, so no transpose is needed."""
        chunks = Q.quantize_linear_weight_chunked(lin.weight.detach(), value, chunk_bytes, block)
        return QuantLinear(chunks, lin.bias.detach() if lin.bias is not None else None)

    def dequantized_weight(self) -> torch.Tensor:
        """mmdit.rs:435-444 — diagnostics only."""
        return self.weight.dequantize()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _fused(self.weight, x, None)


class BaseLinear(nn.Module):
    """crates/loractl-core/src/mmdit.rs:451-520: `Plain(Linear)` or `Quant(QuantLinear)`."""

    def __init__(self, inner: nn.Module):
        super().__init__()
        self.inner = inner

    @staticmethod
    def plain(lin: nn.Linear) -> "BaseLinear":
        return BaseLinear(lin)

    @staticmethod
    def quant(q: QuantLinear) -> "BaseLinear":
        return BaseLinear(q)

    @property
    def is_quant(self) -> bool:
        return isinstance(self.inner, QuantLinear)

    @property
    def d_in(self) -> int:
        return self.inner.d_in if self.is_quant else self.inner.in_features

    @property
    def d_out(self) -> int:
        return self.inner.d_out if self.is_quant else self.inner.out_features

    def as_plain(self) -> nn.Linear:
        if self.is_quant:
            raise RuntimeError("BaseLinear::as_plain called on a quantized (Quant) site")
        return self.inner

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.inner(x)


def _grads_live_in(bucket, a: torch.Tensor, b: torch.Tensor) -> bool:
    """True when `a.grad` / `b.grad` currently ARE the bucket views: only then may the backward add
    into the bucket itself (a caller that reset `.grad` expects autograd to fill it)."""
    return (bucket is not None and a.grad is not None and b.grad is not None
            and a.grad.data_ptr() == bucket[0].data_ptr() and b.grad.data_ptr() == bucket[1].data_ptr())


class _LoraLinearFn(torch.autograd.Function):
    """One LoRA'd quantized site.  Saves x and H = x.A for the backward; the frozen weight is
    state (quant.rs:217-219), never a graph parent."""

    @staticmethod
    def forward(ctx, x2, a, b, wq, scaling, mirror, bucket=None):
        """`bucket` = (dA view, dB view) of a flat gradient buffer: the backward adds into them in place
        (what autograd's accumulation into `.grad` would do with two more kernels) and returns no
        gradient for `a`, `b`."""
        y, h = Q.linear_fwd_raw(wq, x2, a, b, scaling, mirror=mirror)
        ctx.wq, ctx.scaling, ctx.mirror, ctx.bucket = wq, scaling, mirror, bucket
        ctx.save_for_backward(x2, h, a, b)
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, h, a, b = ctx.saved_tensors
        need_dx, need_da, need_db = ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2]
        if _grads_live_in(ctx.bucket, a, b):
            dx, _, _ = Q.linear_bwd_raw(ctx.wq, dy.contiguous(), x2, h, a, b, ctx.scaling, need_dx=need_dx,
                                        need_da=need_da, need_db=need_db, da_out=ctx.bucket[0], db_out=ctx.bucket[1],
                                        accumulate=True, mirror=ctx.mirror)
            return dx, None, None, None, None, None, None
        dx, da, db = Q.linear_bwd_raw(ctx.wq, dy.contiguous(), x2, h, a, b, ctx.scaling,
                                      need_dx=need_dx, need_da=need_da, need_db=need_db, mirror=ctx.mirror)
        return dx, da, db, None, None, None, None


def _fused(wq: Q.QuantWeight, x: torch.Tensor, delta: Optional[LoraDelta]) -> torch.Tensor:
    """`BaseLinear::forward`'s Quant arm (mmdit.rs:487-519): flatten the leading dims to
    `[n, d_in]`, run the op, reshape back with `d_out` last."""
    if x.shape[-1] != wq.d_in:
        raise ValueError(f"last dim {x.shape[-1]} != d_in {wq.d_in}")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, wq.d_in).contiguous()
    if delta is None:
        y = Q._QuantMatmulT.apply(x2, wq)
    else:
        if delta.dropout > 0.0 and delta.training:
            raise RuntimeError(
                "lora.dropout > 0 is not supported on a quantized site of the b200 backend "
                "(the fused kernel has no dropout; the reference also forbids it under recompute)")
        # bf16 activations take the tensor-core path, which wants the factors as bf16 operands
        mirror = delta.operand_mirror() if x2.dtype == torch.bfloat16 else None
        y = _LoraLinearFn.apply(x2, delta.lora_a, delta.lora_b, wq, delta.scaling, mirror, delta.bucket_grads)
    return y.reshape(*lead, wq.d_out)


class _GroupedLoraLinearFn(torch.autograd.Function):
    """Several LoRA'd quantized sites on the same input: one grouped forward; the backward runs each
    site's own `lq_linear_bwd` (dX contributions add up, as autograd would add them)."""

    @staticmethod
    def forward(ctx, x2, meta, *factors):
        sites = []
        for i, (wq, scaling, has_delta, _, _) in enumerate(meta):
            a, b = (factors[2 * i], factors[2 * i + 1]) if has_delta else (None, None)
            sites.append((wq, a, b, scaling))
        outs = Q.linear_fwd_grouped_raw(sites, x2)
        ctx.meta = meta
        ctx.save_for_backward(x2, *[h if h is not None else x2.new_empty(0) for _, h in outs], *factors)
        return tuple(y for y, _ in outs)

    @staticmethod
    def backward(ctx, *dys):
        n = len(ctx.meta)
        x2 = ctx.saved_tensors[0]
        hs = ctx.saved_tensors[1:1 + n]
        factors = ctx.saved_tensors[1 + n:]
        dx_total, grads = None, []
        for i, (wq, scaling, has_delta, mirror, bucket) in enumerate(ctx.meta):
            a, b = (factors[2 * i], factors[2 * i + 1]) if has_delta else (None, None)
            h = hs[i] if has_delta else None
            need_dx = ctx.needs_input_grad[0]
            direct = has_delta and _grads_live_in(bucket, a, b)
            dx, da, db = Q.linear_bwd_raw(wq, dys[i].contiguous(), x2, h, a, b, scaling, need_dx=need_dx,
                                          need_da=has_delta and ctx.needs_input_grad[2 + 2 * i],
                                          need_db=has_delta and ctx.needs_input_grad[3 + 2 * i], mirror=mirror,
                                          da_out=bucket[0] if direct else None, db_out=bucket[1] if direct else None,
                                          accumulate=direct)
            if dx is not None:
                dx_total = dx if dx_total is None else dx_total + dx
            grads += [None, None] if direct else [da, db]
        return (dx_total, None, *grads)


def site_group(adapters: Optional[LoraAdapters], sites, x: torch.Tensor):
    """`site()` for several (path, base) pairs that read the SAME `x` — wq / wk / wv and gate / up in
    the reference (crates/loractl-core/src/mmdit.rs:599-610,701-706).  Quantized bases go through one
    grouped call; anything else falls back to `site()` one by one.  Returns the outputs in order."""
    deltas = [adapters.get(path) if adapters is not None else None for path, _ in sites]
    if not all(base.is_quant for _, base in sites) or not x.is_cuda:
        return [apply_site(base, d, x) for (_, base), d in zip(sites, deltas)]
    d_in = sites[0][1].d_in
    if x.shape[-1] != d_in or any(base.d_in != d_in for _, base in sites):
        raise ValueError("the sites of a group share x: their d_in must agree")
    for d in deltas:
        if d is not None and d.dropout > 0.0 and d.training:
            raise RuntimeError("lora.dropout > 0 is not supported on a quantized site of the b200 backend")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, d_in).contiguous()
    meta, factors = [], []
    for (_, base), d in zip(sites, deltas):
        mirror = d.operand_mirror() if (d is not None and x2.dtype == torch.bfloat16) else None
        meta.append((base.inner.weight, d.scaling if d is not None else 1.0, d is not None, mirror,
                     d.bucket_grads if d is not None else None))
        if d is not None:
            factors += [d.lora_a, d.lora_b]
        else:  # placeholders keep the argument positions regular
            factors += [x2.new_empty(0), x2.new_empty(0)]
    ys = _GroupedLoraLinearFn.apply(x2, tuple(meta), *factors)
    return [y.reshape(*lead, base.d_out) for y, (_, base) in zip(ys, sites)]


def apply_site(base: BaseLinear, delta: Optional[LoraDelta], x: torch.Tensor) -> torch.Tensor:
    if base.is_quant:
        return _fused(base.inner.weight, x, delta)
    out = base(x)
    return out if delta is None else out + delta(x)


def site(adapters: Optional[LoraAdapters], path: str, base: BaseLinear, x: torch.Tensor) -> torch.Tensor:
    """crates/loractl-core/src/mmdit.rs:526-536: run a base linear at an injectable site, adding
    any adapter registered for `path`."""
    delta = adapters.get(path) if adapters is not None else None
    return apply_site(base, delta, x)

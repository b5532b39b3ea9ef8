"""LoRA modules — the mirror of crates/loractl-core/src/lora.rs.

`LoraDelta` (base-free) and `LoraLinear` (base-owning) keep the reference's field names
(`lora_a`, `lora_b`, `scaling`, `dropout`) and layouts: `lora_a` is `[d_in, rank]`,
`lora_b` is `[rank, d_out]` (burn `Linear` layout, lora.rs:129-136), both f32 and
trainable; `lora_b` starts at zero so a fresh adapter is an exact no-op.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import nn


def init_factors(d_input: int, d_output: int, rank: int, device=None) -> Tuple[nn.Parameter, nn.Parameter]:
    """crates/loractl-core/src/lora.rs:123-137: A gets burn's default Linear init
    (Kaiming-uniform, gain 1/sqrt(3), fan-in = d_input  =>  U(-1/sqrt(d_input), 1/sqrt(d_input))),
    B is zeros."""
    bound = 1.0 / math.sqrt(d_input)
    a = torch.empty(d_input, rank, dtype=torch.float32, device=device).uniform_(-bound, bound)
    b = torch.zeros(rank, d_output, dtype=torch.float32, device=device)
    return nn.Parameter(a), nn.Parameter(b)


class LoraDelta(nn.Module):
    """crates/loractl-core/src/lora.rs:155-204: only the trainable factors and the scaling;
    `forward` returns the scaled delta `(alpha / rank) * B(A(x))`, never `base(x) + delta`."""

    def __init__(self, d_input: int, d_output: int, rank: int, alpha: float, dropout_prob: float = 0.0,
                 device=None):
        super().__init__()
        rank = max(int(rank), 1)  # lora.rs:185
        self.lora_a, self.lora_b = init_factors(d_input, d_output, rank, device)
        self.scaling = float(alpha) / rank
        self.dropout = float(dropout_prob)
        self.rank = rank
        # bf16 operand mirror of (lora_a, lora_b) for the tensor-core path, rebuilt when the factors
        # change; `param_epoch` is bumped by writers that bypass torch (the fused AdamW kernel)
        self._mirror: Optional[torch.Tensor] = None
        self._mirror_key = None
        self.param_epoch = [0]
        # (dA view, dB view) of a flat gradient bucket, set by `FlatAdapters`: the fused backward then adds
        # straight into them instead of returning fresh tensors for autograd to accumulate
        self.bucket_grads = None

    def _mirror_state(self):
        a, b = self.lora_a, self.lora_b
        return (a._version, b._version, a.data_ptr(), b.data_ptr(), self.param_epoch[0])

    def operand_mirror(self) -> Optional[torch.Tensor]:
        """The factors as bf16 GEMM operands (`lq_lora_mirror_update`), refreshed with one launch
        whenever `lora_a` / `lora_b` changed since it was built; None off the GPU."""
        a, b = self.lora_a, self.lora_b
        if not a.is_cuda:
            return None
        key = self._mirror_state()
        if self._mirror is None or self._mirror_key != key:
            from . import quant as Q

            self._mirror = Q.lora_mirror(a.detach(), b.detach(), self._mirror)
            self._mirror_key = key
        return self._mirror

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """The stand-alone delta (lora.rs:199-203), in plain tensor ops.  The fused kernel path
        does not call this: `site()` hands the factors to `lq_linear_fwd`.  It exists for
        sites whose base is a plain `Linear`."""
        if self.dropout > 0.0 and self.training:
            x = torch.nn.functional.dropout(x, self.dropout, True)
        return (x.to(torch.float32) @ self.lora_a @ self.lora_b).mul(self.scaling).to(x.dtype)


def freeze(module: nn.Module) -> nn.Module:
    """crates/loractl-core/src/lora.rs:211-214: mark every parameter as not requiring grad."""
    for p in module.parameters():
        p.requires_grad_(False)
    return module


class LoraLinear(nn.Module):
    """crates/loractl-core/src/lora.rs:34-111: a frozen base plus a LoRA adapter,
    `y = base(x) + (alpha / rank) * B(A(dropout(x)))`.  The base may be a plain `nn.Linear`
    or a quantized `QuantLinear`; with the latter the whole forward/backward is one fused
    call into the CUDA library."""

    def __init__(self, base: nn.Module, rank: int, alpha: float, dropout_prob: float = 0.0, device=None):
        super().__init__()
        from .linear import BaseLinear, QuantLinear  # local import: linear.py imports this module

        if isinstance(base, nn.Linear):
            d_in, d_out = base.in_features, base.out_features
            base = BaseLinear.plain(freeze(base))
        elif isinstance(base, QuantLinear):
            d_in, d_out = base.d_in, base.d_out
            base = BaseLinear.quant(base)
        elif isinstance(base, BaseLinear):
            d_in, d_out = base.d_in, base.d_out
        else:
            raise TypeError(f"unsupported base {type(base).__name__}")
        self.base = base
        self.delta = LoraDelta(d_in, d_out, rank, alpha, dropout_prob, device)

    @property
    def lora_a(self):
        return self.delta.lora_a

    @property
    def lora_b(self):
        return self.delta.lora_b

    @property
    def scaling(self):
        return self.delta.scaling

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .linear import apply_site

        return apply_site(self.base, self.delta, x)

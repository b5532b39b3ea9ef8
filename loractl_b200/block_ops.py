"""Fused element-wise companions of the LoRA'd linears inside a DiT block, with autograd:

    modulated_layer_norm(x, shift, scale) = layer_norm(x) * (1 + scale) + shift
    gated_residual(x, gate, y)            = x + gate * y
    swiglu(gate, up)                      = silu(gate) * up           (mmdit.rs:695-708)
    sigmoid_gate(x, gate)                 = x * sigmoid(gate)         (mmdit.rs:659-664)
    zrmsnorm(x, scale)                    = x / sqrt(mean(x^2) + 1e-5) * (scale + 1)   (mmdit.rs:282-330)

the pattern of crates/loractl-core/src/mmdit.rs:857-869 (`(prescale + 1) * prenorm(x) + preshift`,
`x + pregate * attn(..)`, ...).  `x`, `y` are `[b, tokens, h]`; `shift`, `scale`, `gate` are
`[b, 1, h]` (or `[b, h]`) and broadcast over the tokens of their sample.  Each op is one kernel
forward; the backward is one pass for the token-shaped gradient plus a fixed-order two-stage sum
over tokens for the modulation gradients (deterministic, as block-checkpoint recompute needs).
CUDA tensors only (f32 or bf16): like every other op of this package there is no CPU path.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from . import _lib as L
from .quant import _dtype_code, _require_cuda, _stream_ptr

LN_EPS = 1e-5  # torch.nn.functional.layer_norm's default, which the harness block used before

_WS: Dict[Tuple[torch.device, int], torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _WS.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WS[key] = ws
    return ws


def _dims(x: torch.Tensor) -> Tuple[int, int, int]:
    if x.dim() != 3:
        raise ValueError(f"expected [b, tokens, h], got {list(x.shape)}")
    return x.shape[0], x.shape[1], x.shape[2]


def _mod(v: torch.Tensor, b: int, h: int, like: torch.Tensor, name: str) -> torch.Tensor:
    if v.numel() != b * h:
        raise ValueError(f"{name} must hold [b = {b}, h = {h}] values, got {list(v.shape)}")
    return v.reshape(b, h).to(like.dtype).contiguous()


class _ModulatedLayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shift, scale):
        _require_cuda(x, "x")
        b, t, h = _dims(x)
        xc = x.contiguous()
        sh, sc = _mod(shift, b, h, xc, "shift"), _mod(scale, b, h, xc, "scale")
        y = torch.empty_like(xc)
        mean = torch.empty(b * t, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        with torch.cuda.device(x.device):
            L.check(L.lib().lq_ln_modulate_fwd(xc.data_ptr(), sh.data_ptr(), sc.data_ptr(), _dtype_code(xc), b, t, h,
                                               LN_EPS, y.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                               _stream_ptr(x.device)))
        ctx.save_for_backward(xc, sc, mean, rstd)
        ctx.shapes = (shift.shape, scale.shape, shift.dtype, scale.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, sc, mean, rstd = ctx.saved_tensors
        b, t, h = _dims(xc)
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        dshift = torch.empty((b, h), dtype=torch.float32, device=xc.device)
        dscale = torch.empty_like(dshift)
        with torch.cuda.device(xc.device):
            n = L.lib().lq_block_ops_workspace_bytes(b, t, h)
            ws = _workspace(xc.device, n)
            L.check(L.lib().lq_ln_modulate_bwd(dyc.data_ptr(), xc.data_ptr(), sc.data_ptr(), mean.data_ptr(),
                                               rstd.data_ptr(), _dtype_code(xc), b, t, h, dx.data_ptr(),
                                               dshift.data_ptr(), dscale.data_ptr(), ws.data_ptr(), ws.numel(),
                                               _stream_ptr(xc.device)))
        shs, scs, shd, scd = ctx.shapes
        return dx, dshift.to(shd).reshape(shs), dscale.to(scd).reshape(scs)


class _GatedResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, y):
        _require_cuda(y, "y")
        b, t, h = _dims(y)
        yc = y.contiguous()
        xc = x.to(yc.dtype).contiguous()
        g = _mod(gate, b, h, yc, "gate")
        out = torch.empty_like(yc)
        with torch.cuda.device(y.device):
            L.check(L.lib().lq_gate_residual_fwd(xc.data_ptr(), g.data_ptr(), yc.data_ptr(), _dtype_code(yc), b, t, h,
                                                 out.data_ptr(), _stream_ptr(y.device)))
        ctx.save_for_backward(g, yc)
        ctx.meta = (gate.shape, gate.dtype, x.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        g, yc = ctx.saved_tensors
        b, t, h = _dims(yc)
        dc = dout.contiguous()
        dy = torch.empty_like(yc)
        dgate = torch.empty((b, h), dtype=torch.float32, device=yc.device)
        with torch.cuda.device(yc.device):
            n = L.lib().lq_block_ops_workspace_bytes(b, t, h)
            ws = _workspace(yc.device, n)
            L.check(L.lib().lq_gate_residual_bwd(dc.data_ptr(), g.data_ptr(), yc.data_ptr(), _dtype_code(yc), b, t, h,
                                                 dy.data_ptr(), dgate.data_ptr(), ws.data_ptr(), ws.numel(),
                                                 _stream_ptr(yc.device)))
        gs, gd, xd = ctx.meta
        return dc.to(xd), dgate.to(gd).reshape(gs), dy


def modulated_layer_norm(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """`layer_norm(x, (h,)) * (1 + scale) + shift`, one kernel."""
    return _ModulatedLayerNorm.apply(x, shift, scale)


def gated_residual(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """`x + gate * y`, one kernel."""
    return _GatedResidual.apply(x, gate, y)


class _PairAct(torch.autograd.Function):
    """Element-wise map of two same-shaped tensors with both input gradients from one backward pass."""

    @staticmethod
    def forward(ctx, a, b, kind):
        _require_cuda(a, "input")
        if a.shape != b.shape or a.dtype != b.dtype:
            raise ValueError(f"operands must agree in shape and dtype, got {list(a.shape)} {a.dtype} / {list(b.shape)} {b.dtype}")
        ac, bc = a.contiguous(), b.contiguous()
        out = torch.empty_like(ac)
        fn = L.lib().lq_swiglu_fwd if kind == "swiglu" else L.lib().lq_sigmoid_gate_fwd
        with torch.cuda.device(a.device):
            L.check(fn(ac.data_ptr(), bc.data_ptr(), _dtype_code(ac), ac.numel(), out.data_ptr(), _stream_ptr(a.device)))
        ctx.save_for_backward(ac, bc)
        ctx.kind = kind
        return out

    @staticmethod
    def backward(ctx, dout):
        ac, bc = ctx.saved_tensors
        dc = dout.to(ac.dtype).contiguous()
        da, db = torch.empty_like(ac), torch.empty_like(bc)
        fn = L.lib().lq_swiglu_bwd if ctx.kind == "swiglu" else L.lib().lq_sigmoid_gate_bwd
        with torch.cuda.device(ac.device):
            L.check(fn(dc.data_ptr(), ac.data_ptr(), bc.data_ptr(), _dtype_code(ac), ac.numel(), da.data_ptr(),
                       db.data_ptr(), _stream_ptr(ac.device)))
        return da, db, None


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """`silu(gate) * up`, one kernel each way."""
    return _PairAct.apply(gate, up, "swiglu")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """`x * sigmoid(gate)`, one kernel each way."""
    return _PairAct.apply(x, gate, "sigmoid_gate")


ZRMS_EPS = 1e-5  # crates/loractl-core/src/mmdit.rs:282-330


class _ZRmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        _require_cuda(x, "x")
        h = x.shape[-1]
        if scale.numel() != h:
            raise ValueError(f"scale must hold {h} values, got {list(scale.shape)}")
        xc = x.contiguous()
        sc = scale.detach().to(torch.float32).contiguous()
        rows = xc.numel() // h
        y = torch.empty_like(xc)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            L.check(L.lib().lq_zrmsnorm_fwd(xc.data_ptr(), sc.data_ptr(), _dtype_code(xc), rows, h, ZRMS_EPS, y.data_ptr(),
                                            rstd.data_ptr(), _stream_ptr(x.device)))
        ctx.save_for_backward(xc, sc, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, sc, rstd = ctx.saved_tensors
        h = xc.shape[-1]
        dc = dy.to(xc.dtype).contiguous()
        dx = torch.empty_like(xc)
        with torch.cuda.device(xc.device):
            L.check(L.lib().lq_zrmsnorm_bwd(dc.data_ptr(), xc.data_ptr(), sc.data_ptr(), rstd.data_ptr(), _dtype_code(xc),
                                            xc.numel() // h, h, dx.data_ptr(), _stream_ptr(xc.device)))
        return dx, None


def zrmsnorm(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """ZRmsNorm over the last axis with a frozen `scale` (no gradient flows to it), one kernel each way."""
    return _ZRmsNorm.apply(x, scale)

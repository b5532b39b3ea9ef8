"""Scaled-fp8 (e4m3fn + weight_scale) weights — the compute-facing part of
crates/loractl-core/src/fp8.rs.  The reference decodes fp8 to f32 at load time
(fp8.rs:279-329); here the bytes stay fp8 in HBM and are decoded inside the kernels."""
from __future__ import annotations

import ctypes as C
import math
from typing import List

import torch

from . import _lib as L
from .quant import QuantWeight, _require_cuda, _stream_ptr


def decode_e4m3fn(byte: int) -> float:
    """crates/loractl-core/src/fp8.rs:45-56."""
    sign = -1.0 if byte & 0x80 else 1.0
    exp, man = (byte >> 3) & 0x0F, byte & 0x07
    if exp == 0x0F and man == 0x07:
        return math.nan
    if exp == 0:
        return sign * (man / 8.0) * 2.0 ** -6
    return sign * (1.0 + man / 8.0) * 2.0 ** (exp - 7)


def e4m3fn_lut() -> List[float]:
    """crates/loractl-core/src/fp8.rs:39-41: the 256-entry decode table."""
    return [decode_e4m3fn(b) for b in range(256)]


def scale_kind_for(weight_shape, scale_shape) -> int:
    """The sidecar rule of fp8.rs:59-68,109-206: `[]`/`[1]` is scalar, `[out_features]` is
    per-channel, anything else is a hard error."""
    n = 1
    for d in scale_shape:
        n *= d
    if len(scale_shape) == 0 or (len(scale_shape) == 1 and scale_shape[0] == 1):
        return L.LQ_SCALE_SCALAR
    if len(scale_shape) == 1 and scale_shape[0] == weight_shape[0]:
        return L.LQ_SCALE_PER_CHANNEL
    raise ValueError(
        f"weight_scale shape {list(scale_shape)} is neither scalar nor [out_features = {weight_shape[0]}]")


def weight_from_fp8(weight_bytes: torch.Tensor, weight_scale: torch.Tensor) -> QuantWeight:
    """Wraps a `[d_out, d_in]` uint8 / float8_e4m3fn tensor and its `weight_scale` sidecar."""
    _require_cuda(weight_bytes, "weight bytes")
    if weight_bytes.dim() != 2:
        raise ValueError("fp8 weight must be 2-D [d_out, d_in]")
    wb = weight_bytes.view(torch.uint8).contiguous()
    kind = scale_kind_for(tuple(wb.shape), tuple(weight_scale.shape))
    sc = weight_scale.detach().to(wb.device, torch.float32).reshape(-1).contiguous()
    out = C.c_void_p()
    with torch.cuda.device(wb.device):
        L.check(L.lib().lq_weight_from_fp8(wb.data_ptr(), sc.data_ptr(), kind, wb.shape[0], wb.shape[1],
                                           _stream_ptr(wb.device), C.byref(out)))
        torch.cuda.current_stream(wb.device).synchronize()
    return QuantWeight(out.value, wb.device)


def fp8_quantize(weight: torch.Tensor, per_channel: bool = False) -> QuantWeight:
    """reference/fp8_reference.py:84-94 `quantize`, on the device."""
    _require_cuda(weight, "weight")
    w = weight.detach().to(torch.float32).contiguous()
    out = C.c_void_p()
    with torch.cuda.device(w.device):
        L.check(L.lib().lq_fp8_quantize(w.data_ptr(), w.shape[0], w.shape[1], 1 if per_channel else 0,
                                        _stream_ptr(w.device), C.byref(out)))
        torch.cuda.current_stream(w.device).synchronize()
    return QuantWeight(out.value, w.device)

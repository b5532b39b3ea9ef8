"""ctypes view of the C oracle (oracle/lq_oracle.c).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(_build.build()))
        _lib.lqo_decode_e4m3fn.restype = C.c_float
        _lib.lqo_decode_e4m3fn.argtypes = [C.c_uint8]
        _lib.lqo_dequant_chunk_rows.restype = C.c_size_t
        _lib.lqo_dequant_chunk_rows.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_size_t]
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def quantize(w, group, bits):
    w = np.ascontiguousarray(w, np.float32)
    m, k = w.shape
    codes = np.empty((m, k), np.int8)
    scales = np.empty((m, k // max(group, 1)), np.float32)
    rc = lib().lqo_quantize(_p(w), C.c_int64(m), C.c_int64(k), C.c_int(group), C.c_int(bits), _p(codes), _p(scales))
    if rc != 0:
        raise ValueError("the input dim must be a multiple of the quant block")
    return codes, scales


def dequantize(codes, scales, group):
    m, k = codes.shape
    out = np.empty((m, k), np.float32)
    lib().lqo_dequantize(_p(codes), _p(scales), C.c_int64(m), C.c_int64(k), C.c_int(group), _p(out))
    return out


def dequant_chunk_rows(d_out, d_in, chunk_bytes):
    n = lib().lqo_dequant_chunk_rows(d_out, d_in, chunk_bytes, None, 0)
    rows = (C.c_uint64 * n)()
    lib().lqo_dequant_chunk_rows(d_out, d_in, chunk_bytes, rows, n)
    return [int(r) for r in rows]


def e4m3fn_lut():
    return np.array([lib().lqo_decode_e4m3fn(i) for i in range(256)], np.float32)


def fp8_dequant(b, scale):
    b = np.ascontiguousarray(b, np.uint8)
    scale = np.ascontiguousarray(scale, np.float32).reshape(-1)
    m, k = b.shape
    out = np.empty((m, k), np.float32)
    lib().lqo_fp8_dequant(_p(b), _p(scale), C.c_int64(scale.size), C.c_int64(m), C.c_int64(k), _p(out))
    return out


def lora_linear_fwd(x, codes, scales, group, a, b, s, bias=None):
    x = np.ascontiguousarray(x, np.float32)
    n, k = x.shape
    m = codes.shape[0]
    r = 0 if a is None else a.shape[1]
    y = np.empty((n, m), np.float32)
    h = np.empty((n, max(r, 1)), np.float32)
    dq = np.empty((m, k), np.float32)
    a = None if a is None else np.ascontiguousarray(a, np.float32)
    b = None if b is None else np.ascontiguousarray(b, np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().lqo_lora_linear_fwd(_p(x), C.c_int64(n), _p(codes), _p(scales), C.c_int(group), C.c_int64(m), C.c_int64(k),
                              _p(bias), _p(a), _p(b), C.c_int(r), C.c_float(s), _p(y), _p(h), _p(dq))
    return y, (h if r else None)


def lora_linear_bwd(dy, x, h, codes, scales, group, a, b, s):
    dy = np.ascontiguousarray(dy, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    n, k = x.shape
    m = codes.shape[0]
    r = 0 if a is None else a.shape[1]
    dx = np.empty((n, k), np.float32)
    da = np.empty((k, max(r, 1)), np.float32)
    db = np.empty((max(r, 1), m), np.float32)
    dh = np.empty((n, max(r, 1)), np.float32)
    dq = np.empty((m, k), np.float32)
    a = None if a is None else np.ascontiguousarray(a, np.float32)
    b = None if b is None else np.ascontiguousarray(b, np.float32)
    h = None if h is None else np.ascontiguousarray(h, np.float32)
    lib().lqo_lora_linear_bwd(_p(dy), _p(x), _p(h), C.c_int64(n), _p(codes), _p(scales), C.c_int(group), C.c_int64(m),
                              C.c_int64(k), _p(a), _p(b), C.c_int(r), C.c_float(s), _p(dx), _p(da), _p(db), _p(dh),
                              _p(dq))
    return dx, (da if r else None), (db if r else None)

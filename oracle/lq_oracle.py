"""CPU oracle for the quantized frozen-base LoRA linear (numpy restatement).

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is
compared against; nothing in the shipped package imports it.  Only `tests/`,
`__graft_entry__.smoke()` and the CPU-baseline legs of `bench.py` may use it.

Every function restates, in plain numpy f32 arithmetic, one piece of
loractl-core's path (paths are relative to the loractl repository root):

* quantize / dequantize        reference/quant_int4_reference.py:46-58,
                               reference/quant_reference.py:40-52,
                               crates/loractl-core/src/quant.rs:61-82
* dequant_chunk_rows           crates/loractl-core/src/quant.rs:102-117
* quant_matmul_t (+ backward)  crates/loractl-core/src/quant.rs:172-178,221-235
* base linear (flatten, bias)  crates/loractl-core/src/mmdit.rs:483-519
* LoRA delta forward           crates/loractl-core/src/lora.rs:199-203
* LoRA analytic gradients      reference/lora_reference.py:103-123
* e4m3fn decode                crates/loractl-core/src/fp8.rs:45-56
* fp8 scale broadcast          crates/loractl-core/src/fp8.rs:305-317
* fp8 encode (repack)          reference/fp8_reference.py:84-102
* det_vals LCG                 crates/loractl-core/tests/block_ckpt.rs:44-52
* rel_deviation / RelGate      crates/loractl-core/src/accuracy.rs:43-128

The quantize arithmetic itself lives in burn-ndarray 0.21.0 / burn-backend
0.21.0 (crates.io, pinned by the reference's Cargo.lock), which are not part
of the loractl tree; the published algorithm is: per block absmax,
scale = 2*absmax/(b-a) with (a,b)=(-qmax,qmax), q = clamp(round(w/scale)),
dq = q*scale, all in f32, `round` = Rust f32::round (half away from zero).

Pinned against: quant_int4_golden.json, quant_int8_golden.json (dq, y),
fp8_lut_golden.json (bit-for-bit), fp8_dequant_golden.json, lora_toy.json —
see tests/test_oracle_golden.py.  Parity unpinned (no reference vector exists):
exact .5 rounding ties, all-zero groups (defined here as scale=0, q=0),
G=64 groups, backward dX, dA/dB at realistic shapes, packed byte layout.
"""
from __future__ import annotations

import numpy as np

QUANT_BLOCK = 32  # crates/loractl-core/src/quant.rs:52
FP8_MAX = 448.0  # reference/fp8_reference.py:66

f32 = np.float32


def qmax_for_bits(bits: int) -> int:
    """Symmetric range max: Q4S -> 7, Q8S -> 127 (reference/quant_int4_reference.py:13-16)."""
    if bits == 4:
        return 7
    if bits == 8:
        return 127
    raise ValueError(f"unsupported quant bits {bits} (expected 4 or 8)")


def round_half_away(x: np.ndarray) -> np.ndarray:
    """Rust `f32::round`: nearest integer, ties away from zero.

    `x - trunc(x)` is exact in floating point, so no double rounding occurs
    (unlike `trunc(x + 0.5)`, which mis-rounds 0.49999997).
    """
    x = np.asarray(x, dtype=f32)
    t = np.trunc(x)
    frac = x - t
    return (t + np.where(np.abs(frac) >= f32(0.5), np.copysign(f32(1.0), x), f32(0.0))).astype(f32)


def quantize(w: np.ndarray, group: int = QUANT_BLOCK, bits: int = 4):
    """Per-(row, group) symmetric quantization of a `[d_out, d_in]` weight.

    Returns `(codes int8 [M,K], scales f32 [M,K/G])`.  Raises when
    `d_in % group != 0` (crates/loractl-core/src/quant.rs:76-80 asserts).
    An all-zero group yields scale 0 and codes 0 (a stated choice: the
    reference would compute 0/0 there and no reference test covers it).
    """
    w = np.ascontiguousarray(w, dtype=f32)
    if w.ndim != 2:
        raise ValueError("weight must be 2-D [d_out, d_in]")
    m, k = w.shape
    if group <= 0 or k % group != 0:
        raise ValueError(
            f"linear weight [{m}, {k}]: the input dim must be a multiple of the quant block ({group})"
        )
    qmax = f32(qmax_for_bits(bits))
    blocks = w.reshape(m, k // group, group)
    absmax = np.abs(blocks).max(axis=-1, keepdims=True).astype(f32)
    scale = (absmax / qmax).astype(f32)
    safe = np.where(scale > 0, scale, f32(1.0)).astype(f32)
    ratio = (blocks / safe).astype(f32)
    q = np.clip(round_half_away(ratio), -qmax, qmax)
    q = np.where(scale > 0, q, f32(0.0))
    return q.reshape(m, k).astype(np.int8), scale.reshape(m, k // group).astype(f32)


def dequantize(codes: np.ndarray, scales: np.ndarray, group: int = QUANT_BLOCK) -> np.ndarray:
    """`dq = q * scale` in f32 (burn-ndarray `dequantize_one`)."""
    m, k = codes.shape
    q = codes.astype(f32).reshape(m, k // group, group)
    return (q * scales.astype(f32)[:, :, None]).astype(f32).reshape(m, k)


def dequant_chunk_rows(d_out: int, d_in: int, chunk_bytes: int) -> list[int]:
    """Balanced row-chunk layout (crates/loractl-core/src/quant.rs:102-117)."""
    full_bytes = d_out * d_in * 4
    if chunk_bytes == 0 or full_bytes <= chunk_bytes or d_out <= 1:
        return [d_out]
    row_bytes = d_in * 4
    max_rows = max(chunk_bytes // row_bytes, 1)
    n_chunks = -(-d_out // max_rows)
    base, rem = divmod(d_out, n_chunks)
    return [base + 1 if i < rem else base for i in range(n_chunks)]


def quant_matmul_t(x: np.ndarray, dq: np.ndarray) -> np.ndarray:
    """`out[n, d_out] = x[n, d_in] . dequant(wq)[d_out, d_in]^T` (quant.rs:172-178)."""
    return (np.asarray(x, f32) @ np.asarray(dq, f32).T).astype(f32)


def lora_linear_fwd(x, dq, a=None, b=None, scaling: float = 1.0, bias=None):
    """One LoRA'd quantized site: `site()` at crates/loractl-core/src/mmdit.rs:526-536.

    x [N,K] f32, dq [M,K] f32 (dequantized frozen weight), a [K,r], b [r,M],
    bias [M].  Returns `(y [N,M], h [N,r] or None)` with
    `y = (x.dq^T + bias) + scaling * ((x.a).b)` — the reference's op order.
    """
    x = np.asarray(x, f32)
    y = quant_matmul_t(x, dq)
    if bias is not None:
        y = (y + np.asarray(bias, f32)[None, :]).astype(f32)
    h = None
    if a is not None:
        h = (x @ np.asarray(a, f32)).astype(f32)
        delta = ((h @ np.asarray(b, f32)).astype(f32) * f32(scaling)).astype(f32)
        y = (y + delta).astype(f32)
    return y, h


def lora_linear_bwd(dy, x, dq, a=None, b=None, scaling: float = 1.0):
    """Backward of `lora_linear_fwd`.

    dX through the frozen weight is `dY . dq` (quant.rs:221-235); the adapter
    gradients follow reference/lora_reference.py:103-123:
    `dB = s.H^T.dY`, `dH = s.dY.B^T`, `dA = X^T.dH`, `dX += dH.A^T`.
    Returns `(dx [N,K], da [K,r] or None, db [r,M] or None)`.
    """
    dy = np.asarray(dy, f32)
    x = np.asarray(x, f32)
    dx = (dy @ np.asarray(dq, f32)).astype(f32)
    if a is None:
        return dx, None, None
    a = np.asarray(a, f32)
    b = np.asarray(b, f32)
    s = f32(scaling)
    h = (x @ a).astype(f32)
    db = (s * (h.T @ dy)).astype(f32)
    dh = (s * (dy @ b.T)).astype(f32)
    da = (x.T @ dh).astype(f32)
    dx = (dx + dh @ a.T).astype(f32)
    return dx, da, db


# ----------------------------------------------------------------------------
# fp8 e4m3fn
# ----------------------------------------------------------------------------
def decode_e4m3fn(byte: int) -> float:
    """One e4m3fn byte -> f32 (crates/loractl-core/src/fp8.rs:45-56)."""
    sign = -1.0 if byte & 0x80 else 1.0
    exp = (byte >> 3) & 0x0F
    man = byte & 0x07
    if exp == 0x0F and man == 0x07:
        return float("nan")
    if exp == 0:
        return sign * (man / 8.0) * 2.0 ** -6
    return sign * (1.0 + man / 8.0) * 2.0 ** (exp - 7)


def e4m3fn_lut() -> np.ndarray:
    """The 256-entry decode table (crates/loractl-core/src/fp8.rs:39-41)."""
    return np.array([decode_e4m3fn(i) for i in range(256)], dtype=f32)


def encode_e4m3fn(x: np.ndarray) -> np.ndarray:
    """f32 -> e4m3fn byte, round-to-nearest-even, NaN on overflow (no inf).

    Restates torch's `tensor.to(torch.float8_e4m3fn)` as used by
    reference/fp8_reference.py:84-94.  |x| that rounds above 448 becomes
    NaN (0x7f | sign), like torch (the format has no infinity).
    """
    x = np.asarray(x, dtype=f32)
    lut = e4m3fn_lut()
    pos = lut[:0x7F].astype(np.float64)  # 0 .. 448, monotonically increasing
    ax = np.abs(x).astype(np.float64)
    idx = np.searchsorted(pos, ax, side="left")  # first pos >= ax
    idx = np.clip(idx, 1, len(pos) - 1)
    lo, hi = pos[idx - 1], pos[idx]
    dlo, dhi = ax - lo, hi - ax
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((idx % 2) == 0))  # ties -> even mantissa
    code = np.where(pick_hi, idx, idx - 1).astype(np.int64)
    code = np.where(ax > 464.0, 0x7F, code)  # past the tie with the (absent) 480: out of range
    code = np.where(np.isnan(x), 0x7F, code)
    sign = np.signbit(x).astype(np.int64) << 7
    return (code | sign).astype(np.uint8)


def fp8_quantize(w: np.ndarray, per_channel: bool = False):
    """Scaled-fp8 repack of one weight (reference/fp8_reference.py:84-94).

    `scale = amax/448` clamped to >= 1e-12, 0-d or per output row.
    Returns `(bytes uint8 [M,K], scale f32 [] or [M])`.
    """
    w = np.asarray(w, dtype=f32)
    if per_channel:
        scale = np.maximum((np.abs(w).max(axis=1) / f32(FP8_MAX)).astype(f32), f32(1e-12))
        q = encode_e4m3fn((w / scale[:, None]).astype(f32))
    else:
        scale = np.maximum((np.abs(w).max() / f32(FP8_MAX)).astype(f32), f32(1e-12))
        q = encode_e4m3fn((w / scale).astype(f32))
    return q, np.asarray(scale, dtype=f32)


def fp8_dequant(weight_bytes: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """`LUT[byte] * scale`; scalar (`[]`/`[1]`) or per-out-channel `scale[i // row_len]`
    over a row-major `[M, K]` byte matrix (crates/loractl-core/src/fp8.rs:305-317)."""
    wb = np.asarray(weight_bytes, dtype=np.uint8)
    scale = np.asarray(scale, dtype=f32)
    vals = e4m3fn_lut()[wb]
    if scale.size == 1:
        return (vals * scale.reshape(())).astype(f32)
    if wb.ndim != 2 or scale.shape != (wb.shape[0],):
        raise ValueError(f"weight_scale shape {scale.shape} is neither scalar nor [out_features]")
    return (vals * scale[:, None]).astype(f32)


# ----------------------------------------------------------------------------
# helpers shared with the reference's tests
# ----------------------------------------------------------------------------
def det_vals(n: int, seed: int) -> np.ndarray:
    """LCG in [-1, 1) (crates/loractl-core/tests/block_ckpt.rs:44-52)."""
    out = np.empty(n, dtype=f32)
    state = seed & 0xFFFFFFFF
    for i in range(n):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = f32(f32(state >> 8) / f32(1 << 24) * f32(2.0) - f32(1.0))
    return out


def rel_deviation(ours: np.ndarray, reference: np.ndarray) -> float:
    """Peak-normalised max deviation (crates/loractl-core/src/accuracy.rs:96-115)."""
    ours = np.asarray(ours, dtype=f32).ravel()
    reference = np.asarray(reference, dtype=f32).ravel()
    if ours.size == 0 or ours.size != reference.size:
        return float("inf")
    if not (np.isfinite(ours).all() and np.isfinite(reference).all()):
        return float("inf")
    peak = float(np.abs(reference).max())
    return float(np.abs(ours - reference).max()) / max(peak, 1e-12)


def rel_gate(d_ours: float, d_bar: float, floor: float, ceil: float) -> bool:
    """`finite and d <= max(2*d_bar, floor) and d <= ceil` (accuracy.rs:84-93)."""
    return bool(np.isfinite(d_ours) and d_ours <= max(2.0 * d_bar, floor) and d_ours <= ceil)


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    """f64 cosine similarity (crates/loractl-core/tests/common/mod.rs:47-52)."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))

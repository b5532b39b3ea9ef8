"""Frozen-base quantization core — the host-side mirror of crates/loractl-core/src/quant.rs.

Same names and argument meaning as the reference: `QUANT_BLOCK`, `Quant`,
`quant_value`, `quantize_linear_weight`, `quantize_linear_weight_chunked`,
`dequant_chunk_rows`, `quant_matmul_t`.  The burn `QFloat` tensor becomes a
`QuantWeight`: an owning handle on the packed device storage of
libloractl_b200.  All compute runs in the CUDA library; nothing here has a
CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import List, Optional

import torch

from . import _lib as L

QUANT_BLOCK = 32  # crates/loractl-core/src/quant.rs:52


class Quant(enum.Enum):
    """crates/loractl-core/src/config.rs:637-649; spellings of `FromStr` at :655-664."""

    NONE = "none"
    INT8 = "int8"
    INT4 = "int4"

    @staticmethod
    def parse(s: str) -> "Quant":
        k = s.lower()
        if k in ("none", "off", "f32"):
            return Quant.NONE
        if k in ("int8", "i8"):
            return Quant.INT8
        if k in ("int4", "i4"):
            return Quant.INT4
        raise ValueError(f"unknown quant {s!r} (none|int8|int4)")


def quant_value(q: Quant) -> Optional[int]:
    """crates/loractl-core/src/quant.rs:156-162: None -> no quantization, Int8 -> Q8S (8 bits),
    Int4 -> Q4S (4 bits)."""
    return {Quant.NONE: None, Quant.INT8: 8, Quant.INT4: 4}[q]


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return L.LQ_F32
    if t.dtype == torch.bfloat16:
        return L.LQ_BF16
    raise TypeError(f"unsupported activation dtype {t.dtype}: the b200 backend computes in f32 or bf16")


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must live on a CUDA device: the b200 backend has no CPU path")


class QuantWeight:
    """Owning handle of one frozen quantized `[d_out, d_in]` weight (file layout,
    crates/loractl-core/src/mmdit.rs:404-412).  Stands where the reference holds a burn
    `QFloat` tensor; immutable, never receives a gradient."""

    def __init__(self, handle: int, device: torch.device):
        self._h = C.c_void_p(handle)
        self.device = device
        info = L.WeightInfo()
        L.check(L.lib().lq_weight_info_get(self._h, C.byref(info)))
        self.d_out, self.d_in = int(info.d_out), int(info.d_in)
        self.scheme, self.group, self.scale_kind = int(info.scheme), int(info.group), int(info.scale_kind)
        self.packed_bytes, self.scale_bytes = int(info.packed_bytes), int(info.scale_bytes)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                L.lib().lq_weight_destroy(h)
            except Exception:
                pass

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    @property
    def shape(self):
        return (self.d_out, self.d_in)

    def dims(self):
        return [self.d_out, self.d_in]

    @property
    def bits(self) -> int:
        return {L.LQ_INT4: 4, L.LQ_INT8: 8, L.LQ_FP8_E4M3: 8}[self.scheme]

    def set_bias(self, bias: Optional[torch.Tensor]) -> None:
        with torch.cuda.device(self.device):
            if bias is None:
                L.check(L.lib().lq_weight_set_bias(self._h, None, _stream_ptr(self.device)))
                return
            b = bias.detach().to(self.device, torch.float32).contiguous()
            if b.numel() != self.d_out:
                raise ValueError(f"bias has {b.numel()} elements, expected d_out = {self.d_out}")
            L.check(L.lib().lq_weight_set_bias(self._h, b.data_ptr(), _stream_ptr(self.device)))
            torch.cuda.current_stream(self.device).synchronize()  # b may be a temporary

    def attach_bf16_copy(self, buffer: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Keeps a resident bf16 `[d_out, d_in]` copy of the dequantised weight (`lq_weight_attach_bf16_copy`):
        bf16 calls at >= 65 tokens then run no dequantisation pass.  `buffer` (bf16, `d_out * d_in`
        elements) may be supplied to reuse memory, e.g. one block's worth under block checkpointing."""
        n = self.d_out * self.d_in
        if buffer is None:
            buffer = torch.empty(n, dtype=torch.bfloat16, device=self.device)
        if buffer.dtype != torch.bfloat16 or buffer.numel() < n or not buffer.is_contiguous():
            raise ValueError("bf16 copy buffer must be a contiguous bf16 tensor of at least d_out * d_in elements")
        with torch.cuda.device(self.device):
            L.check(L.lib().lq_weight_attach_bf16_copy(self._h, buffer.data_ptr(), _stream_ptr(self.device)))
        self._bf16_copy = buffer  # keeps the memory alive while attached
        return buffer

    def detach_bf16_copy(self) -> None:
        L.check(L.lib().lq_weight_attach_bf16_copy(self._h, None, None))
        self._bf16_copy = None

    def prepare_fp8_backward(self) -> None:
        """Builds the transposed e4m3 copy the native-fp8 backward reads, at load time, so the
        step loop stays allocation-free (otherwise the first such backward builds it)."""
        with torch.cuda.device(self.device):
            L.check(L.lib().lq_weight_prepare_fp8_backward(self._h, _stream_ptr(self.device)))

    def unpack(self):
        """Logical content: (codes int8 [M,K], scales f32 [M,K/G]); for fp8, (bytes uint8 [M,K],
        scale f32 [1] or [M]).  Lets tests check bit-exactness independent of the tile layout."""
        with torch.cuda.device(self.device):
            codes = torch.empty((self.d_out, self.d_in), dtype=torch.int8, device=self.device)
            if self.scheme == L.LQ_FP8_E4M3:
                ns = self.d_out if self.scale_kind == L.LQ_SCALE_PER_CHANNEL else 1
                scales = torch.empty((ns,), dtype=torch.float32, device=self.device)
            else:
                scales = torch.empty((self.d_out, self.d_in // self.group), dtype=torch.float32, device=self.device)
            L.check(L.lib().lq_unpack(self._h, codes.data_ptr(), scales.data_ptr(), _stream_ptr(self.device)))
        if self.scheme == L.LQ_FP8_E4M3:
            codes = codes.view(torch.uint8)
        return codes, scales

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """burn `dequantize` / `QuantLinear::dequantized_weight` (mmdit.rs:435-444): full [M,K]."""
        out = torch.empty((self.d_out, self.d_in), dtype=dtype, device=self.device)
        with torch.cuda.device(self.device):
            L.check(L.lib().lq_dequantize(self._h, out.data_ptr(), _dtype_code(out), _stream_ptr(self.device)))
        return out


def quantize_linear_weight(weight: torch.Tensor, value: int, block: int = QUANT_BLOCK) -> QuantWeight:
    """crates/loractl-core/src/quant.rs:74-82.  `weight` is `[d_out, d_in]` (f32 or bf16, CUDA);
    `value` is 8 (Q8S) or 4 (Q4S).  Raises when `d_in % block != 0` (the reference panics)."""
    _require_cuda(weight, "weight")
    if weight.dim() != 2:
        raise ValueError("weight must be 2-D [d_out, d_in]")
    w = weight.detach().contiguous()
    out = C.c_void_p()
    with torch.cuda.device(w.device):
        L.check(L.lib().lq_quantize(w.data_ptr(), _dtype_code(w), w.shape[0], w.shape[1], block, value,
                                    _stream_ptr(w.device), C.byref(out)))
        torch.cuda.current_stream(w.device).synchronize()  # `w` may be a temporary copy
    return QuantWeight(out.value, w.device)


def dequant_chunk_rows(d_out: int, d_in: int, chunk_bytes: int) -> List[int]:
    """crates/loractl-core/src/quant.rs:102-117 (pure host function, evaluated in the library)."""
    n = C.c_size_t()
    L.check(L.lib().lq_dequant_chunk_rows(d_out, d_in, chunk_bytes, None, 0, C.byref(n)))
    rows = (C.c_uint64 * n.value)()
    L.check(L.lib().lq_dequant_chunk_rows(d_out, d_in, chunk_bytes, rows, n.value, C.byref(n)))
    return [int(r) for r in rows]


def quantize_linear_weight_chunked(weight: torch.Tensor, value: int, chunk_bytes: int,
                                   block: int = QUANT_BLOCK) -> List[QuantWeight]:
    """crates/loractl-core/src/quant.rs:130-150: one quantized weight per row chunk, in d_out
    order; blocks live within rows, so each chunk is bit-identical to the same rows of the
    whole-tensor quantization."""
    rows = dequant_chunk_rows(weight.shape[0], weight.shape[1], chunk_bytes)
    if len(rows) == 1:
        return [quantize_linear_weight(weight, value, block)]
    out, start = [], 0
    for r in rows:
        out.append(quantize_linear_weight(weight[start:start + r], value, block))
        start += r
    return out


def weight_from_codes(codes: torch.Tensor, scales: torch.Tensor, block: int, bits: int) -> QuantWeight:
    """Builds a weight from logical (codes int8 [M,K], scales f32 [M,K/block])."""
    _require_cuda(codes, "codes")
    c = codes.contiguous()
    s = scales.to(torch.float32).contiguous()
    out = C.c_void_p()
    with torch.cuda.device(c.device):
        L.check(L.lib().lq_weight_from_codes(c.data_ptr(), s.data_ptr(), c.shape[0], c.shape[1], block, bits,
                                             _stream_ptr(c.device), C.byref(out)))
        torch.cuda.current_stream(c.device).synchronize()
    return QuantWeight(out.value, c.device)


def concat_chunks(chunks: List[QuantWeight]) -> QuantWeight:
    """Joins row chunks (which concatenate along d_out in order, mmdit.rs:417-424) into one
    packed weight: the kernels treat chunks as row ranges of a single buffer, so no
    per-chunk matmul and no `cat` of outputs is needed."""
    if len(chunks) == 1:
        return chunks[0]
    parts = [c.unpack() for c in chunks]
    codes = torch.cat([p[0] for p in parts], 0)
    scales = torch.cat([p[1] for p in parts], 0)
    return weight_from_codes(codes, scales, chunks[0].group, chunks[0].bits)


# ---- workspace -------------------------------------------------------------------------

_workspaces: dict = {}


def workspace_for(wq: QuantWeight, n_tokens: int, rank: int, dtype_code: int) -> torch.Tensor:
    """Caller-owned scratch for the hot-path calls, cached per (device, stream) and grown on
    demand, so the step loop performs no allocation once warm."""
    need = int(L.lib().lq_linear_workspace_bytes(wq.handle, n_tokens, rank, dtype_code))
    key = (wq.device.index, torch.cuda.current_stream(wq.device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need + 256, dtype=torch.uint8, device=wq.device)
        _workspaces[key] = ws
    return ws


def _aligned(ws: torch.Tensor):
    off = (-ws.data_ptr()) % 256
    return ws.data_ptr() + off, ws.numel() - off


def _compute_code(t: torch.Tensor, fp8_compute: bool) -> int:
    """dtype code of one call: the tensor's element type, or LQ_BF16_W8A8 when native fp8 compute
    is requested (bf16 activations, scaled-fp8 weight)."""
    dt = _dtype_code(t)
    if fp8_compute:
        if dt != L.LQ_BF16:
            raise TypeError("native fp8 compute takes bf16 activations")
        return L.LQ_BF16_W8A8
    return dt


def lora_mirror(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 operand mirror of one site's factors (`lq_lora_mirror_update`): `a` is `[d_in, r]`, `b` is
    `[r, d_out]`, both f32 on the device.  Returns the (256-byte aligned) byte buffer to pass as
    `mirror=` to `linear_fwd_raw` / `linear_bwd_raw`; pass `out` to refresh an existing one in place."""
    _require_cuda(a, "lora_a")
    d_in, r = a.shape
    d_out = b.shape[1]
    need = int(L.lib().lq_lora_mirror_bytes(d_in, d_out, r))
    if out is None:
        raw = torch.empty(need + 256, dtype=torch.uint8, device=a.device)
        off = (-raw.data_ptr()) % 256
        out = raw[off:off + need]
    with torch.cuda.device(a.device):
        L.check(L.lib().lq_lora_mirror_update(a.data_ptr(), b.data_ptr(), d_in, d_out, r, out.data_ptr(),
                                              _stream_ptr(a.device)))
    return out


def lora_mirror_alloc(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """An uninitialised, 256-byte aligned mirror buffer for factors of these shapes."""
    d_in, r = a.shape
    need = int(L.lib().lq_lora_mirror_bytes(d_in, b.shape[1], r))
    raw = torch.empty(need + 256, dtype=torch.uint8, device=a.device)
    off = (-raw.data_ptr()) % 256
    return raw[off:off + need]


def lora_mirror_batch(jobs) -> None:
    """Refreshes many mirrors with one launch per 24 sites (`lq_lora_mirror_update_batch`).  `jobs` is a
    sequence of (a [d_in, r], b [r, d_out], mirror buffer) on one device."""
    jobs = list(jobs)
    if not jobs:
        return
    import ctypes as C

    arr = (L.MirrorJob * len(jobs))()
    for i, (a, b, m) in enumerate(jobs):
        _require_cuda(a, "lora_a")
        arr[i] = L.MirrorJob(a.data_ptr(), b.data_ptr(), a.shape[0], b.shape[1], a.shape[1], m.data_ptr())
    dev = jobs[0][0].device
    with torch.cuda.device(dev):
        L.check(L.lib().lq_lora_mirror_update_batch(C.cast(arr, C.c_void_p), len(jobs), _stream_ptr(dev)))


def linear_fwd_raw(wq: QuantWeight, x2: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor],
                   scaling: float, want_h: bool = True, fp8_compute: bool = False,
                   mirror: Optional[torch.Tensor] = None):
    """Direct call of `lq_linear_fwd` on a flattened `[N, K]` activation.  Returns (y, h).
    `fp8_compute` selects LQ_BF16_W8A8 (tcgen05 e4m3 x e4m3; scaled-fp8 weights only)."""
    _require_cuda(x2, "x")
    n = x2.shape[0]
    rank = 0 if a is None else a.shape[1]
    dt = _compute_code(x2, fp8_compute)
    y = torch.empty((n, wq.d_out), dtype=x2.dtype, device=x2.device)
    h = torch.empty((n, rank), dtype=torch.float32, device=x2.device) if (rank and want_h) else None
    with torch.cuda.device(x2.device):
        ws = workspace_for(wq, n, rank, dt)
        wp, wn = _aligned(ws)
        L.check(L.lib().lq_linear_fwd(
            wq.handle, x2.data_ptr(), n, dt,
            a.data_ptr() if rank else None, b.data_ptr() if rank else None, rank, float(scaling),
            y.data_ptr(), h.data_ptr() if h is not None else None, wp, wn, _stream_ptr(x2.device),
            mirror.data_ptr() if (mirror is not None and rank) else None))
    return y, h


def linear_fwd_grouped_raw(sites, x2: torch.Tensor, want_h: bool = True):
    """`lq_linear_fwd_grouped`: several sites that read the same flattened activation `x2`.
    `sites` is a list of `(wq, a, b, scaling)` (a, b None for a base-only site).  Returns a list of
    `(y, h)`.  At <= 16 bf16 tokens with int4 weights of one width the group is one launch pair."""
    _require_cuda(x2, "x")
    n = x2.shape[0]
    dt = _dtype_code(x2)
    arr = (L.GroupSite * len(sites))()
    outs, keep = [], []
    for i, (wq, a, b, scaling) in enumerate(sites):
        rank = 0 if a is None else a.shape[1]
        y = torch.empty((n, wq.d_out), dtype=x2.dtype, device=x2.device)
        h = torch.empty((n, rank), dtype=torch.float32, device=x2.device) if (rank and want_h) else None
        arr[i].w = wq.handle
        arr[i].A = a.data_ptr() if rank else None
        arr[i].B = b.data_ptr() if rank else None
        arr[i].rank = rank
        arr[i].scaling = float(scaling)
        arr[i].Y = y.data_ptr()
        arr[i].H_out = h.data_ptr() if h is not None else None
        outs.append((y, h))
        keep.append((a, b))
    with torch.cuda.device(x2.device):
        need = int(L.lib().lq_linear_grouped_workspace_bytes(arr, len(sites), n, dt))
        key = (x2.device.index, torch.cuda.current_stream(x2.device).cuda_stream)
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < need + 256:
            ws = torch.empty(need + 512, dtype=torch.uint8, device=x2.device)
            _workspaces[key] = ws
        wp, wn = _aligned(ws)
        L.check(L.lib().lq_linear_fwd_grouped(arr, len(sites), x2.data_ptr(), n, dt, wp, wn, _stream_ptr(x2.device)))
    return outs


def linear_bwd_raw(wq: QuantWeight, dy2: torch.Tensor, x2: Optional[torch.Tensor], h: Optional[torch.Tensor],
                   a: Optional[torch.Tensor], b: Optional[torch.Tensor], scaling: float,
                   need_dx: bool = True, need_da: bool = True, need_db: bool = True,
                   da_out: Optional[torch.Tensor] = None, db_out: Optional[torch.Tensor] = None,
                   accumulate: bool = False, fp8_compute: bool = False, mirror: Optional[torch.Tensor] = None):
    """Direct call of `lq_linear_bwd`.  Returns (dx, da, db).  `da_out`/`db_out` let the caller
    point the gradients into a flat bucket (with `accumulate` to add instead of overwrite)."""
    n = dy2.shape[0]
    rank = 0 if a is None else a.shape[1]
    dt = _compute_code(dy2, fp8_compute)
    dev = dy2.device
    dx = torch.empty((n, wq.d_in), dtype=dy2.dtype, device=dev) if need_dx else None
    da = db = None
    if rank:
        if need_da:
            da = da_out if da_out is not None else torch.empty((wq.d_in, rank), dtype=torch.float32, device=dev)
        if need_db:
            db = db_out if db_out is not None else torch.empty((rank, wq.d_out), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        ws = workspace_for(wq, n, rank, dt)
        wp, wn = _aligned(ws)
        L.check(L.lib().lq_linear_bwd(
            wq.handle, dy2.data_ptr(), x2.data_ptr() if x2 is not None else None,
            h.data_ptr() if h is not None else None, n, dt,
            a.data_ptr() if rank else None, b.data_ptr() if rank else None, rank, float(scaling),
            dx.data_ptr() if dx is not None else None, da.data_ptr() if da is not None else None,
            db.data_ptr() if db is not None else None, 1 if accumulate else 0, wp, wn, _stream_ptr(dev),
            mirror.data_ptr() if (mirror is not None and rank) else None))
    return dx, da, db


class _QuantMatmulT(torch.autograd.Function):
    """The custom op of crates/loractl-core/src/quant.rs:210-262: forward `x . dequant(wq)^T`,
    backward `grad_x = grad_out . dequant(wq)`; the weight is state, never a graph parent."""

    @staticmethod
    def forward(ctx, x2, wq):
        ctx.wq = wq
        y, _ = linear_fwd_raw(wq, x2, None, None, 1.0)
        return y

    @staticmethod
    def backward(ctx, dy):
        dx, _, _ = linear_bwd_raw(ctx.wq, dy.contiguous(), None, None, None, None, 1.0)
        return dx, None


def quant_matmul_t(x: torch.Tensor, wq: QuantWeight) -> torch.Tensor:
    """`QuantBackend::quant_matmul_t` (crates/loractl-core/src/quant.rs:172-178):
    `out[n, d_out] = x[n, d_in] . dequant(wq[d_out, d_in])^T`; no gradient flows to `wq`.
    (The handle's bias, if any, is added: attach none for the bare op.)"""
    if not isinstance(wq, QuantWeight):
        raise TypeError("quant_matmul_t requires a quantized weight — see quantize_linear_weight")
    if x.dim() != 2 or x.shape[1] != wq.d_in:
        raise ValueError(f"x must be [n, {wq.d_in}], got {list(x.shape)}")
    return _QuantMatmulT.apply(x.contiguous(), wq)


def check_device_status(device: Optional[torch.device] = None) -> None:
    """Synchronises the current stream and raises if a kernel's bounded wait gave up."""
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(dev):
        L.check(L.lib().lq_check_device_status(_stream_ptr(dev)))

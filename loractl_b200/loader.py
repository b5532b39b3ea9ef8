"""Streaming quantize-at-load: a `.safetensors` checkpoint (f32 / bf16 / f16 or scaled fp8) becomes
packed int4/int8 (or resident fp8) weight handles on the device, one tensor at a time.

Mirrors `load_quant_module` (crates/loractl-core/src/diffusion_trainer.rs:1094-1267) and the
checkpoint classification of `load_fp8_snapshots` / `load_plain_snapshots`
(crates/loractl-core/src/fp8.rs:109-362).  Where the reference forces ONE transient f32
`[d_out, d_in]` per site on the host (fp8 decoded by a single CPU thread), quantizes it and drops
it, this loader never leaves the checkpoint's own element type on the host side:

    mmap'd file -> pinned staging buffer -> (copy stream) device staging -> one quantize kernel

with two staging slots, so the host copy of tensor i+1, the upload of tensor i and the kernel of
tensor i-1 overlap.  A scaled-fp8 tensor is requantized by one fused kernel
(`lq_quantize_from_fp8`: LUT decode x weight_scale -> group absmax -> codes), bit-identical to
decoding to f32 first.

The `.safetensors` container is parsed here (8-byte little-endian header length, JSON header,
raw little-endian tensor data); `write_safetensors` exists for tests and the load benchmark.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from concurrent.futures import ThreadPoolExecutor
import mmap
import struct
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

from . import _lib as L
from .fp8 import scale_kind_for
from .quant import QuantWeight, _stream_ptr

# safetensors dtype tag -> bytes per element
_DTYPE_BYTES = {"F32": 4, "BF16": 2, "F16": 2, "F8_E4M3": 1}
_TORCH_DTYPE = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16}


class CheckpointError(ValueError):
    """A malformed or unsupported checkpoint; the message names the key and the file."""


@dataclass
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int  # byte offsets inside the data section
    end: int


class SafetensorsFile:
    """Read-only, mmap-backed view of one `.safetensors` file."""

    def __init__(self, path: str):
        self.path = str(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 8:
            raise CheckpointError(f"{self.path}: too short to hold a safetensors header")
        (n,) = struct.unpack("<Q", self._mm[:8])
        if 8 + n > len(self._mm):
            raise CheckpointError(f"{self.path}: header length {n} exceeds the file")
        try:
            header = json.loads(self._mm[8:8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError(f"parsing safetensors header of {self.path}: {e}") from e
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self._data0 = 8 + n
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            b, e = info["data_offsets"]
            shape = tuple(int(d) for d in info["shape"])
            ent = TensorEntry(name, info["dtype"], shape, int(b), int(e))
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPE_BYTES.get(ent.dtype, 0) if ent.dtype in _DTYPE_BYTES else None
            if e < b or self._data0 + e > len(self._mm) or (want is not None and want != e - b):
                raise CheckpointError(f"'{name}' has inconsistent data offsets [{b}, {e}) in {self.path}")
            self.entries[name] = ent

    def fileno(self) -> int:
        return self._f.fileno()

    def file_offset(self, name: str) -> int:
        return self._data0 + self.entries[name].begin

    def raw(self, name: str) -> memoryview:
        ent = self.entries[name]
        return memoryview(self._mm)[self._data0 + ent.begin:self._data0 + ent.end]

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass  # a numpy view is still alive; the mapping goes with it
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Dict[str, Tuple[str, Tuple[int, ...], bytes]],
                      metadata: Optional[Dict[str, str]] = None) -> None:
    """Writes `{name: (dtype tag, shape, little-endian bytes)}` in the safetensors layout
    (names sorted, data contiguous, header padded with spaces to a multiple of 8 bytes)."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    for name in sorted(tensors):
        dtype, shape, data = tensors[name]
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + len(data)]}
        off += len(data)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in sorted(tensors):
            f.write(tensors[name][2])


@dataclass
class PlanItem:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    scale_name: Optional[str]  # fp8 only: the '<name>_scale' sidecar
    scale_kind: Optional[int]


def classify(sf: SafetensorsFile) -> List[PlanItem]:
    """Pass 1 of fp8.rs:119-206, from the header alone: rejects the legacy scaled-fp8 format,
    fp8 tensors without an F32 `<name>_scale` sidecar, sidecars of the wrong shape, orphan
    sidecars and unsupported dtypes; drops `.comfy_quant` / `.input_scale` metadata tensors.
    Returns the model tensors (sidecars consumed) in file order."""
    ents = sf.entries
    for name in ents:
        if name == "scaled_fp8" or name.endswith(".scale_weight"):
            raise CheckpointError(
                f"scaled-fp8 checkpoint {sf.path} uses the legacy ComfyUI 'scaled fp8' quant format "
                f"('scaled_fp8' marker / '.scale_weight' keys, found '{name}'): not supported — re-export "
                f"with per-tensor '<name>.weight_scale' sidecars")
    skip = set()
    kinds: Dict[str, int] = {}
    for name, e in ents.items():
        if e.dtype != "F8_E4M3":
            continue
        sname = f"{name}_scale"
        s = ents.get(sname)
        if s is None:
            raise CheckpointError(f"fp8 tensor '{name}' has no '{sname}' sidecar in {sf.path}")
        if s.dtype != "F32":
            raise CheckpointError(f"'{sname}' dtype {s.dtype} — expected F32 (in {sf.path})")
        if len(s.shape) == 1 and s.shape[0] == 0:
            raise CheckpointError(f"'{sname}' is empty ([0]) for weight '{name}' {list(e.shape)} in {sf.path}")
        try:
            kinds[name] = scale_kind_for(e.shape if e.shape else (0,), s.shape)
        except ValueError:
            out = e.shape[0] if e.shape else 0
            raise CheckpointError(
                f"'{sname}' shape {list(s.shape)} is neither scalar ([]/[1]) nor per-output-channel ([{out}]) "
                f"for weight '{name}' {list(e.shape)} in {sf.path}") from None
        skip.add(sname)
    plan: List[PlanItem] = []
    for name, e in ents.items():
        if name in skip:
            continue
        if e.dtype == "F8_E4M3":
            plan.append(PlanItem(name, e.dtype, e.shape, f"{name}_scale", kinds[name]))
            continue
        if name.endswith(".weight_scale"):
            raise CheckpointError(f"'{name}' has no fp8 base weight '{name[:-len('_scale')]}' in {sf.path}")
        if name.endswith(".comfy_quant") or name.endswith(".input_scale"):
            continue
        if e.dtype not in _TORCH_DTYPE:
            raise CheckpointError(f"'{name}' has unsupported dtype {e.dtype} in {sf.path}")
        plan.append(PlanItem(name, e.dtype, e.shape, None, None))
    return plan


def is_fp8_checkpoint(sf: SafetensorsFile) -> bool:
    """crates/loractl-core/src/fp8.rs:76-98: any F8_E4M3 tensor in the header."""
    return any(e.dtype == "F8_E4M3" for e in sf.entries.values())


@dataclass
class LoadReport:
    quantized: int = 0
    kept_fp8: int = 0
    left_plain: int = 0
    file_bytes: int = 0        # bytes of tensor data read from the checkpoint
    packed_bytes: int = 0      # bytes of packed weights + scales now resident


_COPY_THREADS = 8


def _host_read(fd: int, dst: np.ndarray, offset: int, pool: ThreadPoolExecutor) -> None:
    """Reads one tensor's bytes from the file straight into pinned memory with positional reads,
    split over a few threads for large tensors (the read releases the GIL).  Reading, unlike copying
    out of a fresh mapping, takes no page fault per 4 KB of checkpoint."""
    n = dst.shape[0]

    def read(o: int, m: int) -> None:
        done = 0
        while done < m:
            got = os.preadv(fd, [memoryview(dst[o + done:o + m])], offset + o + done)
            if got <= 0:
                raise CheckpointError("unexpected end of checkpoint file")
            done += got

    if n < (8 << 20):
        read(0, n)
        return
    step = ((-(-n // _COPY_THREADS)) + 4095) & ~4095
    futs = [pool.submit(read, o, min(step, n - o)) for o in range(0, n, step)]
    for f in futs:
        f.result()


class _Slot:
    def __init__(self, nbytes: int, device: torch.device):
        self.host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        self.dev = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.uploaded = torch.cuda.Event()
        self.consumed = torch.cuda.Event()
        self.used = False


_STAGING: Dict[torch.device, List[_Slot]] = {}


def _staging(device: torch.device, nbytes: int) -> List[_Slot]:
    """The two staging slots of a device, kept between calls (pinning host memory costs more than
    uploading through it) and grown when a checkpoint holds a larger tensor."""
    cur = _STAGING.get(device)
    if cur is None or cur[0].host.numel() < nbytes:
        cur = [_Slot(nbytes, device), _Slot(nbytes, device)]
        _STAGING[device] = cur
    for sl in cur:
        sl.used = False
    return cur


def release_staging() -> None:
    """Frees the pinned and device staging buffers kept by `load_quant_module`."""
    _STAGING.clear()


def load_quant_module(path: str, device: torch.device, bits: int = 4, block: int = 64,
                      want: Optional[Callable[[str, Tuple[int, ...]], bool]] = None,
                      keep_fp8: bool = False, progress: Optional[Callable[[str, int, int], None]] = None):
    """Loads every 2-D `*.weight` of the checkpoint whose `d_in` is a multiple of `block` as a
    quantized handle (`bits` 4 or 8), one tensor at a time; everything else — 1-D tensors, weights
    with an unaligned `d_in` (the reference leaves those sites `Plain`, mmdit.rs:1134-1158), or
    names `want(name, shape)` rejects — comes back as a plain f32 device tensor.

    `keep_fp8=True` keeps scaled-fp8 weights as resident fp8 handles (`lq_weight_from_fp8`) instead
    of requantizing them.  Returns `(handles: {name: QuantWeight}, plain: {name: Tensor}, LoadReport)`.
    """
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    lib = L.lib()
    handles: Dict[str, QuantWeight] = {}
    plain: Dict[str, torch.Tensor] = {}
    rep = LoadReport()
    with SafetensorsFile(path) as sf, torch.cuda.device(device):
        plan = classify(sf)
        def slot_bytes(p: PlanItem) -> int:
            e = sf.entries[p.name]
            extra = 0
            if p.scale_name:  # the sidecar rides in the same slot, after the weight bytes
                se = sf.entries[p.scale_name]
                extra = 256 + (se.end - se.begin)
            return ((e.end - e.begin + 255) & ~255) + extra

        nmax = max((slot_bytes(p) for p in plan), default=0)
        if nmax == 0:
            return handles, plain, rep
        slots = _staging(device, nmax)
        pool = ThreadPoolExecutor(max_workers=_COPY_THREADS)
        copy_stream = torch.cuda.Stream(device)
        main = torch.cuda.current_stream(device)
        sp = _stream_ptr(device)
        for i, item in enumerate(plan):
            if progress:
                progress(item.name, i, len(plan))
            ent = sf.entries[item.name]
            n = ent.end - ent.begin
            slot = slots[i & 1]
            if slot.used:
                slot.consumed.synchronize()  # the kernel that read this slot's device buffer is done
            # host: checkpoint bytes -> pinned staging (the only host-side touch of the data); the
            # fp8 sidecar follows the weight in the same slot so that one upload carries both
            hostv = slot.host.numpy()
            _host_read(sf.fileno(), hostv[:n], sf.file_offset(item.name), pool)
            total, s_off, s_n = n, 0, 0
            if item.scale_name:
                se = sf.entries[item.scale_name]
                s_off, s_n = (n + 255) & ~255, se.end - se.begin
                _host_read(sf.fileno(), hostv[s_off:s_off + s_n], sf.file_offset(item.scale_name), pool)
                total = s_off + s_n
            with torch.cuda.stream(copy_stream):
                slot.dev[:total].copy_(slot.host[:total], non_blocking=True)
                slot.uploaded.record(copy_stream)
            main.wait_event(slot.uploaded)
            slot.used = True
            rep.file_bytes += n
            quantizable = (len(item.shape) == 2 and item.name.endswith(".weight") and item.shape[1] % block == 0
                           and item.shape[1] > 0 and (want is None or want(item.name, item.shape)))
            src = slot.dev[:n]
            if item.dtype == "F8_E4M3":
                sc = slot.dev[s_off:s_off + s_n].view(torch.float32)
                rep.file_bytes += s_n
                if len(item.shape) != 2:
                    raise CheckpointError(f"fp8 tensor '{item.name}' is not 2-D in {sf.path}")
                out = C.c_void_p()
                if quantizable and not keep_fp8:
                    L.check(lib.lq_quantize_from_fp8(src.data_ptr(), sc.data_ptr(), item.scale_kind, item.shape[0],
                                                     item.shape[1], block, bits, sp, C.byref(out)))
                    handles[item.name] = QuantWeight(out.value, device)
                    rep.quantized += 1
                elif keep_fp8:
                    L.check(lib.lq_weight_from_fp8(src.data_ptr(), sc.data_ptr(), item.scale_kind, item.shape[0],
                                                   item.shape[1], sp, C.byref(out)))
                    handles[item.name] = QuantWeight(out.value, device)
                    rep.kept_fp8 += 1
                else:  # unaligned d_in: plain f32 weight, decoded on the device
                    L.check(lib.lq_weight_from_fp8(src.data_ptr(), sc.data_ptr(), item.scale_kind, item.shape[0],
                                                   item.shape[1], sp, C.byref(out)))
                    tmp = QuantWeight(out.value, device)
                    plain[item.name] = tmp.dequantize(torch.float32)
                    main.synchronize()
                    del tmp
                    rep.left_plain += 1
            else:
                t = src.view(_TORCH_DTYPE[item.dtype]).reshape(item.shape)
                if quantizable and item.dtype in ("F32", "BF16"):
                    out = C.c_void_p()
                    code = L.LQ_F32 if item.dtype == "F32" else L.LQ_BF16
                    L.check(lib.lq_quantize(t.data_ptr(), code, item.shape[0], item.shape[1], block, bits, sp, C.byref(out)))
                    handles[item.name] = QuantWeight(out.value, device)
                    rep.quantized += 1
                elif quantizable:  # f16: widen on the device, then quantize
                    w32 = t.to(torch.float32)
                    out = C.c_void_p()
                    L.check(lib.lq_quantize(w32.data_ptr(), L.LQ_F32, item.shape[0], item.shape[1], block, bits, sp,
                                            C.byref(out)))
                    handles[item.name] = QuantWeight(out.value, device)
                    w32.record_stream(main)
                    rep.quantized += 1
                else:
                    plain[item.name] = t.to(torch.float32).clone()
                    rep.left_plain += 1
            slot.consumed.record(main)
        main.synchronize()
        pool.shutdown()
        if progress:
            progress("", len(plan), len(plan))
    for h in handles.values():
        rep.packed_bytes += h.packed_bytes + h.scale_bytes
    return handles, plain, rep

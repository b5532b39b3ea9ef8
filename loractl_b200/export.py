"""Interop file formats of the trained adapters: what the kernels train, written so that ComfyUI /
kohya-ss / Krea loaders and the reference itself can read it, and read back for a resume.

Mirrors crates/loractl-core/src/export.rs (`export_adapters`, `import_adapters`, the two name
mappers, `sd_webui_hashes`) and the AdamW sidecar of crates/loractl-core/src/resume.rs:68-112,375-600.

File layout per adapted site (export.rs:262-326): `<key>.lora_down.weight` = A transposed to
`[rank, d_in]`, `<key>.lora_up.weight` = B transposed to `[d_out, rank]`, `<key>.alpha` = the `[1]`
scalar `scaling * rank`; all f32, tensors in name order, optional `__metadata__`.  With metadata
the file also carries `sshs_model_hash` / `sshs_legacy_hash`, computed over a first in-memory
serialization that holds only the `ss_*` subset of the metadata (export.rs:330-349).
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .adapters import LoraAdapters
from .loader import CheckpointError, SafetensorsFile

KOHYA_SS = "kohya_ss"
KREA2_DIFFUSERS = "krea2_diffusers"


class KohyaMapper:
    """`lora_<path with dots -> underscores>` + `.lora_down.weight` / `.lora_up.weight` / `.alpha`
    (export.rs:57-78)."""

    @staticmethod
    def prefix(path: str) -> str:
        return "lora_" + path.replace(".", "_")

    def down_key(self, path: str) -> str:
        return f"{self.prefix(path)}.lora_down.weight"

    def up_key(self, path: str) -> str:
        return f"{self.prefix(path)}.lora_up.weight"

    def alpha_key(self, path: str) -> str:
        return f"{self.prefix(path)}.alpha"


class Krea2DiffusersMapper:
    """Diffusers-style module paths with kohya suffixes, the convention ComfyUI's Krea 2 LoRA loader
    accepts (export.rs:80-137): `blocks.{i}` -> `transformer_blocks.{i}`, `txtfusion.` ->
    `text_fusion.`, and the trailing projection renamed (`attn.wq` -> `attn.to_q`, ...,
    `attn.wo` -> `attn.to_out.0`, `mlp.up` -> `ff.up`, ...)."""

    RENAMES = (("attn.wq", "attn.to_q"), ("attn.wk", "attn.to_k"), ("attn.wv", "attn.to_v"),
               ("attn.gate", "attn.to_gate"), ("attn.wo", "attn.to_out.0"), ("mlp.gate", "ff.gate"),
               ("mlp.up", "ff.up"), ("mlp.down", "ff.down"))

    @classmethod
    def diffusers_path(cls, path: str) -> str:
        out = path
        if out.startswith("blocks."):
            out = "transformer_blocks." + out[len("blocks."):]
        elif out.startswith("txtfusion."):
            out = "text_fusion." + out[len("txtfusion."):]
        for native, diffusers in cls.RENAMES:
            if out.endswith(native):
                return out[:-len(native)] + diffusers
        return out

    def down_key(self, path: str) -> str:
        return f"{self.diffusers_path(path)}.lora_down.weight"

    def up_key(self, path: str) -> str:
        return f"{self.diffusers_path(path)}.lora_up.weight"

    def alpha_key(self, path: str) -> str:
        return f"{self.diffusers_path(path)}.alpha"


def mapper_for(fmt: str):
    if fmt == KOHYA_SS:
        return KohyaMapper()
    if fmt == KREA2_DIFFUSERS:
        return Krea2DiffusersMapper()
    raise ValueError(f"unknown export format {fmt!r} (kohya_ss | krea2_diffusers)")


def serialize(tensors: Dict[str, Tuple[Tuple[int, ...], bytes]], metadata: Optional[Dict[str, str]]) -> bytes:
    """An all-f32 safetensors buffer: 8-byte little-endian header length, JSON header
    (`__metadata__` first when present, then the tensors in name order), header padded with spaces
    to a multiple of 8, data in the same order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {k: metadata[k] for k in sorted(metadata)}
    off = 0
    names = sorted(tensors)
    for name in names:
        shape, data = tensors[name]
        header[name] = {"dtype": "F32", "shape": list(shape), "data_offsets": [off, off + len(data)]}
        off += len(data)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    return struct.pack("<Q", len(blob)) + blob + b"".join(tensors[n][1] for n in names)


def sd_webui_hashes(buf: bytes) -> Tuple[str, str]:
    """(`sshs_model_hash`, `sshs_legacy_hash`) of a serialized buffer (export.rs:206-260): SHA-256
    of the tensor-data region, and the first 8 hex digits of the SHA-256 of the 64 KiB at file
    offset 0x100000 (an empty read for files under 1 MiB)."""
    (n,) = struct.unpack("<Q", buf[:8])
    start = min(8 + n, len(buf))
    model = hashlib.sha256(buf[start:]).hexdigest()
    legacy = hashlib.sha256(buf[0x100000:0x100000 + 0x10000] if len(buf) > 0x100000 else b"").hexdigest()
    return model, legacy[:8]


def _f32_bytes(t: torch.Tensor) -> Tuple[Tuple[int, ...], bytes]:
    a = t.detach().to("cpu", torch.float32).contiguous().numpy()
    return tuple(a.shape), a.astype("<f4", copy=False).tobytes()


def export_adapters(adapters: LoraAdapters, fmt: str, path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    """export.rs:262-361.  `metadata` None or empty writes no `__metadata__` at all."""
    m = mapper_for(fmt)
    tensors: Dict[str, Tuple[Tuple[int, ...], bytes]] = {}
    for delta, target in zip(adapters.deltas, adapters.targets):
        rank = delta.lora_a.shape[1]
        tensors[m.down_key(target)] = _f32_bytes(delta.lora_a.t())   # [rank, d_in]
        tensors[m.up_key(target)] = _f32_bytes(delta.lora_b.t())     # [d_out, rank]
        alpha = np.float32(float(delta.scaling) * rank)
        tensors[m.alpha_key(target)] = ((1,), np.asarray([alpha], dtype="<f4").tobytes())
    header = None
    if metadata:
        hashed = serialize(tensors, {k: v for k, v in metadata.items() if k.startswith("ss_")})
        model_hash, legacy_hash = sd_webui_hashes(hashed)
        header = dict(metadata)
        header["sshs_model_hash"] = model_hash
        header["sshs_legacy_hash"] = legacy_hash
    parent = os.path.dirname(str(path))
    if parent:
        os.makedirs(parent, exist_ok=True)
    with open(path, "wb") as f:
        f.write(serialize(tensors, header))


def import_adapters(adapters: LoraAdapters, fmt: str, path: str) -> int:
    """export.rs:363-449: reads every configured site's factors back (transposing to `A [d_in, rank]`,
    `B [rank, d_out]`), refusing non-f32, non-finite or mis-shaped tensors and an `.alpha` that
    disagrees with the configured `scaling * rank`.  Returns the number of sites restored."""
    m = mapper_for(fmt)
    with SafetensorsFile(path) as sf:
        def matrix(key: str) -> torch.Tensor:
            ent = sf.entries.get(key)
            if ent is None:
                raise CheckpointError(f"adapter export is missing tensor {key}")
            if ent.dtype != "F32":
                raise CheckpointError(f"tensor {key} is {ent.dtype}, expected F32")
            vals = np.frombuffer(sf.raw(key), dtype="<f4").reshape(ent.shape).copy()
            bad = np.flatnonzero(~np.isfinite(vals))
            if bad.size:
                raise CheckpointError(f"tensor {key} is not finite (element {int(bad[0])} is "
                                      f"{vals.reshape(-1)[bad[0]]}) — refusing to resume from a corrupt adapter")
            return torch.from_numpy(vals)

        restored = 0
        with torch.no_grad():
            for delta, target in zip(adapters.deltas, adapters.targets):
                a = matrix(m.down_key(target)).t()
                b = matrix(m.up_key(target)).t()
                if tuple(a.shape) != tuple(delta.lora_a.shape) or tuple(b.shape) != tuple(delta.lora_b.shape):
                    raise CheckpointError(
                        f"resume shape mismatch at {target}: file A {list(a.shape)} / B {list(b.shape)} vs configured "
                        f"A {list(delta.lora_a.shape)} / B {list(delta.lora_b.shape)} — did lora.rank change?")
                akey = m.alpha_key(target)
                if akey in sf.entries:
                    file_alpha = float(np.frombuffer(sf.raw(akey), dtype="<f4")[0])
                    want = float(np.float32(float(delta.scaling) * delta.lora_a.shape[1]))
                    if abs(file_alpha - want) > 1e-6 * max(1.0, abs(want)):
                        raise CheckpointError(f"resume alpha mismatch at {target}: file {file_alpha} vs configured {want}")
                delta.lora_a.copy_(a.to(delta.lora_a.device))
                delta.lora_b.copy_(b.to(delta.lora_b.device))
                restored += 1
    return restored


# ---- AdamW sidecar (resume.rs:68-112,375-600) -------------------------------------------------
ARTIFACT_KIND_KEY, ARTIFACT_KIND = "loractl_artifact_kind", "optimizer-state"
TIME_KEY, LOSS_SCALE_KEY = "loractl_adamw_time", "loractl_loss_scale"
CLEAN_STREAK_KEY, STEPS_DONE_KEY = "loractl_clean_streak", "loractl_steps_done"
FACTOR_KEYS = (("lora_down", True), ("lora_up", False))


def moment_key(target: str, suffix: str, kind: str) -> str:
    """`<site>.<lora_down|lora_up>.<exp_avg|exp_avg_sq>` — never ends in `.weight` / `.alpha`, so no
    LoRA loader's key map can match this file (resume.rs:88-104)."""
    return f"{target}.{suffix}.{kind}"


def optim_sidecar_path(adapter_path: str) -> str:
    """Beside the adapter, same stem, `.optim.safetensors` (resume.rs:106-119)."""
    d, name = os.path.split(str(adapter_path))
    stem = os.path.splitext(name)[0] or "adapter"
    return os.path.join(d, stem + ".optim.safetensors")


def save_optimizer_state(flat, optim_steps: int, loss_scale: float, clean_streak: int, steps_done: int,
                         path: str) -> bool:
    """Writes the flat AdamW moments of `flat` (an `optim.FlatAdapters`) per site and factor, in the
    parameters' own layout, with the bias-correction step count and the loss-scale state in
    `__metadata__`.  Nothing is written (and False returned) before the first update, so an
    existing sidecar is not clobbered by an empty one (resume.rs:440-452)."""
    if optim_steps <= 0:
        return False
    tensors: Dict[str, Tuple[Tuple[int, ...], bytes]] = {}
    ads = flat.adapters
    for i, (delta, target) in enumerate(zip(ads.deltas, ads.targets)):
        for j, (suffix, is_down) in enumerate(FACTOR_KEYS):
            p = delta.lora_a if is_down else delta.lora_b
            o = flat.offsets[2 * i + j]
            for kind, buf in (("exp_avg", flat.exp_avg), ("exp_avg_sq", flat.exp_avg_sq)):
                tensors[moment_key(target, suffix, kind)] = _f32_bytes(buf[o:o + p.numel()].view(p.shape))
    header = {ARTIFACT_KIND_KEY: ARTIFACT_KIND, TIME_KEY: str(int(optim_steps)), LOSS_SCALE_KEY: repr(float(loss_scale)),
              CLEAN_STREAK_KEY: str(int(clean_streak)), STEPS_DONE_KEY: str(int(steps_done))}
    parent = os.path.dirname(str(path))
    if parent:
        os.makedirs(parent, exist_ok=True)
    with open(path, "wb") as f:
        f.write(serialize(tensors, header))
    return True


def load_optimizer_state(flat, path: str) -> Dict[str, float]:
    """Restores the moments into `flat` and returns `{time, loss_scale, clean_streak, steps_done}`.
    Refuses a file that is not an optimizer sidecar, misses a tensor or has a wrong shape."""
    with SafetensorsFile(path) as sf:
        if sf.metadata.get(ARTIFACT_KIND_KEY) != ARTIFACT_KIND:
            raise CheckpointError(f"{path} is not an optimizer-state sidecar "
                                  f"({ARTIFACT_KIND_KEY} = {sf.metadata.get(ARTIFACT_KIND_KEY)!r})")
        ads = flat.adapters
        for i, (delta, target) in enumerate(zip(ads.deltas, ads.targets)):
            for j, (suffix, is_down) in enumerate(FACTOR_KEYS):
                p = delta.lora_a if is_down else delta.lora_b
                o = flat.offsets[2 * i + j]
                for kind, buf in (("exp_avg", flat.exp_avg), ("exp_avg_sq", flat.exp_avg_sq)):
                    key = moment_key(target, suffix, kind)
                    ent = sf.entries.get(key)
                    if ent is None:
                        raise CheckpointError(f"optimizer state is missing tensor {key}")
                    if ent.dtype != "F32" or tuple(ent.shape) != tuple(p.shape):
                        raise CheckpointError(f"optimizer state tensor {key} is {ent.dtype} {list(ent.shape)}, "
                                              f"expected F32 {list(p.shape)}")
                    vals = torch.from_numpy(np.frombuffer(sf.raw(key), dtype="<f4").reshape(ent.shape).copy())
                    buf[o:o + p.numel()].view(p.shape).copy_(vals.to(buf.device))
        md = sf.metadata
        return {"time": int(md.get(TIME_KEY, "0")), "loss_scale": float(md.get(LOSS_SCALE_KEY, "1")),
                "clean_streak": int(md.get(CLEAN_STREAK_KEY, "0")), "steps_done": int(md.get(STEPS_DONE_KEY, "0"))}

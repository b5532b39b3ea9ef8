"""CPU tests of the checkpoint side of streaming quantize-at-load: the safetensors container and the
header classification rules of crates/loractl-core/src/fp8.rs:119-206 (the cases its own tests
exercise in crates/loractl-core/tests/fp8.rs: legacy format, missing / mistyped / misshapen
sidecars, orphan sidecars, dropped quant metadata, unsupported dtypes)."""
import json
import struct

import numpy as np
import pytest

from loractl_b200 import loader as LD


def f32(a):
    a = np.asarray(a, dtype="<f4")
    return ("F32", tuple(a.shape), a.tobytes())


def fp8(shape, seed=0):
    rng = np.random.default_rng(seed)
    b = rng.integers(0, 0x7F, size=shape, dtype=np.uint8)  # no NaN encodings
    return ("F8_E4M3", tuple(shape), b.tobytes())


def test_container_roundtrip_and_metadata(tmp_path):
    p = tmp_path / "a.safetensors"
    w = np.arange(12, dtype=np.float32).reshape(3, 4)
    LD.write_safetensors(p, {"b.weight": f32(w), "a.bias": f32([1.0, 2.0])}, {"format": "pt"})
    raw = p.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    assert n % 8 == 0 and json.loads(raw[8:8 + n])["b.weight"]["shape"] == [3, 4]
    with LD.SafetensorsFile(p) as sf:
        assert sf.metadata == {"format": "pt"} and set(sf.entries) == {"a.bias", "b.weight"}
        assert np.array_equal(np.frombuffer(sf.raw("b.weight"), dtype="<f4").reshape(3, 4), w)
        assert not LD.is_fp8_checkpoint(sf)
        assert [i.name for i in LD.classify(sf)] == ["a.bias", "b.weight"]


def test_truncated_and_inconsistent_files_are_errors(tmp_path):
    p = tmp_path / "t.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(LD.CheckpointError, match="too short"):
        LD.SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(LD.CheckpointError, match="inconsistent data offsets"):
        LD.SafetensorsFile(p)


def test_fp8_classification_accepts_scalar_and_per_channel_sidecars(tmp_path):
    p = tmp_path / "f.safetensors"
    LD.write_safetensors(p, {
        "blk.wq.weight": fp8((8, 64)), "blk.wq.weight_scale": f32(np.full((8,), 0.5)),
        "blk.wo.weight": fp8((4, 64), 1), "blk.wo.weight_scale": f32(np.float32(0.25)),
        "blk.wk.weight": fp8((4, 64), 2), "blk.wk.weight_scale": f32([0.125]),
        "blk.norm.weight": f32(np.ones(64)),
        "blk.wq.comfy_quant": f32([0.0]), "blk.wq.input_scale": f32([1.0]),
    })
    with LD.SafetensorsFile(p) as sf:
        assert LD.is_fp8_checkpoint(sf)
        plan = {i.name: i for i in LD.classify(sf)}
    assert set(plan) == {"blk.wq.weight", "blk.wo.weight", "blk.wk.weight", "blk.norm.weight"}
    assert plan["blk.wq.weight"].scale_kind == 1 and plan["blk.wo.weight"].scale_kind == 0
    assert plan["blk.wk.weight"].scale_kind == 0 and plan["blk.norm.weight"].scale_name is None


@pytest.mark.parametrize("tensors,msg", [
    ({"scaled_fp8": f32([0.0])}, "legacy ComfyUI"),
    ({"a.weight": fp8((4, 64)), "a.scale_weight": f32([1.0])}, "legacy ComfyUI"),
    ({"a.weight": fp8((4, 64))}, "has no 'a.weight_scale' sidecar"),
    ({"a.weight": fp8((4, 64)), "a.weight_scale": ("BF16", (1,), b"\0\0")}, "expected F32"),
    ({"a.weight": fp8((4, 64)), "a.weight_scale": f32(np.ones(3))}, "neither scalar"),
    ({"a.weight": fp8((4, 64)), "a.weight_scale": f32(np.ones((4, 1)))}, "neither scalar"),
    ({"a.weight": fp8((0, 64)), "a.weight_scale": f32(np.ones((0,)))}, r"is empty \(\[0\]\)"),
    ({"a.weight": f32(np.ones((4, 64))), "a.weight_scale": f32([1.0])}, "has no fp8 base weight 'a.weight'"),
    ({"a.weight": ("I64", (2,), b"\0" * 16)}, "unsupported dtype I64"),
])
def test_fp8_classification_rejections(tmp_path, tensors, msg):
    p = tmp_path / "bad.safetensors"
    LD.write_safetensors(p, tensors)
    with LD.SafetensorsFile(p) as sf:
        with pytest.raises(LD.CheckpointError, match=msg):
            LD.classify(sf)

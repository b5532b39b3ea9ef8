"""CPU tests of the adapter interop formats (crates/loractl-core/src/export.rs, resume.rs), against
the reference's own goldens: tests/golden/lora_export.json (kohya-ss keys, transposes and alpha of
the 4 x 6 rank-2 toy, crates/loractl-core/tests/adapter_export.rs:82-152) and
tests/golden/krea2_lora_keys.json (the site keys ComfyUI's Krea 2 loader accepts,
crates/loractl-core/tests/krea2_lora_keys.rs)."""
import hashlib
import json
import struct

import numpy as np
import pytest
import torch

from loractl_b200 import export as EX
from loractl_b200 import loader as LD
from loractl_b200.adapters import LoraAdapters, LoraConfig, LoraSite, TargetSpec, build_adapters
from loractl_b200.lora import LoraDelta


def toy_set(golden):
    hp = golden["hyperparams"]
    d = LoraDelta(hp["d_in"], hp["d_out"], hp["rank"], hp["alpha"])
    a_t = np.asarray(golden["a_transposed"], np.float32).reshape(golden["a_shape"])
    b_t = np.asarray(golden["b_transposed"], np.float32).reshape(golden["b_shape"])
    with torch.no_grad():
        d.lora_a.copy_(torch.from_numpy(a_t.T.copy()))
        d.lora_b.copy_(torch.from_numpy(b_t.T.copy()))
    return LoraAdapters([d], [hp["path"]]), a_t, b_t


def test_kohya_export_matches_golden(golden_dir, tmp_path):
    golden = json.loads((golden_dir / "lora_export.json").read_text())
    ads, a_t, b_t = toy_set(golden)
    p = tmp_path / "toy.safetensors"
    EX.export_adapters(ads, EX.KOHYA_SS, p)
    with LD.SafetensorsFile(p) as sf:
        assert sorted(sf.entries) == golden["kohya_keys"] and sf.metadata == {}
        k = "lora_transformer_h_0_attn_c_attn"
        assert sf.entries[k + ".alpha"].shape == (1,) and sf.entries[k + ".alpha"].dtype == "F32"
        assert np.frombuffer(sf.raw(k + ".alpha"), "<f4")[0] == np.float32(golden["alpha_value"])
        assert list(sf.entries[k + ".lora_down.weight"].shape) == golden["a_shape"]
        assert list(sf.entries[k + ".lora_up.weight"].shape) == golden["b_shape"]
        assert np.array_equal(np.frombuffer(sf.raw(k + ".lora_down.weight"), "<f4").reshape(a_t.shape), a_t)
        assert np.array_equal(np.frombuffer(sf.raw(k + ".lora_up.weight"), "<f4").reshape(b_t.shape), b_t)


def test_import_restores_factors_and_guards(golden_dir, tmp_path):
    golden = json.loads((golden_dir / "lora_export.json").read_text())
    ads, _, _ = toy_set(golden)
    p = tmp_path / "toy.safetensors"
    EX.export_adapters(ads, EX.KOHYA_SS, p)
    fresh, _, _ = toy_set(golden)
    with torch.no_grad():
        fresh.deltas[0].lora_a.zero_()
        fresh.deltas[0].lora_b.zero_()
    assert EX.import_adapters(fresh, EX.KOHYA_SS, p) == 1
    assert torch.equal(fresh.deltas[0].lora_a, ads.deltas[0].lora_a)
    assert torch.equal(fresh.deltas[0].lora_b, ads.deltas[0].lora_b)
    # a different rank is refused by name
    hp = golden["hyperparams"]
    other = LoraAdapters([LoraDelta(hp["d_in"], hp["d_out"], 3, hp["alpha"])], [hp["path"]])
    with pytest.raises(LD.CheckpointError, match="did lora.rank change"):
        EX.import_adapters(other, EX.KOHYA_SS, p)
    # a missing site is refused by key
    missing = LoraAdapters([LoraDelta(hp["d_in"], hp["d_out"], hp["rank"], hp["alpha"])], ["transformer.h.1.attn.c_attn"])
    with pytest.raises(LD.CheckpointError, match="missing tensor lora_transformer_h_1_attn_c_attn.lora_down.weight"):
        EX.import_adapters(missing, EX.KOHYA_SS, p)
    # a non-finite factor is refused before anything is written
    with torch.no_grad():
        ads.deltas[0].lora_b[0, 0] = float("nan")
    EX.export_adapters(ads, EX.KOHYA_SS, p)
    with pytest.raises(LD.CheckpointError, match="not finite"):
        EX.import_adapters(fresh, EX.KOHYA_SS, p)


def test_multi_delta_export_writes_distinct_keys_per_target(tmp_path):
    sites = [LoraSite(f"transformer.h.{i}.attn.c_attn", 8, 12) for i in range(3)]
    ads = build_adapters(sites, LoraConfig(rank=2, alpha=4.0, targets=[TargetSpec(r".*")]), "cpu")
    p = tmp_path / "multi.safetensors"
    EX.export_adapters(ads, EX.KOHYA_SS, p)
    with LD.SafetensorsFile(p) as sf:
        assert len(sf.entries) == 9
        for i in range(3):
            for suf in (".lora_down.weight", ".lora_up.weight", ".alpha"):
                assert f"lora_transformer_h_{i}_attn_c_attn{suf}" in sf.entries


def test_every_krea2_key_is_one_comfyui_accepts(golden_dir, tmp_path):
    g = json.loads((golden_dir / "krea2_lora_keys.json").read_text())
    accepted = set(g["accepted_keys"])
    names = ("attn.wq", "attn.wk", "attn.wv", "attn.gate", "attn.wo", "mlp.gate", "mlp.up", "mlp.down")
    paths = [f"blocks.{i}.{n}" for i in range(g["layers"]) for n in names]
    paths += [f"txtfusion.{kind}_blocks.{i}.{n}" for kind in ("layerwise", "refiner") for i in range(2) for n in names]
    sites = [LoraSite(p, 8, 8) for p in paths]
    ads = build_adapters(sites, LoraConfig(rank=4, alpha=8.0, targets=[TargetSpec(r".*")]), "cpu")
    p = tmp_path / "krea2.safetensors"
    EX.export_adapters(ads, EX.KREA2_DIFFUSERS, p)
    with LD.SafetensorsFile(p) as sf:
        keys = list(sf.entries)
    assert len(keys) == 3 * len(paths)
    for k in keys:
        site = next(k[:-len(s)] for s in (".lora_down.weight", ".lora_up.weight", ".alpha") if k.endswith(s))
        assert site in accepted, k
    m = EX.Krea2DiffusersMapper()
    assert m.down_key("blocks.3.attn.wo") == "transformer_blocks.3.attn.to_out.0.lora_down.weight"
    assert m.alpha_key("txtfusion.refiner_blocks.1.mlp.up") == "text_fusion.refiner_blocks.1.ff.up.alpha"


def test_metadata_and_the_two_hashes(golden_dir, tmp_path):
    golden = json.loads((golden_dir / "lora_export.json").read_text())
    ads, _, _ = toy_set(golden)
    p = tmp_path / "meta.safetensors"
    meta = {"ss_network_module": "networks.lora", "ss_steps": "20", "modelspec.title": "toy"}
    EX.export_adapters(ads, EX.KOHYA_SS, p, meta)
    raw = p.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    with LD.SafetensorsFile(p) as sf:
        md = sf.metadata
    assert {k: md[k] for k in meta} == meta
    # the model hash covers the tensor-data region only, so it can be recomputed from the finished file
    assert md["sshs_model_hash"] == hashlib.sha256(raw[8 + n:]).hexdigest()
    # the legacy hash of a file under 1 MiB is the hash of an empty read
    assert md["sshs_legacy_hash"] == hashlib.sha256(b"").hexdigest()[:8]
    # user-editable modelspec.* fields do not change the file's identity
    p2 = tmp_path / "meta2.safetensors"
    EX.export_adapters(ads, EX.KOHYA_SS, p2, dict(meta, **{"modelspec.title": "renamed"}))
    with LD.SafetensorsFile(p2) as sf2:
        assert sf2.metadata["sshs_model_hash"] == md["sshs_model_hash"]


def test_optimizer_sidecar_roundtrip(tmp_path):
    from loractl_b200.optim import FlatAdapters

    sites = [LoraSite(f"blocks.{i}.attn.wq", 8, 12) for i in range(2)]
    ads = build_adapters(sites, LoraConfig(rank=2, alpha=4.0, targets=[TargetSpec(r".*")]), "cpu")
    flat = FlatAdapters(ads, torch.device("cpu"))
    adapter_path = tmp_path / "out" / "adapter.safetensors"
    side = EX.optim_sidecar_path(adapter_path)
    assert side.endswith("adapter.optim.safetensors")
    assert EX.save_optimizer_state(flat, 0, 1.0, 0, 0, side) is False  # nothing stepped: nothing written
    g = torch.Generator().manual_seed(3)
    flat.exp_avg.copy_(torch.randn(flat.numel, generator=g))
    flat.exp_avg_sq.copy_(torch.rand(flat.numel, generator=g))
    assert EX.save_optimizer_state(flat, 7, 512.0, 3, 7, side) is True
    with LD.SafetensorsFile(side) as sf:
        keys = list(sf.entries)
        assert len(keys) == 8 and all(not k.endswith((".weight", ".alpha")) for k in keys)
        assert "blocks.0.attn.wq.lora_down.exp_avg" in keys and "blocks.1.attn.wq.lora_up.exp_avg_sq" in keys
        assert sf.entries["blocks.0.attn.wq.lora_down.exp_avg"].shape == (8, 2)  # the parameter's own layout
    flat2 = FlatAdapters(build_adapters(sites, LoraConfig(rank=2, alpha=4.0, targets=[TargetSpec(r".*")]), "cpu"),
                         torch.device("cpu"))
    st = EX.load_optimizer_state(flat2, side)
    assert st == {"time": 7, "loss_scale": 512.0, "clean_streak": 3, "steps_done": 7}
    for i in range(4):
        o = flat.offsets[i]
        n = flat._params[i].numel()
        assert torch.equal(flat2.exp_avg[o:o + n], flat.exp_avg[o:o + n])
        assert torch.equal(flat2.exp_avg_sq[o:o + n], flat.exp_avg_sq[o:o + n])
    # an adapter export is not a sidecar
    EX.export_adapters(ads, EX.KOHYA_SS, adapter_path)
    with pytest.raises(LD.CheckpointError, match="not an optimizer-state sidecar"):
        EX.load_optimizer_state(flat2, adapter_path)

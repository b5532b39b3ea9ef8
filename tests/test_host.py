"""CPU-side tests: the C ABI loads and exports every declared symbol, and the host logic that
mirrors the reference's interface (chunk layout, vocabulary, adapter registry, guards)."""
import ctypes as C
import json
import math
import pathlib
import re

import pytest
import torch

import loractl_b200 as lb
from loractl_b200 import _lib as L
from oracle import lq_oracle as O

ROOT = pathlib.Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "loractl_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = L.lib()
    names = declared_symbols()
    assert len(names) >= 17
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/loractl_b200.h but not exported"
    assert sorted(L.SIGNATURES) == names, "ctypes SIGNATURES and the header disagree"
    assert lib.lq_abi_version() == 2


def test_dequant_chunk_rows_through_the_c_abi():
    """crates/loractl-core/tests/quant.rs:333-349."""
    for args in [(8, 64, 0), (8, 64, 2048), (8, 64, 2047), (10, 64, 768), (5, 64, 1), (1, 64, 1),
                 (97, 64, 5000), (36864, 6144, 512 << 20), (3072, 3072, 512 << 20)]:
        assert lb.dequant_chunk_rows(*args) == O.dequant_chunk_rows(*args)
    assert lb.dequant_chunk_rows(36864, 6144, 512 << 20) == [18432, 18432]


def test_no_cpu_path_and_null_handle_errors():
    with pytest.raises(RuntimeError, match="no CPU path"):
        lb.quantize_linear_weight(torch.zeros(4, 64), 4)
    rc = L.lib().lq_linear_fwd(None, None, 4, 0, None, None, 0, 1.0, None, None, None, 0, None, None)
    assert rc == L.LQ_ERR_INVALID and b"quantized weight" in L.lib().lq_last_error()
    assert L.lib().lq_linear_workspace_bytes(None, 4, 0, 0) == 0


def test_vocabulary_matches_the_reference_spellings():
    """crates/loractl-core/src/config.rs:534-549,595-604,655-664."""
    assert lb.BackendKind.parse("B200") is lb.BackendKind.B200
    assert lb.BackendKind.parse("libtorch") is lb.BackendKind.TCH
    with pytest.raises(ValueError, match="unknown backend"):
        lb.BackendKind.parse("rocm")
    assert lb.Quant.parse("i4") is lb.Quant.INT4 and lb.Quant.parse("OFF") is lb.Quant.NONE
    with pytest.raises(ValueError, match="unknown quant"):
        lb.Quant.parse("int2")
    assert lb.quant_value(lb.Quant.NONE) is None and lb.quant_value(lb.Quant.INT8) == 8
    assert lb.Precision.parse("bfloat16") is lb.Precision.BF16
    assert lb.QUANT_BLOCK == 32


def test_guard_matrix_rejects_named_combinations():
    """crates/loractl-core/tests/quant_trainer.rs:148-258: illegal combos bail with a named reason."""
    ok = lb.ComputeConfig(backend=lb.BackendKind.B200, precision=lb.Precision.BF16, quant=lb.Quant.INT4,
                          grad_checkpointing=True)
    lb.validate_b200(ok)
    with pytest.raises(ValueError, match="f16"):
        lb.validate_b200(lb.ComputeConfig(backend=lb.BackendKind.B200, precision=lb.Precision.F16))
    with pytest.raises(ValueError, match="grad_checkpointing"):
        lb.validate_b200(ok, lora_dropout=0.1)
    with pytest.raises(ValueError, match="dropout"):
        lb.validate_b200(lb.ComputeConfig(backend=lb.BackendKind.B200, quant=lb.Quant.INT8), lora_dropout=0.1)
    with pytest.raises(ValueError, match="b200"):
        lb.validate_b200(lb.ComputeConfig(backend=lb.BackendKind.CUDA))


def test_build_adapters_targets_and_overrides():
    """crates/loractl-core/src/adapters.rs:116-145 and its unit tests."""
    sites = [lb.LoraSite("blocks.0.attn.wq", 64, 96), lb.LoraSite("blocks.0.attn.wk", 64, 32),
             lb.LoraSite("blocks.0.mlp.up", 64, 256), lb.LoraSite("blocks.10.attn.wq", 64, 96)]
    cfg = lb.LoraConfig(rank=4, alpha=8.0, targets=[lb.TargetSpec(r"attn\.wq$", rank=2, alpha=6.0),
                                                    lb.TargetSpec(r"mlp\.")])
    ad = lb.build_adapters(sites, cfg)
    assert ad.targets == ["blocks.0.attn.wq", "blocks.0.mlp.up", "blocks.10.attn.wq"]
    wq, up = ad.get("blocks.0.attn.wq"), ad.get("blocks.0.mlp.up")
    assert tuple(wq.lora_a.shape) == (64, 2) and tuple(wq.lora_b.shape) == (2, 96) and wq.scaling == 3.0
    assert tuple(up.lora_a.shape) == (64, 4) and up.scaling == 2.0
    assert ad.get("blocks.0.attn.wk") is None and ad.get("blocks.1") is None
    assert float(wq.lora_b.abs().max()) == 0.0 and float(wq.lora_a.abs().max()) > 0.0
    assert float(wq.lora_a.abs().max()) <= 1 / math.sqrt(64)
    with pytest.raises(ValueError, match="invalid LoRA target pattern"):
        lb.build_adapters(sites, lb.LoraConfig(targets=[lb.TargetSpec("(")]))
    # rank clamps to >= 1 (crates/loractl-core/src/lora.rs:185)
    assert lb.LoraDelta(8, 8, 0, 4.0).rank == 1
    # plain-base delta: zero-init B is an exact no-op
    x = torch.randn(3, 64)
    assert torch.equal(ad.apply("blocks.0.attn.wq", x, torch.ones(3, 96)), torch.ones(3, 96))


def test_host_fp8_lut_and_scale_kinds(golden_dir):
    lut = json.loads((golden_dir / "fp8_lut_golden.json").read_text())["lut"]
    ours = lb.e4m3fn_lut()
    for i, v in enumerate(lut):
        assert (math.isnan(ours[i]) if v is None else ours[i] == v)
    from loractl_b200.fp8 import scale_kind_for

    assert scale_kind_for((5, 3), ()) == L.LQ_SCALE_SCALAR and scale_kind_for((5, 3), (1,)) == L.LQ_SCALE_SCALAR
    assert scale_kind_for((5, 3), (5,)) == L.LQ_SCALE_PER_CHANNEL
    with pytest.raises(ValueError):
        scale_kind_for((5, 3), (3,))


def test_split_streams_is_slicing_with_a_concatenating_backward():
    """`harness.split_streams` (pure tensor ops, so it runs here): values equal the plain slices, outputs
    are contiguous, and the gradient of any function of the two parts equals the one through slicing —
    for one sample (bypass: views) and for several (one copy forward, one concatenation backward)."""
    import torch

    from loractl_b200.harness import split_streams

    for b in (1, 3):
        x = torch.randn(b, 7, 5, dtype=torch.float64, requires_grad=True)
        y = x.detach().clone().requires_grad_(True)
        img, txt = split_streams(x, 4)
        assert img.is_contiguous() and txt.is_contiguous()
        assert torch.equal(img, y[:, :4]) and torch.equal(txt, y[:, 4:])
        w_img, w_txt = torch.randn(b, 4, 5, dtype=torch.float64), torch.randn(b, 3, 5, dtype=torch.float64)
        ((img * w_img).sum() + (img ** 2).sum() + (txt * w_txt).sum()).backward()
        ((y[:, :4] * w_img).sum() + (y[:, :4] ** 2).sum() + (y[:, 4:] * w_txt).sum()).backward()
        assert torch.allclose(x.grad, y.grad, rtol=0, atol=1e-12)

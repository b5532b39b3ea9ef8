"""Block-level parity against the reference's own golden trace.

The reference pins its tiny MMDiT against the upstream Krea 2 implementation stage by stage at
1e-4 (crates/loractl-core/tests/mmdit_parity.rs:223-265).  Block 0 is cut out of that trace: the
stage tensors before it (`after_txtmlp`, `after_first`, `tvec`, `pos`, `txtmask`) and after it
(`after_block0`), and the block's weights (tests/golden/mmdit_tiny_block0.safetensors, made by
tests/golden/make_golden.py).

  * CPU: `SingleStreamBlock` with Plain bases must replay `after_block0` within 1e-4 — this pins
    the caller of the hot path (norms, RoPE, GQA gated attention, SwiGLU, modulation, padding).
  * GPU: the same block with every site quantized (`into_quantized`) must (a) equal, to f32
    summation noise, a Plain block built from the dequantized weights — the block composed of
    library sites computes the same function as the reference's composition of burn ops; (b) track
    the unquantized block inside the reference's quant bands (crates/loractl-core/tests/
    quant_mmdit.rs:165-226: int8 5e-2 / cosine 0.999, int4 5e-1 / 0.99); (c) be bit-identical
    with zero-initialised adapters attached (quant_mmdit.rs:228-255); (d) give finite gradients to
    every A and B and move B off zero after one step (quant_mmdit.rs:257-313).
"""
import pathlib

import numpy as np
import pytest
import torch
from safetensors.torch import load_file

from loractl_b200 import single_stream as S

GOLDEN = pathlib.Path(__file__).parent / "golden" / "mmdit_tiny_block0.safetensors"


def load_case(device="cpu"):
    t = {k: v.to(device) for k, v in load_file(str(GOLDEN)).items()}
    cfg = S.MmditConfig.tiny()
    combined = torch.cat([t["stage.after_txtmlp"], t["stage.after_first"]], dim=1)
    img_len = t["stage.after_first"].shape[1]
    mask = torch.cat([t["stage.txtmask"], torch.ones(img_len, device=device)]).reshape(1, -1)
    combined, mask, pos = S.pad_sequence(combined, mask, t["stage.pos"])
    rope = S.rope_tables(pos, cfg.head_dim, cfg.theta)
    t["valid"] = mask.reshape(1, -1, 1)  # 1 where the combined, padded key mask lets a token through
    return cfg, t, combined, t["stage.tvec"], rope, S.additive_mask(mask)


def zero_masked(out, t):
    """The golden is dumped with masked positions zeroed (the masked-position contract of
    crates/loractl-core/tests/mmdit_parity.rs:248-260); only valid tokens are compared."""
    return out * t["valid"]


def peak_rel(a, b):
    a, b = a.detach().float().cpu().numpy().ravel(), b.detach().float().cpu().numpy().ravel()
    return float(np.abs(a - b).max() / np.abs(b).max())


def cosine(a, b):
    a, b = a.detach().double().cpu().numpy().ravel(), b.detach().double().cpu().numpy().ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def test_plain_block_replays_the_reference_golden_on_cpu():
    cfg, t, x, tvec, rope, mask4 = load_case()
    assert x.shape == (1, 256, 96)  # 6 text + 16 image tokens, zero-padded to 256
    blk = S.SingleStreamBlock.from_tensors(cfg, t, "blocks.0")
    out = blk(x, tvec, rope, mask4)
    want = t["stage.after_block0"]
    assert out.shape == want.shape
    assert float((zero_masked(out, t) - want).abs().max()) <= 1e-4  # the reference's stage tolerance


def test_site_enumeration_matches_the_reference():
    cfg = S.MmditConfig.tiny()
    blk = S.SingleStreamBlock(cfg)
    names = [s.path for s in blk.injectable_sites("blocks.3")]
    assert names == [f"blocks.3.{n}" for n in ("attn.wq", "attn.wk", "attn.wv", "attn.wo", "mlp.gate", "mlp.up",
                                                "mlp.down")]
    assert S.MmditConfig.swiglu_dim(96, 4) == 256 and S.MmditConfig.swiglu_dim(6144, 4) == 16384
    assert S.MmditConfig.rope_axes(16) == (4, 6, 6) and S.MmditConfig.rope_axes(128) == (32, 48, 48)


@pytest.mark.gpu
@pytest.mark.parametrize("bits,rel_tol,cos_min", [(8, 5e-2, 0.999), (4, 5e-1, 0.99)])
def test_quantized_block_matches_its_dequantized_twin_and_tracks_the_plain_block(bits, rel_tol, cos_min):
    cfg, t, x, tvec, rope, mask4 = load_case("cuda")
    plain = S.SingleStreamBlock.from_tensors(cfg, t, "blocks.0").cuda()
    ref = plain(x, tvec, rope, mask4)
    assert float((zero_masked(ref, t) - t["stage.after_block0"]).abs().max()) <= 1e-4
    quant = S.SingleStreamBlock.from_tensors(cfg, t, "blocks.0").cuda()
    done, left = quant.into_quantized(bits, block=32)
    assert (done, left) == (8, 0)  # every width (96, 256) is a multiple of the reference's block of 32
    out = quant(x, tvec, rope, mask4)
    # (a) twin: Plain bases holding dequantize(quantize(w)) — same function, f32 arithmetic both ways
    twin = S.SingleStreamBlock.from_tensors(cfg, t, "blocks.0").cuda()
    with torch.no_grad():
        for (_, qb), (_, tb) in zip(quant.base_linears(), twin.base_linears()):
            tb.inner.weight.copy_(qb.inner.dequantized_weight())
    assert peak_rel(out, twin(x, tvec, rope, mask4)) <= 2e-5
    # (b) the reference's quant bands against the unquantized block
    assert float((out - ref).abs().max()) > 0.0, "bit-identical to plain: did quantization run?"
    assert peak_rel(out, ref) <= rel_tol and cosine(out, ref) >= cos_min


@pytest.mark.gpu
def test_zero_init_adapters_are_a_bit_identical_no_op_and_one_step_trains_b():
    import loractl_b200 as lb
    from loractl_b200.adapters import LoraConfig, TargetSpec, build_adapters

    cfg, t, x, tvec, rope, mask4 = load_case("cuda")
    blk = S.SingleStreamBlock.from_tensors(cfg, t, "blocks.0").cuda()
    blk.into_quantized(4, block=32)
    base = blk(x, tvec, rope, mask4)
    adapters = build_adapters(blk.injectable_sites("blocks.0"), LoraConfig(rank=4, alpha=8.0, targets=[TargetSpec(r".*")]),
                              torch.device("cuda"))
    assert len(adapters.deltas) == 7
    out = blk(x, tvec, rope, mask4, adapters, "blocks.0")
    assert torch.equal(out, base)  # zero-initialised B adds exact zeros
    params = [p for d in adapters.deltas for p in (d.lora_a, d.lora_b)]
    opt = torch.optim.Adam(params, lr=1e-2)
    loss = (out - t["stage.after_block0"] * 0.5).pow(2).mean()
    loss.backward()
    lb.check_device_status()
    for d in adapters.deltas:
        assert d.lora_a.grad is not None and d.lora_b.grad is not None
        assert torch.isfinite(d.lora_a.grad).all() and torch.isfinite(d.lora_b.grad).all()
    opt.step()
    assert all(float(d.lora_b.abs().max()) > 0.0 for d in adapters.deltas), "B did not move off zero"

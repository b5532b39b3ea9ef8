"""Pins the CPU oracle to the reference's own golden vectors.

Mirrors crates/loractl-core/tests/quant.rs:96-139 (dq <= 1e-6, y <= 1e-5),
tests/fp8.rs:140-158,602-662 (LUT bit-for-bit, dequant cases) and
tests/lora_reference.rs:49-122 (20 SGD steps within 1e-5).
"""
import json
import math

import numpy as np
import pytest

from oracle import lq_oracle as O


def _load(golden_dir, name):
    return json.loads((golden_dir / name).read_text())


@pytest.mark.parametrize("name,bits", [("quant_int4_golden.json", 4), ("quant_int8_golden.json", 8)])
def test_quant_golden_dq_and_matmul(golden_dir, name, bits):
    g = _load(golden_dir, name)
    assert g["block"] == 32
    w = np.array(g["w"], np.float32)
    x = np.array(g["x"], np.float32)
    codes, scales = O.quantize(w, g["block"], bits)
    dq = O.dequantize(codes, scales, g["block"])
    assert np.abs(dq - np.array(g["dq"], np.float32)).max() <= 1e-6
    y = O.quant_matmul_t(x, dq)
    assert np.abs(y - np.array(g["y"], np.float32)).max() <= 1e-5
    assert np.abs(codes).max() <= O.qmax_for_bits(bits)


def test_quant_extra_golden_blocks_32_and_64(golden_dir):
    for c in _load(golden_dir, "quant_extra_golden.json")["cases"]:
        w = np.array(c["w"], np.float32)
        codes, scales = O.quantize(w, c["block"], c["bits"])
        dq = O.dequantize(codes, scales, c["block"])
        assert np.array_equal(dq, np.array(c["dq"], np.float32)), (c["bits"], c["block"])
        y = O.quant_matmul_t(np.array(c["x"], np.float32), dq)
        assert np.abs(y - np.array(c["y"], np.float32)).max() <= 1e-5


def test_fp8_lut_bit_for_bit(golden_dir):
    lut = _load(golden_dir, "fp8_lut_golden.json")["lut"]
    ours = O.e4m3fn_lut()
    for i, v in enumerate(lut):
        if v is None:
            assert math.isnan(ours[i]) and i in (0x7F, 0xFF)
        else:
            assert np.float32(v).tobytes() == ours[i].tobytes(), i
    assert ours[0x7E] == 448.0 and ours[0x01] == 0.001953125


@pytest.mark.parametrize("case", ["scalar", "per_channel", "scale_shape_one"])
def test_fp8_dequant_golden(golden_dir, case):
    c = _load(golden_dir, "fp8_dequant_golden.json")[case]
    wb = np.array(c["weight_bytes"], np.uint8).reshape(c["shape"])
    got = O.fp8_dequant(wb, np.array(c["scale"], np.float32))
    assert np.abs(got.ravel() - np.array(c["expected"], np.float32)).max() <= 1e-6


def test_fp8_encode_matches_torch_cast(golden_dir):
    g = _load(golden_dir, "fp8_encode_golden.json")
    for c in g["cases"]:
        q, scale = O.fp8_quantize(np.array(c["w"], np.float32), c["per_channel"])
        assert np.array_equal(q, np.array(c["bytes"], np.uint8))
        assert np.array_equal(scale, np.array(c["scale"], np.float32))
        assert np.array_equal(O.fp8_dequant(q, scale), np.array(c["dq"], np.float32))
    b = g["boundaries"]
    assert np.array_equal(O.encode_e4m3fn(np.array(b["x"], np.float32)), np.array(b["bytes"], np.uint8))


def test_lora_toy_twenty_sgd_steps(golden_dir):
    g = _load(golden_dir, "lora_toy.json")
    i = _load(golden_dir, "lora_toy_inputs.json")
    hp = g["hyperparams"]
    w_base = np.array(i["w_base"], np.float32)  # burn layout [d_in, d_out]
    a = np.array(i["a_init"], np.float32)
    b = np.zeros((hp["rank"], hp["d_out"]), np.float32)
    x = np.array(i["x"], np.float32)
    t = np.array(i["t"], np.float32)
    s = hp["alpha"] / hp["rank"]
    losses = []
    for _ in range(hp["steps"]):
        y, _h = O.lora_linear_fwd(x, w_base.T, a, b, s)
        r = y - t
        losses.append(float((r ** 2).mean()))
        dy = (2.0 / r.size) * r
        _dx, da, db = O.lora_linear_bwd(dy, x, w_base.T, a, b, s)
        a = (a - np.float32(hp["lr"]) * da).astype(np.float32)
        b = (b - np.float32(hp["lr"]) * db).astype(np.float32)
    assert np.abs(np.array(losses) - np.array(g["losses"])).max() <= 1e-5
    assert np.abs(a.ravel() - np.array(g["lora_a_final"], np.float32)).max() <= 1e-5
    assert np.abs(b.ravel() - np.array(g["lora_b_final"], np.float32)).max() <= 1e-5
    assert np.array_equal(w_base.ravel(), np.array(g["base_final"], np.float32))


def test_roundtrip_error_bound():
    """crates/loractl-core/tests/quant.rs:191-229: |dq - w| <= scale/2 + 4*eps*absmax."""
    rng = np.random.default_rng(0)
    w = rng.uniform(-3, 3, size=(16, 96)).astype(np.float32)
    for bits in (4, 8):
        codes, scales = O.quantize(w, 32, bits)
        dq = O.dequantize(codes, scales, 32)
        absmax = np.abs(w.reshape(16, 3, 32)).max(-1, keepdims=True)
        bound = scales[:, :, None] / 2 + 4 * np.finfo(np.float32).eps * absmax
        assert (np.abs(dq - w).reshape(16, 3, 32) <= bound).all()


def test_round_half_away_and_zero_group():
    x = np.array([0.5, -0.5, 1.5, 2.5, -2.5, 0.49999997, -0.49999997, 6.5, -6.5], np.float32)
    assert O.round_half_away(x).tolist() == [1, -1, 2, 3, -3, 0, 0, 7, -7]
    w = np.zeros((2, 64), np.float32)
    w[1, 40] = 0.7
    codes, scales = O.quantize(w, 32, 4)
    assert scales[0].tolist() == [0, 0] and not codes[0].any()
    assert codes[1, 40] == 7 and np.isfinite(O.dequantize(codes, scales, 32)).all()


def test_bad_block_raises():
    with pytest.raises(ValueError, match="multiple of the quant block"):
        O.quantize(np.zeros((4, 48), np.float32), 32, 4)


def test_dequant_chunk_rows_contract():
    """crates/loractl-core/tests/quant.rs:333-349."""
    assert O.dequant_chunk_rows(8, 64, 0) == [8]
    assert O.dequant_chunk_rows(8, 64, 8 * 64 * 4) == [8]
    assert O.dequant_chunk_rows(8, 64, 8 * 64 * 4 - 1) == [4, 4]
    assert O.dequant_chunk_rows(10, 64, 3 * 64 * 4) == [3, 3, 2, 2]
    assert O.dequant_chunk_rows(5, 64, 1) == [1, 1, 1, 1, 1]
    assert O.dequant_chunk_rows(1, 64, 1) == [1]
    for m, k, cb in [(97, 64, 5000), (36864, 6144, 512 << 20)]:
        rows = O.dequant_chunk_rows(m, k, cb)
        assert sum(rows) == m and max(rows) - min(rows) <= 1
        assert all(r * k * 4 <= cb for r in rows)


def test_det_vals_lcg():
    v = O.det_vals(4, 1)
    state, want = 1, []
    for _ in range(4):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        want.append(np.float32(np.float32(state >> 8) / np.float32(1 << 24) * 2 - 1))
    assert v.tolist() == want and (np.abs(v) <= 1).all()

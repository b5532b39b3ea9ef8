"""GPU parity of quantize / pack / unpack / dequantize against the CPU oracle.

Integer work is checked bit-for-bit: codes and scales must equal the oracle's
(reference/quant_int4_reference.py:46-58 arithmetic), for int4 and int8, blocks
32 and 64, ragged row counts and partial k-tiles."""
import json

import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import dev, host, seeded

pytestmark = pytest.mark.gpu


def lb():
    import loractl_b200

    return loractl_b200


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("block", [32, 64])
@pytest.mark.parametrize("shape", [(8, 64), (16, 96), (64, 192), (130, 128), (257, 320), (1024, 1024)])
def test_codes_and_scales_bit_exact(bits, block, shape):
    m, k = shape
    if k % block:
        pytest.skip("d_in not a multiple of the block")
    w = seeded(shape, 5, 0.02)
    wq = lb().quantize_linear_weight(dev(w), bits, block)
    codes, scales = wq.unpack()
    oc, os_ = O.quantize(w, block, bits)
    assert np.array_equal(codes.cpu().numpy(), oc)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), os_.view(np.uint32))
    dq = host(wq.dequantize())
    assert np.array_equal(dq.view(np.uint32), O.dequantize(oc, os_, block).view(np.uint32))


@pytest.mark.parametrize("bits", [4, 8])
def test_full_size_site_bit_exact(bits):
    """The single-linear benchmark's weight: 3072 x 3072, N(0, 0.02), block 64."""
    w = seeded((3072, 3072), 5, 0.02)
    wq = lb().quantize_linear_weight(dev(w), bits, 64)
    codes, scales = wq.unpack()
    oc, os_ = O.quantize(w, 64, bits)
    assert np.array_equal(codes.cpu().numpy(), oc)
    assert np.array_equal(scales.cpu().numpy(), os_)
    assert wq.packed_bytes == 3072 * 3072 * bits // 8


@pytest.mark.parametrize("name,bits", [("quant_int4_golden.json", 4), ("quant_int8_golden.json", 8)])
def test_reference_goldens_through_the_gpu(golden_dir, name, bits):
    """crates/loractl-core/tests/quant.rs:96-139: dq <= 1e-6, y <= 1e-5 (f32 path)."""
    g = json.loads((golden_dir / name).read_text())
    w, x = np.array(g["w"], np.float32), np.array(g["x"], np.float32)
    wq = lb().quantize_linear_weight(dev(w), bits, g["block"])
    assert np.abs(host(wq.dequantize()) - np.array(g["dq"], np.float32)).max() <= 1e-6
    y = lb().quant_matmul_t(dev(x), wq)
    assert np.abs(host(y) - np.array(g["y"], np.float32)).max() <= 1e-5


def test_extra_goldens_blocks_32_and_64(golden_dir):
    for c in json.loads((golden_dir / "quant_extra_golden.json").read_text())["cases"]:
        w, x = np.array(c["w"], np.float32), np.array(c["x"], np.float32)
        wq = lb().quantize_linear_weight(dev(w), c["bits"], c["block"])
        assert np.array_equal(host(wq.dequantize()), np.array(c["dq"], np.float32))
        y = lb().quant_matmul_t(dev(x), wq)
        assert np.abs(host(y) - np.array(c["y"], np.float32)).max() <= 1e-5


def test_ties_round_half_away_and_zero_groups():
    w = np.zeros((4, 64), np.float32)
    w[0, :8] = [7.0, 3.5, -3.5, 0.5, -0.5, 2.5, -6.5, 1.0]  # scale 1 -> exact .5 ties
    w[2, 33] = 0.25  # rows 1, 3 and half of row 2 stay all-zero groups
    for block in (32, 64):
        wq = lb().quantize_linear_weight(dev(w), 4, block)
        codes, scales = wq.unpack()
        oc, os_ = O.quantize(w, block, 4)
        assert np.array_equal(codes.cpu().numpy(), oc) and np.array_equal(scales.cpu().numpy(), os_)
        assert codes[0, :8].tolist() == [7, 4, -4, 1, -1, 3, -7, 1]
        assert torch.isfinite(wq.dequantize()).all()


def test_bf16_weight_input_matches_oracle_on_rounded_values():
    w = seeded((64, 128), 9, 0.02)
    wb = torch.from_numpy(w).to(torch.bfloat16)
    wq = lb().quantize_linear_weight(wb.cuda(), 4, 32)
    oc, os_ = O.quantize(wb.to(torch.float32).numpy(), 32, 4)
    codes, scales = wq.unpack()
    assert np.array_equal(codes.cpu().numpy(), oc) and np.array_equal(scales.cpu().numpy(), os_)


def test_roundtrip_error_bound():
    """crates/loractl-core/tests/quant.rs:191-229."""
    rng = np.random.default_rng(1)
    w = rng.uniform(-3, 3, size=(16, 96)).astype(np.float32)
    for bits in (4, 8):
        wq = lb().quantize_linear_weight(dev(w), bits, 32)
        dq = host(wq.dequantize())
        _, scales = O.quantize(w, 32, bits)
        absmax = np.abs(w.reshape(16, 3, 32)).max(-1, keepdims=True)
        bound = scales[:, :, None] / 2 + 4 * np.finfo(np.float32).eps * absmax
        assert (np.abs(dq - w).reshape(16, 3, 32) <= bound).all()


def test_d_in_not_multiple_of_block_fails_loudly():
    """crates/loractl-core/tests/quant.rs:315-321."""
    from loractl_b200._lib import LqError

    with pytest.raises(LqError, match="multiple of the quant block"):
        lb().quantize_linear_weight(torch.zeros(4, 48, device="cuda"), 4, 32)
    with pytest.raises(LqError, match="bits"):
        lb().quantize_linear_weight(torch.zeros(4, 64, device="cuda"), 5, 32)


def test_chunked_quantize_equals_whole_tensor():
    """crates/loractl-core/tests/quant.rs:356-457: chunks are bit-identical to the same rows of
    the whole-tensor quantization, and the chunked forward is bit-identical."""
    w = seeded((97, 64), 3, 0.05)
    whole = lb().quantize_linear_weight(dev(w), 4, 32)
    chunks = lb().quantize_linear_weight_chunked(dev(w), 4, 20 * 64 * 4, 32)
    rows = lb().dequant_chunk_rows(97, 64, 20 * 64 * 4)
    assert [c.d_out for c in chunks] == rows == O.dequant_chunk_rows(97, 64, 20 * 64 * 4) and len(rows) == 5
    wc, ws = whole.unpack()
    assert torch.equal(torch.cat([c.unpack()[0] for c in chunks]), wc)
    assert torch.equal(torch.cat([c.unpack()[1] for c in chunks]), ws)
    x = dev(seeded((7, 64), 4))
    ql = lb().QuantLinear(chunks)
    assert ql.rows == rows
    assert torch.equal(ql(x), lb().quant_matmul_t(x, whole))


def test_fp8_lut_and_dequant_goldens(golden_dir):
    """crates/loractl-core/tests/fp8.rs:140-158,602-662."""
    lut = json.loads((golden_dir / "fp8_lut_golden.json").read_text())["lut"]
    allb = torch.arange(256, dtype=torch.uint8, device="cuda").reshape(16, 16)
    wq = lb().weight_from_fp8(allb, torch.ones((), device="cuda"))
    got = host(wq.dequantize()).ravel()
    host_lut = lb().e4m3fn_lut()
    for i, v in enumerate(lut):
        if v is None:
            assert np.isnan(got[i]) and np.isnan(host_lut[i])
        else:
            assert np.float32(v).tobytes() == got[i].tobytes() == np.float32(host_lut[i]).tobytes(), i
    d = json.loads((golden_dir / "fp8_dequant_golden.json").read_text())
    for case in ("scalar", "per_channel", "scale_shape_one"):
        c = d[case]
        wb = torch.tensor(c["weight_bytes"], dtype=torch.uint8, device="cuda").reshape(c["shape"])
        wq = lb().weight_from_fp8(wb, torch.tensor(c["scale"], dtype=torch.float32, device="cuda"))
        assert np.abs(host(wq.dequantize()).ravel() - np.array(c["expected"], np.float32)).max() <= 1e-6


def test_fp8_bad_scale_shape_is_an_error():
    wb = torch.zeros((5, 3), dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError, match="neither scalar nor"):
        lb().weight_from_fp8(wb, torch.ones(3, device="cuda"))


@pytest.mark.parametrize("per_channel", [False, True])
def test_fp8_quantize_bit_exact(golden_dir, per_channel):
    """reference/fp8_reference.py:84-94 on the device: bytes and scales equal the oracle's, which
    is pinned to torch's own float8_e4m3fn cast."""
    g = json.loads((golden_dir / "fp8_encode_golden.json").read_text())
    for c in g["cases"]:
        if c["per_channel"] != per_channel:
            continue
        wq = lb().fp8_quantize(dev(np.array(c["w"], np.float32)), per_channel)
        b, s = wq.unpack()
        assert np.array_equal(b.cpu().numpy(), np.array(c["bytes"], np.uint8))
        assert np.array_equal(s.cpu().numpy().ravel(), np.array(c["scale"], np.float32).ravel())
        assert np.array_equal(host(wq.dequantize()), np.array(c["dq"], np.float32))
    w = seeded((256, 384), 5, 0.02)
    wq = lb().fp8_quantize(dev(w), per_channel)
    ob, osc = O.fp8_quantize(w, per_channel)
    b, s = wq.unpack()
    assert np.array_equal(b.cpu().numpy(), ob)
    assert np.array_equal(s.cpu().numpy().ravel(), np.asarray(osc).ravel())


def test_fp8_encode_boundaries(golden_dir):
    bnd = json.loads((golden_dir / "fp8_encode_golden.json").read_text())["boundaries"]
    x = np.array(bnd["x"], np.float32)
    n = (len(x) + 15) // 16 * 16
    xp = np.zeros(n, np.float32)
    xp[: len(x)] = x
    # scale 1: make 448 the row maximum so that amax/448 == 1 exactly
    xp = np.concatenate([xp.reshape(-1, 16), np.full((n // 16, 1), 448.0, np.float32)], axis=1)
    keep = np.abs(xp) <= 448.0
    xp = np.where(keep, xp, 0.0).astype(np.float32)
    wq = lb().fp8_quantize(dev(xp), True)
    b, s = wq.unpack()
    assert (s.cpu().numpy() == 1.0).all()
    assert np.array_equal(b.cpu().numpy(), O.encode_e4m3fn(xp))


@pytest.mark.parametrize("scheme", ["int4", "int8", "fp8_scalar", "fp8_channel"])
@pytest.mark.parametrize("shape", [(128, 64), (136, 96), (264, 320), (1024, 1024)])
def test_bf16_dequantize_is_the_f32_value_rounded_once(scheme, shape):
    """The GEMM scratch holds bf16(q * scale) resp. bf16(LUT[b] * scale): the f32 product of the
    reference's dequantize (crates/loractl-core/src/quant.rs:232,250; src/fp8.rs:305-317) rounded
    to nearest even once — bit-exact against the oracle's f32 value cast to bf16."""
    m, k = shape
    w = seeded(shape, 5, 0.02)
    if scheme.startswith("int"):
        bits = 4 if scheme == "int4" else 8
        wq = lb().quantize_linear_weight(dev(w), bits, 32)
        dq = O.dequantize(*O.quantize(w, 32, bits), 32)
    else:
        if k % 16:
            pytest.skip("fp8 fast path needs d_in % 16 == 0")
        pc = scheme == "fp8_channel"
        wq = lb().fp8_quantize(dev(w), pc)
        dq = O.fp8_dequant(*O.fp8_quantize(w, pc))
    got = wq.dequantize(torch.bfloat16).cpu()
    want = torch.from_numpy(dq).to(torch.bfloat16)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))

"""The C oracle against the numpy oracle (itself pinned to the reference's goldens): integer
work bit-for-bit, the f32 linear to summation-order rounding."""
import json

import numpy as np
import pytest

from oracle import c_binding as OC
from oracle import lq_oracle as O
from tests.util import seeded


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("group", [32, 64])
def test_c_quantize_bit_exact(bits, group):
    w = seeded((33, 192), 5, 0.02)
    w[3, :64] = 0.0
    w[4, :4] = [3.5, -3.5, 7.0, 0.5]
    c1, s1 = OC.quantize(w, group, bits)
    c2, s2 = O.quantize(w, group, bits)
    assert np.array_equal(c1, c2) and np.array_equal(s1, s2)
    assert np.array_equal(OC.dequantize(c1, s1, group), O.dequantize(c2, s2, group))
    with pytest.raises(ValueError):
        OC.quantize(np.zeros((2, 48), np.float32), 32, 4)


def test_c_goldens(golden_dir):
    for name, bits in (("quant_int4_golden.json", 4), ("quant_int8_golden.json", 8)):
        g = json.loads((golden_dir / name).read_text())
        w, x = np.array(g["w"], np.float32), np.array(g["x"], np.float32)
        codes, scales = OC.quantize(w, 32, bits)
        assert np.abs(OC.dequantize(codes, scales, 32) - np.array(g["dq"], np.float32)).max() <= 1e-6
        y, _ = OC.lora_linear_fwd(x, codes, scales, 32, None, None, 1.0)
        assert np.abs(y - np.array(g["y"], np.float32)).max() <= 1e-5
    lut = json.loads((golden_dir / "fp8_lut_golden.json").read_text())["lut"]
    ours = OC.e4m3fn_lut()
    for i, v in enumerate(lut):
        assert (np.isnan(ours[i]) if v is None else np.float32(v).tobytes() == ours[i].tobytes())
    d = json.loads((golden_dir / "fp8_dequant_golden.json").read_text())
    for case in d.values():
        wb = np.array(case["weight_bytes"], np.uint8).reshape(case["shape"])
        got = OC.fp8_dequant(wb, np.array(case["scale"], np.float32))
        assert np.abs(got.ravel() - np.array(case["expected"], np.float32)).max() <= 1e-6


def test_c_chunk_rows_and_linear():
    for args in [(8, 64, 0), (10, 64, 3 * 64 * 4), (97, 64, 5000), (36864, 6144, 512 << 20)]:
        assert OC.dequant_chunk_rows(*args) == O.dequant_chunk_rows(*args)
    n, k, m, r = 37, 128, 96, 8
    w, x, dy = seeded((m, k), 5, 0.02), seeded((n, k), 6), seeded((n, m), 9)
    a, b, bias = seeded((k, r), 7, 0.1), seeded((r, m), 8, 0.01), seeded((m,), 10)
    codes, scales = O.quantize(w, 64, 4)
    dq = O.dequantize(codes, scales, 64)
    y, h = OC.lora_linear_fwd(x, codes, scales, 64, a, b, 2.0, bias)
    oy, oh = O.lora_linear_fwd(x, dq, a, b, 2.0, bias)
    assert O.rel_deviation(y, oy) <= 1e-5 and O.rel_deviation(h, oh) <= 1e-5
    dx, da, db = OC.lora_linear_bwd(dy, x, h, codes, scales, 64, a, b, 2.0)
    odx, oda, odb = O.lora_linear_bwd(dy, x, dq, a, b, 2.0)
    assert O.rel_deviation(dx, odx) <= 1e-5 and O.rel_deviation(da, oda) <= 1e-5 and O.rel_deviation(db, odb) <= 1e-5

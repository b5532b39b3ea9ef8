"""The frozen int4 GEMM with the dequantisation inside the mainloop (no bf16 weight copy in HBM).

Three properties are pinned:
  * with the exact conversion the in-mainloop path is BIT-IDENTICAL, forward and backward, to the
    path that first dequantises the weight into a bf16 scratch (same operand values, same tiles,
    same accumulation order) — so every parity result of the scratch path carries over;
  * with the two-instruction conversion, w = bf16(q * bf16(scale)), it stays inside the bf16 band
    against the f32 oracle (Y, dX <= 6e-3 of the output's peak, cosine >= 0.9999);
  * ragged shapes (a half-empty CTA pair, d_in with 64 or 128 columns left over, token counts that
    are not tile multiples), both quant block sizes, bias, rank 0 and rank > 64.
"""
import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import bf16_round, dev, host, reldev, seeded

pytestmark = pytest.mark.gpu


def lb():
    import loractl_b200

    return loractl_b200


def set_option(name, value):
    from loractl_b200 import _lib as L

    L.check(L.lib().lq_option_set(name.encode(), int(value)))


@pytest.fixture(autouse=True)
def w4_on_for_these_tests():
    """The in-mainloop path is an option (off by default: the scratch-copy path measured faster at
    every size tried); these tests switch it on and restore the defaults afterwards."""
    set_option("w4", 1)
    set_option("w4_exact", 1)
    set_option("tail_split", 0)  # the scratch path's k-cut of a thin last round changes its summation order
    yield
    set_option("w4", 0)
    set_option("w4_exact", 1)
    set_option("tail_split", 1)


def case(n, k, m, r, block, seed=5):
    w = seeded((m, k), seed, 0.02)
    x = bf16_round(seeded((n, k), seed + 1))
    dy = bf16_round(seeded((n, m), seed + 4))
    a = seeded((k, r), seed + 2, 1.0 / np.sqrt(k)) if r else None
    b = seeded((r, m), seed + 3, 0.01) if r else None
    wq = lb().quantize_linear_weight(dev(w), 4, block)
    dq = O.dequantize(*O.quantize(w, block, 4), block)
    return wq, dq, x, dy, a, b


def run(wq, x, dy, a, b, s):
    from loractl_b200 import quant as Q

    xd, dyd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16)
    ad = dev(a) if a is not None else None
    bd = dev(b) if b is not None else None
    y, h = Q.linear_fwd_raw(wq, xd, ad, bd, s)
    dx, da, db = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, s)
    lb().check_device_status()
    return y, dx, da, db


SHAPES = [
    # n, k, m, r, block
    (256, 256, 256, 16, 64),
    (130, 320, 384, 8, 64),     # ragged tokens; d_in leaves one 64-column tile; d_out half-fills the last pair
    (300, 448, 640, 16, 32),    # block 32: two scale groups per packed k-tile
    (1024, 768, 768, 8, 64),    # the text model's attention projections
    (513, 512, 1032, 80, 64),   # rank > 64: two extension k-blocks; d_out not a multiple of 128
    (2048, 3072, 3072, 0, 64),  # base only (exact quant_matmul_t semantics)
]


@pytest.mark.parametrize("n,k,m,r,block", SHAPES)
def test_exact_conversion_is_bit_identical_to_the_scratch_path(n, k, m, r, block):
    wq, dq, x, dy, a, b = case(n, k, m, r, block)
    bias = seeded((m,), 10, 0.1)
    wq.set_bias(dev(bias))
    set_option("w4", 0)
    ref = run(wq, x, dy, a, b, 2.0)
    set_option("w4", 1)
    set_option("w4_exact", 1)
    got = run(wq, x, dy, a, b, 2.0)
    assert torch.equal(got[0], ref[0]), "Y differs from the scratch path"
    assert torch.equal(got[1], ref[1]), "dX differs from the scratch path"
    if r:
        assert torch.equal(got[2], ref[2]) and torch.equal(got[3], ref[3])
    oy, _ = O.lora_linear_fwd(x, dq, a, b, 2.0, bias)
    odx = O.lora_linear_bwd(dy, x, dq, a, b, 2.0)[0]
    assert reldev(host(got[0]), oy) <= 6e-3 and reldev(host(got[1]), odx) <= 6e-3


@pytest.mark.parametrize("mode", [0, 2])
@pytest.mark.parametrize("n,k,m,r,block", SHAPES[:5])
def test_cheaper_conversions_stay_in_the_bf16_band(n, k, m, r, block, mode):
    wq, dq, x, dy, a, b = case(n, k, m, r, block)
    set_option("w4_exact", mode)
    y, dx, da, db = run(wq, x, dy, a, b, 2.0)
    oy, _ = O.lora_linear_fwd(x, dq, a, b, 2.0)
    odx, oda, odb = O.lora_linear_bwd(dy, x, dq, a, b, 2.0)
    assert torch.isfinite(y).all() and torch.isfinite(dx).all()
    assert reldev(host(y), oy) <= 6e-3 and O.cosine(host(y), oy) >= 0.9999
    assert reldev(host(dx), odx) <= 6e-3 and O.cosine(host(dx), odx) >= 0.9999
    assert reldev(host(da), oda) <= 8e-3 and reldev(host(db), odb) <= 8e-3


def test_in_mainloop_path_is_deterministic_and_zero_b_is_a_no_op():
    """Recompute under block checkpointing replays the forward: it must reproduce it bit for bit
    (crates/loractl-core/tests/block_ckpt.rs:236-283); a zero-initialised B must not change a bit
    of the base output (crates/loractl-core/tests/quant_mmdit.rs:228-255)."""
    from loractl_b200 import quant as Q

    wq, dq, x, dy, a, b = case(384, 512, 768, 16, 64)
    xd, dyd, ad, bd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16), dev(a), dev(b)
    y0, _ = Q.linear_fwd_raw(wq, xd, None, None, 1.0)
    y1, _ = Q.linear_fwd_raw(wq, xd, ad, torch.zeros_like(bd), 1.0)
    assert torch.equal(y0, y1)
    ya, ha = Q.linear_fwd_raw(wq, xd, ad, bd, 1.0)
    yb, _ = Q.linear_fwd_raw(wq, xd, ad, bd, 1.0)
    assert torch.equal(ya, yb)
    g1 = Q.linear_bwd_raw(wq, dyd, xd, ha, ad, bd, 1.0)
    g2 = Q.linear_bwd_raw(wq, dyd, xd, ha, ad, bd, 1.0)
    assert all(torch.equal(p, q) for p, q in zip(g1, g2))
    lb().check_device_status()


def test_split_scale_conversion_is_as_close_to_the_oracle_as_the_exact_one():
    """w = fma(q, s_hi, bf16(q * s_lo)) rounds q * scale once except within 2^-18 of a rounding
    boundary, so its deviation from the f32 oracle must equal the exact conversion's to three digits."""
    wq, dq, x, dy, _, _ = case(1024, 1024, 1024, 0, 64)
    oy, _ = O.lora_linear_fwd(x, dq, None, None, 1.0)
    devs = {}
    for mode in (1, 2, 0):
        set_option("w4_exact", mode)
        y, _, _, _ = run(wq, x, dy, None, None, 1.0)
        devs[mode] = reldev(host(y), oy)
    assert abs(devs[2] - devs[1]) <= 0.02 * devs[1], devs
    assert devs[0] <= 6e-3, devs


def test_unknown_option_is_refused():
    from loractl_b200 import _lib as L

    assert L.lib().lq_option_set(b"no_such_switch", 1) == L.LQ_ERR_INVALID

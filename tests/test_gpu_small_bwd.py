"""GPU parity of the small-batch backward (N <= 16 tokens, int4, quant block 64 or 32): dX over the packed weight
stream with the nibbles converted in registers, dH / dA / dB formed by the same two launches.

Tolerance: the bf16 path's band — dX within 6e-3 of its peak against the f32 oracle on the same
bf16-rounded inputs (inside the kernel the integer codes are exact; dY * scale is rounded to bf16
once per element), cosine >= 0.9999; dA, dB within 2e-3 of their peaks (f32 arithmetic throughout,
only the inputs are bf16).  The same shapes through the tensor-regime backward (the environment
switch that disables this path is read once per process, so the comparison is against the oracle
only) are covered by tests/test_gpu_tc.py."""
import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import bf16_round, dev, host, reldev, seeded

pytestmark = pytest.mark.gpu


def lb():
    import loractl_b200

    return loractl_b200


def case(n, k, m, r, seed=5, block=64):
    w = seeded((m, k), seed, 0.02)
    x = bf16_round(seeded((n, k), seed + 1))
    dy = bf16_round(seeded((n, m), seed + 4))
    a = seeded((k, r), seed + 2, 1.0 / np.sqrt(k)) if r else None
    b = seeded((r, m), seed + 3, 0.01) if r else None
    wq = lb().quantize_linear_weight(dev(w), 4, block)
    dq = O.dequantize(*O.quantize(w, block, 4), block)
    return wq, dq, x, dy, a, b


SHAPES = [
    # k (d_in), m (d_out)
    (64, 128),      # one k-tile: three of the four consumer warps idle
    (320, 264),     # 5 k-tiles (a ragged last chunk), d_out not a multiple of 128 (zero-filled dY columns)
    (1024, 768),
    (3072, 2056),   # many splits over the m-tiles; several partial dH rows per token
]


@pytest.mark.parametrize("block", [64, 32])
@pytest.mark.parametrize("n", [1, 3, 8, 11, 16])
@pytest.mark.parametrize("k,m", SHAPES)
@pytest.mark.parametrize("r", [0, 4, 32])
def test_small_batch_backward_matches_oracle(n, k, m, r, block):
    from loractl_b200 import quant as Q

    wq, dq, x, dy, a, b = case(n, k, m, r, block=block)
    xd, dyd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16)
    ad, bd = (dev(a), dev(b)) if r else (None, None)
    _, h = Q.linear_fwd_raw(wq, xd, ad, bd, 2.0)
    dx, da, db = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 2.0)
    lb().check_device_status()
    odx, oda, odb = O.lora_linear_bwd(dy, x, dq, a, b, 2.0)
    assert dx.shape == (n, k) and torch.isfinite(dx).all()
    assert reldev(host(dx), odx) <= 6e-3
    if n * k >= 1024:
        assert O.cosine(host(dx), odx) >= 0.9999
    if r:
        assert reldev(host(da), oda) <= 2e-3 and reldev(host(db), odb) <= 2e-3


def test_recomputed_h_accumulate_and_partial_outputs():
    """H not kept by the caller is recomputed from X and A; `accumulate` adds into dA / dB; a call that
    wants only some of the outputs leaves the others alone."""
    from loractl_b200 import quant as Q

    wq, dq, x, dy, a, b = case(5, 1024, 768, 16)
    xd, dyd, ad, bd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16), dev(a), dev(b)
    _, h = Q.linear_fwd_raw(wq, xd, ad, bd, 0.5)
    ref = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 0.5)
    no_h = Q.linear_bwd_raw(wq, dyd, xd, None, ad, bd, 0.5)
    assert torch.equal(ref[0], no_h[0]) and torch.equal(ref[1], no_h[1])
    assert reldev(host(no_h[2]), host(ref[2])) <= 1e-5  # H recomputed in f32 from the same bf16 X
    # accumulate: twice the gradient on top of a known start
    da0, db0 = torch.full_like(ref[1], 0.25), torch.full_like(ref[2], -0.5)
    Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 0.5, da_out=da0, db_out=db0, accumulate=True)
    assert torch.allclose(da0, ref[1] + 0.25, rtol=0, atol=1e-6) and torch.allclose(db0, ref[2] - 0.5, rtol=0, atol=1e-6)
    # only dX; only the adapter gradients
    dx_only = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 0.5, need_da=False, need_db=False)
    assert torch.equal(dx_only[0], ref[0]) and dx_only[1] is None and dx_only[2] is None
    g_only = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 0.5, need_dx=False)
    assert g_only[0] is None and torch.equal(g_only[1], ref[1]) and torch.equal(g_only[2], ref[2])
    lb().check_device_status()


def test_modulation_site_full_size_and_determinism():
    """The adaLN modulation projection of the benchmark block (3072 -> 18432, rank 32) at 1 and 8 tokens."""
    from loractl_b200 import quant as Q

    wq, dq, x, dy, a, b = case(8, 3072, 18432, 32)
    ad, bd = dev(a), dev(b)
    for n in (8, 1):
        xd, dyd = dev(x[:n], torch.bfloat16), dev(dy[:n], torch.bfloat16)
        _, h = Q.linear_fwd_raw(wq, xd, ad, bd, 1.0)
        g1 = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 1.0)
        g2 = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 1.0)
        lb().check_device_status()
        assert all(torch.equal(p, q) for p, q in zip(g1, g2))
        odx, oda, odb = O.lora_linear_bwd(dy[:n], x[:n], dq, a, b, 1.0)
        assert reldev(host(g1[0]), odx) <= 6e-3 and O.cosine(host(g1[0]), odx) >= 0.9999
        assert reldev(host(g1[1]), oda) <= 2e-3 and reldev(host(g1[2]), odb) <= 2e-3


def test_zero_upstream_gradient_gives_zeros():
    """Zero dY must give exact zeros (the +136 offset of the code words cancels exactly)."""
    from loractl_b200 import quant as Q

    wq, dq, x, dy, a, b = case(4, 320, 264, 8)
    xd, ad, bd = dev(x, torch.bfloat16), dev(a), dev(b)
    _, h = Q.linear_fwd_raw(wq, xd, ad, bd, 1.0)
    dx, da, db = Q.linear_bwd_raw(wq, torch.zeros((4, 264), dtype=torch.bfloat16, device="cuda"), xd, h, ad, bd, 1.0)
    assert not dx.any() and not da.any() and not db.any()

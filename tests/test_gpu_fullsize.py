"""Parity at the headline benchmark's full size: scaled-fp8 3072 -> 12288 weight with per-output-channel
scales, LoRA rank 32, 8192 bf16 tokens, forward and backward, through the C ABI, for both compute
types (bf16 and native e4m3).

The oracle runs on the same seeded inputs.  The two frozen contractions (Y and dX) are row-separable
in the token index, so the oracle evaluates them on a seeded subset of 192 tokens only (seconds of
CPU time); everything that reduces over tokens (dA, dB) or is small (H) is evaluated in full.  The
fp8 repack of the whole weight is bit-exact against the oracle.  Tolerances are the ones stated in
test_gpu_tc.py (bf16) and test_gpu_w8a8.py (native fp8)."""
import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import bf16_round, dev, host, reldev, seeded

pytestmark = pytest.mark.gpu

N, K, M, R, S = 8192, 3072, 12288, 32, 1.0


@pytest.fixture(scope="module")
def case():
    import loractl_b200 as lb

    w = seeded((M, K), 5, 0.02)
    wb, sc = O.fp8_quantize(w, per_channel=True)
    wq = lb.fp8_quantize(dev(w), True)
    x = bf16_round(seeded((N, K), 6))
    dy = bf16_round(seeded((N, M), 9))
    a = seeded((K, R), 7, 1.0 / np.sqrt(K))
    b = seeded((R, M), 8, 0.01)
    dq = O.fp8_dequant(wb, sc)
    rows = np.sort(np.random.default_rng(3).choice(N, 192, replace=False))
    # oracle: H, dH, dA, dB in full; Y and dX on the token subset
    h = (x @ a).astype(np.float32)
    dh = (S * (dy @ b.T)).astype(np.float32)
    ref = {
        "wb": wb, "sc": sc, "rows": rows, "h": h,
        "y": (x[rows] @ dq.T + S * (h[rows] @ b)).astype(np.float32),
        "dx": (dy[rows] @ dq + dh[rows] @ a.T).astype(np.float32),
        "da": (x.T @ dh).astype(np.float32),
        "db": (S * (h.T @ dy)).astype(np.float32),
    }
    return wq, x, dy, a, b, ref


def test_full_size_fp8_repack_is_bit_exact(case):
    wq, *_, ref = case
    assert (wq.d_out, wq.d_in) == (M, K)
    assert np.array_equal(host(wq.dequantize(torch.float32)), O.fp8_dequant(ref["wb"], ref["sc"]))


@pytest.mark.parametrize("fp8_compute", [False, True])
def test_full_size_forward_backward(case, fp8_compute):
    import loractl_b200 as lb
    from loractl_b200 import quant as Q

    wq, x, dy, a, b, ref = case
    band, gband = (5e-2, 8e-3) if fp8_compute else (6e-3, 8e-3)
    cos = 0.999 if fp8_compute else 0.9999
    if fp8_compute:
        wq.prepare_fp8_backward()
    xd, dyd, ad, bd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16), dev(a), dev(b)
    rows = torch.from_numpy(ref["rows"]).to("cuda")
    y, h = Q.linear_fwd_raw(wq, xd, ad, bd, S, fp8_compute=fp8_compute)
    lb.check_device_status()
    ys = host(y[rows])
    assert reldev(ys, ref["y"]) <= band and O.cosine(ys, ref["y"]) >= cos
    assert reldev(host(h), ref["h"]) <= 6e-3
    assert bool(torch.isfinite(y).all())
    dx, da, db = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, S, fp8_compute=fp8_compute)
    lb.check_device_status()
    dxs = host(dx[rows])
    assert reldev(dxs, ref["dx"]) <= band and O.cosine(dxs, ref["dx"]) >= cos
    assert reldev(host(da), ref["da"]) <= gband and reldev(host(db), ref["db"]) <= gband
    assert bool(torch.isfinite(dx).all())
    # the step is deterministic: a second run is bit-identical
    y2, h2 = Q.linear_fwd_raw(wq, xd, ad, bd, S, fp8_compute=fp8_compute)
    dx2, da2, db2 = Q.linear_bwd_raw(wq, dyd, xd, h2, ad, bd, S, fp8_compute=fp8_compute)
    assert torch.equal(y, y2) and torch.equal(dx, dx2) and torch.equal(da, da2) and torch.equal(db, db2)

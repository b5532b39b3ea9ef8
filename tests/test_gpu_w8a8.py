"""GPU tests of native fp8 compute (LQ_BF16_W8A8): the stored e4m3 weight bytes are the MMA
operand (tcgen05 kind::f8f6f4), activations are quantised to e4m3 per token, scales are applied in
the epilogue and the LoRA extension stays bf16.

The reference has no fp8 compute (crates/loractl-core/src/fp8.rs only decodes), so the oracle is
"dequantize the fp8 weight to f32, then f32 matmul" on the same bf16-rounded activations, and the
tolerance is the one an e4m3 activation (3 mantissa bits) allows: Y and dX within 5e-2 of the
output's peak with cosine >= 0.999 — the same order as the reference's own fp8 accuracy gate
(d_bar 1.55e-2, ceil 4e-2, crates/loractl-core/tests/reduced_precision_accuracy.rs:44-63, which
covers weight-only fp8).  dA and dB never pass through 8 bits: they keep the bf16 band (8e-3)."""
import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import bf16_round, dev, host, reldev, seeded

pytestmark = pytest.mark.gpu


def lb():
    import loractl_b200

    return loractl_b200


def case(n, k, m, r, per_channel):
    w = seeded((m, k), 5, 0.02)
    x, dy = bf16_round(seeded((n, k), 6)), bf16_round(seeded((n, m), 9))
    a = seeded((k, r), 7, 1.0 / np.sqrt(k)) if r else None
    b = seeded((r, m), 8, 0.01) if r else None
    wq = lb().fp8_quantize(dev(w), per_channel)
    dq = O.fp8_dequant(*O.fp8_quantize(w, per_channel))
    return wq, dq, x, dy, a, b


@pytest.mark.parametrize("n,k,m,r", [(256, 256, 512, 16), (300, 512, 784, 8), (64, 128, 144, 4),
                                     (1024, 1024, 1024, 32), (513, 384, 1040, 80), (4096, 3072, 3072, 32)])
@pytest.mark.parametrize("per_channel", [True, False])
def test_w8a8_matches_oracle(n, k, m, r, per_channel):
    from loractl_b200 import quant as Q

    if n >= 4096 and not per_channel:
        pytest.skip("full-size case once")
    wq, dq, x, dy, a, b = case(n, k, m, r, per_channel)
    bias = seeded((m,), 10, 0.1)
    wq.set_bias(dev(bias))
    s = 2.0
    xd, dyd, ad, bd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16), dev(a), dev(b)
    y, h = Q.linear_fwd_raw(wq, xd, ad, bd, s, fp8_compute=True)
    lb().check_device_status()
    oy, oh = O.lora_linear_fwd(x, dq, a, b, s, bias)
    assert torch.isfinite(y).all()
    assert reldev(host(y), oy) <= 5e-2 and O.cosine(host(y), oy) >= 0.999
    assert reldev(host(h), oh) <= 6e-3
    wq.prepare_fp8_backward()
    dx, da, db = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, s, fp8_compute=True)
    lb().check_device_status()
    odx, oda, odb = O.lora_linear_bwd(dy, x, dq, a, b, s)
    assert reldev(host(dx), odx) <= 5e-2 and O.cosine(host(dx), odx) >= 0.999
    assert reldev(host(da), oda) <= 8e-3 and reldev(host(db), odb) <= 8e-3


def test_w8a8_base_only_zero_b_identity_and_determinism():
    from loractl_b200 import quant as Q

    wq, dq, x, dy, a, b = case(300, 256, 528, 16, True)
    xd, dyd, ad, bd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16), dev(a), dev(b)
    y0, _ = Q.linear_fwd_raw(wq, xd, None, None, 1.0, fp8_compute=True)
    assert reldev(host(y0), O.lora_linear_fwd(x, dq)[0]) <= 5e-2
    yz, _ = Q.linear_fwd_raw(wq, xd, ad, torch.zeros_like(bd), 1.0, fp8_compute=True)
    assert torch.equal(y0, yz)  # zero-initialised B adds exact zeros to the accumulator
    y1, h1 = Q.linear_fwd_raw(wq, xd, ad, bd, 1.0, fp8_compute=True)
    y2, h2 = Q.linear_fwd_raw(wq, xd, ad, bd, 1.0, fp8_compute=True)
    assert torch.equal(y1, y2) and torch.equal(h1, h2)
    g1 = Q.linear_bwd_raw(wq, dyd, xd, h1, ad, bd, 1.0, fp8_compute=True)
    g2 = Q.linear_bwd_raw(wq, dyd, xd, h1, ad, bd, 1.0, fp8_compute=True)
    assert all(torch.equal(p, q) for p, q in zip(g1, g2))
    dx0, _, _ = Q.linear_bwd_raw(wq, dyd, None, None, None, None, 1.0, fp8_compute=True)
    assert reldev(host(dx0), O.lora_linear_bwd(dy, x, dq)[0]) <= 5e-2


def test_w8a8_is_refused_for_int_weights_and_f32_activations():
    from loractl_b200 import quant as Q
    from loractl_b200._lib import LqError

    w4 = lb().quantize_linear_weight(dev(seeded((64, 64), 5, 0.02)), 4, 32)
    with pytest.raises(LqError, match="scaled-fp8 weight"):
        Q.linear_fwd_raw(w4, torch.zeros((8, 64), device="cuda", dtype=torch.bfloat16), None, None, 1.0,
                         fp8_compute=True)
    w8 = lb().fp8_quantize(dev(seeded((64, 64), 5, 0.02)), True)
    with pytest.raises(TypeError, match="bf16 activations"):
        Q.linear_fwd_raw(w8, torch.zeros((8, 64), device="cuda"), None, None, 1.0, fp8_compute=True)


def test_w8a8_per_channel_scales_are_applied_to_the_right_channels():
    """The global band (5e-2 of the output's peak) could hide a wrong scale on a few output channels.
    Give the channels scales spread over three orders of magnitude and check every output column of Y
    (scale applied in the epilogue) and every column of dX with a one-hot dY (scale folded into dY on
    the reduction axis) against the oracle, each column normalised by ITS OWN peak."""
    from loractl_b200 import quant as Q

    n, k, m = 256, 256, 512
    rng = np.random.default_rng(3)
    row_gain = np.exp(rng.uniform(np.log(1e-2), np.log(10.0), size=(m, 1))).astype(np.float32)
    w = seeded((m, k), 5, 0.02) * row_gain  # per-channel absmax, hence scale, varies 1000-fold
    x = bf16_round(seeded((n, k), 6))
    wq = lb().fp8_quantize(dev(w), True)
    dq = O.fp8_dequant(*O.fp8_quantize(w, True))
    xd = dev(x, torch.bfloat16)
    y, _ = Q.linear_fwd_raw(wq, xd, None, None, 1.0, fp8_compute=True)
    oy, _ = O.lora_linear_fwd(x, dq, None, None, 1.0)
    yh = host(y)
    col_peak = np.abs(oy).max(axis=0)
    col_dev = np.abs(yh - oy).max(axis=0) / col_peak
    assert col_dev.max() <= 8e-2, (int(col_dev.argmax()), float(col_dev.max()))
    # backward: dY selects one output channel per token, so row n of dX is s_w[c] * W8[c, :] for c = n % m
    dy = np.zeros((n, m), np.float32)
    dy[np.arange(n), (np.arange(n) * 2) % m] = 1.0
    wq.prepare_fp8_backward()
    dx, _, _ = Q.linear_bwd_raw(wq, dev(dy, torch.bfloat16), xd, None, None, None, 1.0, fp8_compute=True)
    lb().check_device_status()
    odx = O.lora_linear_bwd(dy, x, dq)[0]
    dxh = host(dx)
    row_peak = np.abs(odx).max(axis=1)
    row_dev = np.abs(dxh - odx).max(axis=1) / row_peak
    assert row_dev.max() <= 8e-2, (int(row_dev.argmax()), float(row_dev.max()))

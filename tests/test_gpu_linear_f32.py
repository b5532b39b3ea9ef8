"""GPU parity of the f32-arithmetic LoRA linear (forward and backward) against the CPU oracle.

Tolerance: the path computes in f32 with FMA accumulation; the oracle is numpy f32.  They
differ only by summation order, so results must agree to 2e-5 of the output's peak
(crates/loractl-core/tests/quant.rs:464-539 uses the same peak-normalised 1e-5-class bound)."""
import json

import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import dev, host, reldev, seeded

pytestmark = pytest.mark.gpu
TOL = 2e-5


def lb():
    import loractl_b200

    return loractl_b200


def make_case(n, k, m, r, bits=4, block=32, bias=False, scheme="int"):
    w = seeded((m, k), 5, 0.02)
    x = seeded((n, k), 6)
    a = seeded((k, r), 7, 1.0 / np.sqrt(k)) if r else None
    b = seeded((r, m), 8, 0.01) if r else None
    dy = seeded((n, m), 9)
    bv = seeded((m,), 10, 0.1) if bias else None
    if scheme == "int":
        wq = lb().quantize_linear_weight(dev(w), bits, block)
        codes, scales = O.quantize(w, block, bits)
        dq = O.dequantize(codes, scales, block)
    else:
        wq = lb().fp8_quantize(dev(w), scheme == "fp8_channel")
        dq = O.fp8_dequant(*O.fp8_quantize(w, scheme == "fp8_channel"))
    if bv is not None:
        wq.set_bias(dev(bv))
    return wq, dq, x, a, b, dy, bv


@pytest.mark.parametrize("n,k,m,r", [(4, 64, 8, 0), (5, 64, 96, 4), (1, 64, 96, 2), (37, 96, 130, 16),
                                     (130, 320, 257, 8), (256, 512, 384, 32)])
@pytest.mark.parametrize("bits,block", [(4, 32), (4, 64), (8, 32)])
def test_forward_backward_match_oracle(n, k, m, r, bits, block):
    if k % block:
        pytest.skip("d_in not a multiple of the block")
    from loractl_b200 import quant as Q

    wq, dq, x, a, b, dy, bv = make_case(n, k, m, r, bits, block, bias=(m % 2 == 0))
    s = 2.0
    xd, dyd = dev(x), dev(dy)
    ad, bd = (dev(a), dev(b)) if r else (None, None)
    y, h = Q.linear_fwd_raw(wq, xd, ad, bd, s)
    oy, oh = O.lora_linear_fwd(x, dq, a, b, s, bv)
    assert reldev(host(y), oy) <= TOL
    if r:
        assert reldev(host(h), oh) <= TOL
    dx, da, db = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, s)
    odx, oda, odb = O.lora_linear_bwd(dy, x, dq, a, b, s)
    assert reldev(host(dx), odx) <= TOL
    if r:
        assert reldev(host(da), oda) <= TOL and reldev(host(db), odb) <= TOL
        # H = NULL recomputes X . A inside the backward
        dx2, da2, db2 = Q.linear_bwd_raw(wq, dyd, xd, None, ad, bd, s)
        assert torch.equal(dx2, dx) and torch.equal(da2, da) and reldev(host(db2), odb) <= TOL


@pytest.mark.parametrize("scheme", ["fp8_scalar", "fp8_channel"])
def test_fp8_forward_backward_match_oracle(scheme):
    from loractl_b200 import quant as Q

    wq, dq, x, a, b, dy, bv = make_case(33, 96, 72, 8, scheme=scheme)
    y, h = Q.linear_fwd_raw(wq, dev(x), dev(a), dev(b), 1.0)
    oy, _ = O.lora_linear_fwd(x, dq, a, b, 1.0)
    assert reldev(host(y), oy) <= TOL
    dx, da, db = Q.linear_bwd_raw(wq, dev(dy), dev(x), h, dev(a), dev(b), 1.0)
    odx, oda, odb = O.lora_linear_bwd(dy, x, dq, a, b, 1.0)
    assert reldev(host(dx), odx) <= TOL and reldev(host(da), oda) <= TOL and reldev(host(db), odb) <= TOL


def test_custom_op_equals_matmul_over_dequantized_weight(golden_dir):
    """crates/loractl-core/tests/quant.rs:258-311: forward and dX of the op over the still-quantized
    weight equal the same kernel over the pre-dequantized constant (here: to summation order,
    since the latter runs in torch)."""
    g = json.loads((golden_dir / "quant_int4_golden.json").read_text())
    w, x = dev(np.array(g["w"], np.float32)), dev(np.array(g["x"], np.float32))
    wq = lb().quantize_linear_weight(w, 4, 32)
    x1 = x.clone().requires_grad_(True)
    y1 = lb().quant_matmul_t(x1, wq)
    (y1 * y1).sum().backward()
    x2 = x.clone().requires_grad_(True)
    y2 = x2 @ wq.dequantize().T
    (y2 * y2).sum().backward()
    assert reldev(host(y1), host(y2)) <= TOL and reldev(host(x1.grad), host(x2.grad)) <= TOL


def test_zero_init_lora_is_bit_identical_noop():
    """crates/loractl-core/tests/quant_mmdit.rs:228-255."""
    w = seeded((96, 64), 5, 0.02)
    lin = torch.nn.Linear(64, 96, bias=True).cuda()
    with torch.no_grad():
        lin.weight.copy_(dev(w))
    base = lb().BaseLinear.quant(lb().QuantLinear.from_linear(lin, 4))
    ad = lb().build_adapters([lb().LoraSite("blocks.0.attn.wq", 64, 96)],
                             lb().LoraConfig(rank=4, alpha=4.0, targets=[lb().TargetSpec(r"attn\.wq$")]), "cuda")
    assert ad.targets == ["blocks.0.attn.wq"] and float(ad.deltas[0].lora_b.abs().max()) == 0.0
    x = dev(seeded((2, 5, 64), 6))
    plain = lb().site(None, "blocks.0.attn.wq", base, x)
    adapted = lb().site(ad, "blocks.0.attn.wq", base, x)
    other = lb().site(ad, "blocks.0.attn.wk", base, x)
    assert plain.shape == (2, 5, 96)
    assert torch.equal(plain, adapted) and torch.equal(plain, other)


def test_one_step_moves_b_off_zero_and_grads_are_finite():
    """crates/loractl-core/tests/quant_mmdit.rs:257-313."""
    lin = torch.nn.Linear(64, 96, bias=False).cuda()
    mod = lb().LoraLinear(lb().QuantLinear.from_linear(lin, 4), rank=4, alpha=8.0, device="cuda")
    opt = torch.optim.Adam([mod.lora_a, mod.lora_b], lr=1e-2)
    x = dev(seeded((9, 64), 6))
    t = dev(seeded((9, 96), 7))
    loss = ((mod(x) - t) ** 2).mean()
    loss.backward()
    assert torch.isfinite(mod.lora_a.grad).all() and torch.isfinite(mod.lora_b.grad).all()
    assert float(mod.lora_a.grad.abs().max()) == 0.0  # B == 0 => dA == 0 at step 0
    assert float(mod.lora_b.grad.abs().max()) > 0.0
    opt.step()
    assert float(mod.lora_b.abs().max()) > 0.0


def test_lora_toy_twenty_sgd_steps_on_the_gpu(golden_dir):
    """crates/loractl-core/tests/lora_reference.rs:49-122: 20 SGD steps of
    `base(x) + s.B(A(x))` against the torch golden, through the fused kernel and autograd.
    The 4 x 3 toy is embedded in a quantizable 64-wide problem: the toy's base weights are
    multiples of 0.05, so int8 codes round(100 W) with scale 0.01 hold them (to one f32
    rounding of 0.01 q), and the zero padding contributes exact zeros."""
    from loractl_b200 import quant as Q

    g = json.loads((golden_dir / "lora_toy.json").read_text())
    i = json.loads((golden_dir / "lora_toy_inputs.json").read_text())
    hp = g["hyperparams"]
    k, m = 64, 8
    wt = np.array(i["w_base"], np.float32).T  # [d_out, d_in]
    codes = np.zeros((m, k), np.int8)
    codes[:3, :4] = np.round(wt * 100).astype(np.int8)
    scales = np.full((m, k // 32), 0.01, np.float32)
    wq = Q.weight_from_codes(dev(codes, torch.int8), dev(scales), 32, 8)
    a = np.zeros((k, 2), np.float32)
    a[:4] = np.array(i["a_init"], np.float32)
    b = np.zeros((2, m), np.float32)
    x = np.zeros((5, k), np.float32)
    x[:, :4] = np.array(i["x"], np.float32)
    t = np.array(i["t"], np.float32)
    A = dev(a).requires_grad_(True)
    B = dev(b).requires_grad_(True)
    xd, td = dev(x), dev(t)
    from loractl_b200.linear import _LoraLinearFn

    losses = []
    for _ in range(hp["steps"]):
        y = _LoraLinearFn.apply(xd, A, B, wq, hp["alpha"] / hp["rank"], None)[:, :3]
        loss = ((y - td) ** 2).mean()
        losses.append(float(loss))
        A.grad = B.grad = None
        loss.backward()
        with torch.no_grad():
            A -= hp["lr"] * A.grad
            B -= hp["lr"] * B.grad
    # int8 codes * 0.01 reproduce W to f32 rounding of 0.01*q, so allow 1e-5 + that rounding
    assert np.abs(np.array(losses) - np.array(g["losses"])).max() <= 2e-5
    assert np.abs(host(A)[:4].ravel() - np.array(g["lora_a_final"], np.float32)).max() <= 2e-5
    assert np.abs(host(B)[:, :3].ravel() - np.array(g["lora_b_final"], np.float32)).max() <= 2e-5


def test_empty_batch_and_accumulate():
    from loractl_b200 import quant as Q

    wq, dq, x, a, b, dy, _ = make_case(6, 64, 32, 4)
    ad, bd = dev(a), dev(b)
    y, h = Q.linear_fwd_raw(wq, torch.empty((0, 64), device="cuda"), ad, bd, 1.0)
    assert y.shape == (0, 32)
    dx, da, db = Q.linear_bwd_raw(wq, torch.empty((0, 32), device="cuda"), torch.empty((0, 64), device="cuda"),
                                  None, ad, bd, 1.0)
    assert dx.shape == (0, 64) and float(da.abs().max()) == 0.0 and float(db.abs().max()) == 0.0
    # accumulate = add into a caller bucket
    xd, dyd = dev(x), dev(dy)
    _, h = Q.linear_fwd_raw(wq, xd, ad, bd, 1.0)
    _, da1, db1 = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 1.0)
    bucket_a, bucket_b = da1.clone(), db1.clone()
    Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 1.0, da_out=bucket_a, db_out=bucket_b, accumulate=True)
    assert reldev(host(bucket_a), 2 * host(da1)) <= 1e-6 and reldev(host(bucket_b), 2 * host(db1)) <= 1e-6


def test_argument_errors_are_loud():
    from loractl_b200 import quant as Q
    from loractl_b200._lib import LqError

    wq, *_ = make_case(4, 64, 32, 0)
    with pytest.raises(ValueError, match="x must be"):
        lb().quant_matmul_t(torch.zeros(4, 32, device="cuda"), wq)
    with pytest.raises(TypeError, match="requires a quantized weight"):
        lb().quant_matmul_t(torch.zeros(4, 64, device="cuda"), torch.zeros(32, 64, device="cuda"))
    with pytest.raises(TypeError, match="unsupported activation dtype"):
        Q.linear_fwd_raw(wq, torch.zeros(4, 64, device="cuda", dtype=torch.float16), None, None, 1.0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Q.linear_fwd_raw(wq, torch.zeros(4, 64), None, None, 1.0)
    lin = torch.nn.Linear(64, 32, bias=False).cuda()
    mod = lb().LoraLinear(lb().QuantLinear.from_linear(lin, 4), 4, 4.0, dropout_prob=0.1, device="cuda").train()
    with pytest.raises(RuntimeError, match="dropout"):
        mod(torch.zeros(2, 64, device="cuda"))

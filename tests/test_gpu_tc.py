"""GPU tests of the tcgen05 path: the bare bf16 contraction against an f32 matmul of the same
bf16 inputs, then the bf16 LoRA linear (forward and backward) against the f32 CPU oracle.

Tolerances (stated, peak-normalised, `rel_deviation` of crates/loractl-core/src/accuracy.rs:96-115):
  * bare GEMM, f32 output: 1e-5 (bf16 products are exact in f32; only the accumulation order differs);
  * bare GEMM, bf16 output: 4e-3 (one rounding of the result to 8 mantissa bits);
  * LoRA linear with bf16 activations vs the f32 oracle on the same (bf16-rounded) inputs:
    Y, dX within 6e-3 (the frozen weight is rounded once to bf16 before the MMA and the result
    once more on store), dA, dB (f32 outputs, bf16 operands) within 8e-3, cosine >= 0.9999."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import bf16_round, dev, host, reldev, seeded

pytestmark = pytest.mark.gpu


def lb():
    import loractl_b200

    return loractl_b200


def run_gemm(a, b, a_mn, b_mn, out_dtype, block_n, splits=1, bias=None):
    """a: [Mg, Kg] logical, b: [Ng, Kg] logical (torch bf16 on cuda).  *_mn stores the transpose."""
    from loractl_b200 import _lib as L

    mg, kg = a.shape
    ng = b.shape[0]
    a_st = a.t().contiguous() if a_mn else a.contiguous()
    b_st = b.t().contiguous() if b_mn else b.contiguous()
    c = torch.full((mg, ng), float("nan"), dtype=out_dtype, device="cuda")
    part = None
    if splits > 1:
        part = torch.empty(splits * mg * ((ng + 63) // 64 * 64), dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    L.check(L.lib().lq_gemm_bf16(a_st.data_ptr(), int(a_mn), a_st.stride(0), b_st.data_ptr(), int(b_mn),
                                 b_st.stride(0), c.data_ptr(), L.LQ_F32 if out_dtype == torch.float32 else L.LQ_BF16,
                                 ng, mg, ng, kg, block_n, splits, part.data_ptr() if part is not None else None,
                                 bias.data_ptr() if bias is not None else None, st))
    lb().check_device_status()
    return c


GEMM_CASES = [
    # Mg, Ng, Kg, block_n, a_mn, b_mn, splits
    (128, 256, 64, 256, 0, 0, 1),
    (128, 128, 128, 128, 0, 0, 1),
    (256, 512, 256, 256, 0, 0, 1),
    (300, 520, 200, 256, 0, 0, 1),
    (300, 520, 200, 128, 0, 0, 1),
    (300, 520, 200, 192, 0, 0, 1),
    (1024, 3072, 512, 192, 0, 0, 1),
    (1000, 72, 512, 64, 0, 0, 1),
    (1000, 64, 1024, 64, 0, 0, 4),
    (4096, 3072, 3072, 256, 0, 0, 1),
    (136, 64, 320, 64, 1, 1, 1),
    (384, 64, 1000, 64, 1, 1, 5),
    (256, 256, 192, 128, 0, 1, 1),
    (256, 256, 192, 128, 1, 0, 1),
]


@pytest.mark.parametrize("mg,ng,kg,block_n,a_mn,b_mn,splits", GEMM_CASES)
def test_bare_gemm_f32_out(mg, ng, kg, block_n, a_mn, b_mn, splits):
    a = dev(seeded((mg, kg), 1), torch.bfloat16)
    b = dev(seeded((ng, kg), 2), torch.bfloat16)
    ref = a.float() @ b.float().t()
    c = run_gemm(a, b, a_mn, b_mn, torch.float32, block_n, splits)
    assert torch.isfinite(c).all()
    assert reldev(host(c), host(ref)) <= 1e-5


@pytest.mark.parametrize("mg,ng,kg,block_n", [(256, 512, 256, 256), (300, 520, 200, 128), (77, 72, 96, 64)])
def test_bare_gemm_bf16_out_with_bias(mg, ng, kg, block_n):
    a = dev(seeded((mg, kg), 1), torch.bfloat16)
    b = dev(seeded((ng, kg), 2), torch.bfloat16)
    bias = dev(seeded((ng,), 3))
    ref = a.float() @ b.float().t() + bias
    c = run_gemm(a, b, 0, 0, torch.bfloat16, block_n, 1, bias)
    assert reldev(host(c), host(ref)) <= 4e-3


def oracle_case(n, k, m, r, scheme, block=64):
    w = seeded((m, k), 5, 0.02)
    x = bf16_round(seeded((n, k), 6))
    dy = bf16_round(seeded((n, m), 9))
    a = seeded((k, r), 7, 1.0 / np.sqrt(k)) if r else None
    b = seeded((r, m), 8, 0.01) if r else None
    if scheme in ("int4", "int8"):
        bits = 4 if scheme == "int4" else 8
        wq = lb().quantize_linear_weight(dev(w), bits, block)
        dq = O.dequantize(*O.quantize(w, block, bits), block)
    else:
        pc = scheme == "fp8_channel"
        wq = lb().fp8_quantize(dev(w), pc)
        dq = O.fp8_dequant(*O.fp8_quantize(w, pc))
    return wq, dq, x, dy, a, b


@pytest.mark.parametrize("n,k,m,r", [(128, 256, 256, 16), (300, 320, 264, 8), (1, 64, 128, 4), (64, 128, 72, 32),
                                     (1024, 768, 768, 8), (4096, 3072, 3072, 16), (513, 512, 1024, 80)])
@pytest.mark.parametrize("scheme", ["int4", "int8", "fp8_channel"])
def test_bf16_lora_linear_matches_oracle(n, k, m, r, scheme):
    from loractl_b200 import quant as Q

    if scheme != "int4" and n > 1024:
        pytest.skip("full-size case runs for int4 only (time)")
    wq, dq, x, dy, a, b = oracle_case(n, k, m, r, scheme)
    s = 2.0
    xd, dyd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16)
    ad, bd = dev(a), dev(b)
    y, h = Q.linear_fwd_raw(wq, xd, ad, bd, s)
    lb().check_device_status()
    oy, oh = O.lora_linear_fwd(x, dq, a, b, s)
    assert y.dtype == torch.bfloat16
    assert reldev(host(y), oy) <= 6e-3 and O.cosine(host(y), oy) >= 0.9999
    assert reldev(host(h), oh) <= 6e-3
    dx, da, db = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, s)
    lb().check_device_status()
    odx, oda, odb = O.lora_linear_bwd(dy, x, dq, a, b, s)
    assert reldev(host(dx), odx) <= 6e-3 and O.cosine(host(dx), odx) >= 0.9999
    assert reldev(host(da), oda) <= 8e-3 and reldev(host(db), odb) <= 8e-3
    # H = NULL: recomputed inside the backward
    _, _, db2 = Q.linear_bwd_raw(wq, dyd, xd, None, ad, bd, s, need_dx=False, need_da=False)
    assert reldev(host(db2), odb) <= 8e-3


def test_bf16_base_only_and_bias():
    from loractl_b200 import quant as Q

    wq, dq, x, dy, _, _ = oracle_case(200, 256, 384, 0, "int4")
    bias = seeded((384,), 10, 0.1)
    wq.set_bias(dev(bias))
    y, _ = Q.linear_fwd_raw(wq, dev(x, torch.bfloat16), None, None, 1.0)
    oy, _ = O.lora_linear_fwd(x, dq, None, None, 1.0, bias)
    assert reldev(host(y), oy) <= 6e-3
    dx, _, _ = Q.linear_bwd_raw(wq, dev(dy, torch.bfloat16), None, None, None, None, 1.0)
    assert reldev(host(dx), O.lora_linear_bwd(dy, x, dq)[0]) <= 6e-3


def test_bf16_zero_init_b_is_bit_identical_to_base_only_and_deterministic():
    """Zero-initialised B contributes exact zeros to the f32 accumulator, so the adapted output is
    bit-identical to the base-only kernel; and two runs are bit-identical (no atomics), which
    block-checkpoint recompute relies on (crates/loractl-core/tests/block_ckpt.rs:236-283)."""
    from loractl_b200 import quant as Q

    wq, dq, x, dy, a, b = oracle_case(300, 256, 512, 16, "int4")
    xd, dyd, ad = dev(x, torch.bfloat16), dev(dy, torch.bfloat16), dev(a)
    zb = torch.zeros((16, 512), device="cuda")
    y0, _ = Q.linear_fwd_raw(wq, xd, None, None, 1.0)
    y1, _ = Q.linear_fwd_raw(wq, xd, ad, zb, 1.0)
    assert torch.equal(y0, y1)
    bd = dev(b)
    ya, ha = Q.linear_fwd_raw(wq, xd, ad, bd, 1.0)
    yb, hb = Q.linear_fwd_raw(wq, xd, ad, bd, 1.0)
    assert torch.equal(ya, yb) and torch.equal(ha, hb)
    g1 = Q.linear_bwd_raw(wq, dyd, xd, ha, ad, bd, 1.0)
    g2 = Q.linear_bwd_raw(wq, dyd, xd, ha, ad, bd, 1.0)
    assert all(torch.equal(p, q) for p, q in zip(g1, g2))


def test_bf16_autograd_module():
    lin = torch.nn.Linear(256, 384, bias=True).cuda()
    mod = lb().LoraLinear(lb().QuantLinear.from_linear(lin, 4, block=64), rank=8, alpha=16.0, device="cuda")
    with torch.no_grad():
        mod.lora_b.normal_(0, 0.01)
    x = dev(seeded((3, 50, 256), 6), torch.bfloat16).requires_grad_(True)
    y = mod(x)
    assert y.shape == (3, 50, 384) and y.dtype == torch.bfloat16
    y.float().pow(2).mean().backward()
    assert x.grad is not None and x.grad.shape == x.shape
    assert torch.isfinite(mod.lora_a.grad).all() and float(mod.lora_a.grad.abs().max()) > 0
    assert torch.isfinite(mod.lora_b.grad).all() and float(mod.lora_b.grad.abs().max()) > 0


def test_split_gemm_rejects_more_splits_than_k_blocks():
    """A k-range without a k-block would publish an accumulator that no MMA wrote."""
    from loractl_b200 import _lib as L

    a = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((128, 64), dtype=torch.float32, device="cuda")
    part = torch.zeros(2 * 128 * 64, dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = L.lib().lq_gemm_bf16(a.data_ptr(), 0, 64, b.data_ptr(), 0, 64, c.data_ptr(), L.LQ_F32, 64, 128, 64, 64, 64, 2,
                              part.data_ptr(), None, st)
    assert rc == L.LQ_ERR_INVALID
    assert b"splits must not exceed" in L.lib().lq_last_error()


@pytest.mark.parametrize("n,k,m", [(20480, 128, 256), (19200, 192, 520)])
def test_more_tiles_than_cta_pairs_with_a_thin_last_round(n, k, m):
    """More 256 x 256 tiles than resident CTA pairs, the last round filling only a few of them: the
    persistent grid wraps around; every output element must be written exactly once and correctly."""
    from loractl_b200 import quant as Q

    wq, dq, x, dy, a, b = oracle_case(n, k, m, 8, "int4")
    xd, dyd, ad, bd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16), dev(a), dev(b)
    y, h = Q.linear_fwd_raw(wq, xd, ad, bd, 1.5)
    dx, da, db = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 1.5)
    lb().check_device_status()
    assert torch.isfinite(y).all() and torch.isfinite(dx).all()
    oy, _ = O.lora_linear_fwd(x, dq, a, b, 1.5)
    odx, oda, odb = O.lora_linear_bwd(dy, x, dq, a, b, 1.5)
    assert reldev(host(y), oy) <= 6e-3 and reldev(host(dx), odx) <= 6e-3
    assert reldev(host(da), oda) <= 8e-3 and reldev(host(db), odb) <= 8e-3
    y2, _ = Q.linear_fwd_raw(wq, xd, ad, bd, 1.5)
    assert torch.equal(y, y2)


def _set_option(name, value):
    from loractl_b200 import _lib as L

    L.check(L.lib().lq_option_set(name.encode(), int(value)))


@pytest.mark.parametrize("scheme", ["int4", "fp8", "fp8-native"])
@pytest.mark.parametrize("n,k,m", [(2048, 6144, 3072), (2048, 3072, 6144), (2048, 12288, 3072), (512, 12288, 3072),
                                   (640, 3072, 12288)])
def test_thin_last_round_cut_along_k_matches_the_uncut_gemm(n, k, m, scheme):
    """A frozen GEMM with a long reduction (>= 96 k-blocks: d_in 6144 forward, d_out 6144 backward, d_in
    12288 in native fp8) whose last round of the persistent pair grid is at most half full (96 tiles on
    74 pairs here), or whose only round is (a 512-token site: 24 tiles), has those tiles cut into k-ranges (f32 partial tiles, summed in a fixed order by a second launch).  Against the
    same call with the cut switched off: equal up to the reordering of one f32 sum before the bf16
    rounding; against the oracle: the usual band; and bit-identical when repeated."""
    from loractl_b200 import quant as Q

    w = seeded((m, k), 5, 0.02)
    x = bf16_round(seeded((n, k), 6))
    dy = bf16_round(seeded((n, m), 9))
    a, b = seeded((k, 16), 7, 1.0 / np.sqrt(k)), seeded((16, m), 8, 0.01)
    bias = seeded((m,), 10, 0.1)
    if scheme == "int4":
        wq = lb().quantize_linear_weight(dev(w), 4, 64)
        dq = O.dequantize(*O.quantize(w, 64, 4), 64)
    else:
        wq = lb().fp8_quantize(dev(w), True)
        dq = host(wq.dequantize())
    wq.set_bias(dev(bias))
    fp8c = scheme == "fp8-native"
    xd, dyd, ad, bd = dev(x, torch.bfloat16), dev(dy, torch.bfloat16), dev(a), dev(b)

    def run():
        y, h = Q.linear_fwd_raw(wq, xd, ad, bd, 2.0, fp8_compute=fp8c)
        dx, da, db = Q.linear_bwd_raw(wq, dyd, xd, h, ad, bd, 2.0, fp8_compute=fp8c)
        lb().check_device_status()
        return y, dx

    try:
        _set_option("tail_split", 0)
        y0, dx0 = run()
        _set_option("tail_split", 1)
        y1, dx1 = run()
        y2, dx2 = run()
    finally:
        _set_option("tail_split", 1)
    assert torch.equal(y1, y2) and torch.equal(dx1, dx2)
    for got, ref in ((y1, y0), (dx1, dx0)):
        peak = float(ref.float().abs().max())
        assert float((got.float() - ref.float()).abs().max()) <= 8e-3 * peak  # one bf16 ulp at the peak's binade
        assert float((got.float() - ref.float()).abs().mean()) <= 2e-4 * peak
    oy, _ = O.lora_linear_fwd(x, dq, a, b, 2.0, bias)
    odx = O.lora_linear_bwd(dy, x, dq, a, b, 2.0)[0]
    tol = 5e-2 if fp8c else 6e-3
    assert reldev(host(y1), oy) <= tol and reldev(host(dx1), odx) <= tol

"""A resident bf16 copy of the dequantised weight (`lq_weight_attach_bf16_copy`).

While a copy is attached the bf16 tensor-regime calls run no dequantisation pass: the forward reads
the copy as a K-major operand, the backward reads THE SAME buffer as an MN-major operand of the
CTA-pair GEMM.  The copy holds the same bf16(q * scale) values as the per-call scratch, so Y is
bit-identical and dX equal to accumulation-order noise at most (checked bit for bit first)."""
import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import bf16_round, dev, host, reldev, seeded

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("scheme", ["int4", "fp8"])
@pytest.mark.parametrize("n,k,m,r", [(256, 256, 256, 16), (300, 320, 384, 8), (1024, 768, 768, 8), (513, 512, 1032, 80),
                                     (2048, 3072, 3072, 0), (130, 256, 512, 16)])
def test_attached_copy_gives_the_same_results_without_a_dequant_pass(n, k, m, r, scheme):
    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200 import quant as Q

    w = seeded((m, k), 5, 0.02)
    wq = lb.quantize_linear_weight(dev(w), 4, 64) if scheme == "int4" else lb.fp8_quantize(dev(w), True)
    x = dev(bf16_round(seeded((n, k), 6)), torch.bfloat16)
    dy = dev(bf16_round(seeded((n, m), 9)), torch.bfloat16)
    a = dev(seeded((k, r), 7, 1.0 / np.sqrt(k))) if r else None
    b = dev(seeded((r, m), 8, 0.01)) if r else None

    def run():
        y, h = Q.linear_fwd_raw(wq, x, a, b, 2.0)
        dx, da, db = Q.linear_bwd_raw(wq, dy, x, h, a, b, 2.0)
        lb.check_device_status()
        return y, dx, da, db

    ref = run()
    lib = L.lib()
    lib.lq_profile_enable(1)
    lib.lq_profile_collect(None, None, 0)
    copy = wq.attach_bf16_copy()
    assert torch.equal(copy.view(m, k), wq.dequantize().to(torch.bfloat16))
    lib.lq_profile_collect(None, None, 0)  # forget the attach's own pass
    got = run()
    nk = lib.lq_profile_kinds()
    import ctypes as C
    ms, cnt = (C.c_double * nk)(), (C.c_uint64 * nk)()
    lib.lq_profile_collect(ms, cnt, nk)
    lib.lq_profile_enable(0)
    kinds = {lib.lq_profile_kind_name(i).decode(): int(cnt[i]) for i in range(nk)}
    # no dequantisation pass ran (below 256 tokens the backward keeps the transposed scratch: the
    # MN-major read is a CTA-pair kernel, which wants at least one full 256-row tile)
    assert kinds.get("dequant", 0) == (0 if n >= 256 else 1), kinds
    assert torch.equal(got[0], ref[0]), "Y differs"
    if not torch.equal(got[1], ref[1]):
        # MN-major read of the same values; the two routes may tile differently (192- against 256-column
        # tiles, a thin last round cut along k in one and not the other), which reorders f32 sums before
        # the bf16 rounding: single roundings flip, nothing more
        d = (got[1].float() - ref[1].float()).abs()
        peak = float(ref[1].float().abs().max())
        assert float(d.max()) <= 8e-3 * peak and float(d.mean()) <= 2e-4 * peak
    if r:
        assert torch.equal(got[2], ref[2]) and torch.equal(got[3], ref[3])
    wq.detach_bf16_copy()
    again = run()
    assert torch.equal(again[0], ref[0]) and torch.equal(again[1], ref[1])


def test_copy_buffer_is_validated():
    import loractl_b200 as lb

    wq = lb.quantize_linear_weight(dev(seeded((128, 64), 5, 0.02)), 4, 64)
    with pytest.raises(ValueError):
        wq.attach_bf16_copy(torch.empty(10, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        wq.attach_bf16_copy(torch.empty(128 * 64, dtype=torch.float16, device="cuda"))

"""The bf16 operand mirror of a site's LoRA factors (`lq_lora_mirror_update`).

The tensor-core path consumes A and B as bf16 operands; with a caller-kept mirror the hot calls
cast nothing.  The values are the same bf16 roundings either way, so forward and backward must be
BIT-IDENTICAL with and without it; a refreshed mirror must follow parameter updates made through
torch (version counters) and through the fused AdamW kernel (raw pointers)."""
import numpy as np
import pytest
import torch

from tests.util import bf16_round, dev, seeded

pytestmark = pytest.mark.gpu


def _case(n, k, m, r, block=64):
    import loractl_b200 as lb

    wq = lb.quantize_linear_weight(dev(seeded((m, k), 5, 0.02)), 4, block)
    x = dev(bf16_round(seeded((n, k), 6)), torch.bfloat16)
    dy = dev(bf16_round(seeded((n, m), 9)), torch.bfloat16)
    a = dev(seeded((k, r), 7, 1.0 / np.sqrt(k)))
    b = dev(seeded((r, m), 8, 0.01))
    return wq, x, dy, a, b


@pytest.mark.parametrize("n,k,m,r", [(300, 256, 512, 16), (128, 320, 264, 8), (513, 512, 1024, 80), (70, 128, 72, 32)])
def test_mirror_is_bit_identical_to_casting_inside_the_call(n, k, m, r):
    import loractl_b200 as lb
    from loractl_b200 import quant as Q

    wq, x, dy, a, b = _case(n, k, m, r)
    mir = Q.lora_mirror(a, b)
    y0, h0 = Q.linear_fwd_raw(wq, x, a, b, 2.0)
    y1, h1 = Q.linear_fwd_raw(wq, x, a, b, 2.0, mirror=mir)
    assert torch.equal(y0, y1) and torch.equal(h0, h1)
    g0 = Q.linear_bwd_raw(wq, dy, x, h0, a, b, 2.0)
    g1 = Q.linear_bwd_raw(wq, dy, x, h0, a, b, 2.0, mirror=mir)
    assert all(torch.equal(p, q) for p, q in zip(g0, g1))
    g2 = Q.linear_bwd_raw(wq, dy, x, None, a, b, 2.0, mirror=mir)  # H recomputed from the mirror's A^T
    assert torch.equal(g2[2], Q.linear_bwd_raw(wq, dy, x, None, a, b, 2.0)[2])
    lb.check_device_status()


def test_mirror_follows_parameter_updates():
    import loractl_b200 as lb
    from loractl_b200.optim import AdamW, FlatAdapters

    lin = torch.nn.Linear(256, 384, bias=False).cuda()
    site = lb.LoraLinear(lb.QuantLinear.from_linear(lin, 4, block=64), rank=8, alpha=16.0, device="cuda")
    d = site.delta
    x = dev(bf16_round(seeded((200, 256), 3)), torch.bfloat16)
    y0 = site(x)
    m0 = d.operand_mirror()
    assert m0 is not None and d.operand_mirror() is m0  # unchanged factors: no rebuild
    with torch.no_grad():
        d.lora_b.normal_(0, 0.02)  # a torch in-place update bumps the version counter
    y1 = site(x)
    assert not torch.equal(y0, y1)
    from loractl_b200 import quant as Q

    want, _ = Q.linear_fwd_raw(site.base.inner.weight, x, d.lora_a.detach(), d.lora_b.detach(), d.scaling)
    assert torch.equal(y1, want)
    # the fused AdamW writes through raw pointers: the shared epoch marks every mirror stale
    ad = lb.LoraAdapters([d], ["site"])
    flat = FlatAdapters(ad, torch.device("cuda"))
    opt = AdamW(flat)
    y2 = site(x)
    flat.grads.normal_(0, 1.0)
    opt.step(1e-2)
    y3 = site(x)
    want3, _ = Q.linear_fwd_raw(site.base.inner.weight, x, d.lora_a.detach(), d.lora_b.detach(), d.scaling)
    assert torch.equal(y3, want3) and not torch.equal(y2, y3)


def test_mirror_arguments_are_validated():
    from loractl_b200 import _lib as L

    assert L.lib().lq_lora_mirror_bytes(256, 512, 0) == 0
    assert L.lib().lq_lora_mirror_bytes(256, 512, 16) >= 2 * (16 * 256 + 512 * 64 + 16 * 512 + 256 * 64)
    a = torch.zeros((256, 16), device="cuda")
    b = torch.zeros((16, 512), device="cuda")
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    off = (-buf.data_ptr()) % 256 + 16  # misaligned on purpose
    rc = L.lib().lq_lora_mirror_update(a.data_ptr(), b.data_ptr(), 256, 512, 16, buf.data_ptr() + off, None)
    assert rc == L.LQ_ERR_INVALID


def test_batched_mirror_update_equals_per_site_updates():
    """`lq_lora_mirror_update_batch` over many sites (more than one launch's worth, mixed shapes and
    ranks) writes exactly the bytes of one `lq_lora_mirror_update` per site."""
    from loractl_b200 import quant as Q

    shapes = [(256 + 64 * (i % 3), 128 + 128 * (i % 4), (4, 16, 32, 80)[i % 4]) for i in range(29)]
    jobs, singles = [], []
    for i, (k, m, r) in enumerate(shapes):
        a, b = dev(seeded((k, r), 50 + i, 0.1)), dev(seeded((r, m), 90 + i, 0.1))
        ref = Q.lora_mirror_alloc(a, b)
        ref.fill_(0xFF)  # the alignment gaps between the four arrays are written by neither route
        singles.append(Q.lora_mirror(a, b, ref))
        buf = Q.lora_mirror_alloc(a, b)
        buf.fill_(0xFF)
        jobs.append((a, b, buf))
    Q.lora_mirror_batch(jobs)
    torch.cuda.synchronize()
    for (a, b, buf), ref in zip(jobs, singles):
        assert torch.equal(buf, ref)
    Q.lora_mirror_batch([])  # an empty batch is a no-op

"""`lq_linear_fwd_grouped`: sites that read the same activation in one call — wq / wk / wv and gate / up
in the reference (crates/loractl-core/src/mmdit.rs:599-610,701-706).  At <= 16 bf16 tokens over int4
weights of one width the group is ONE launch of the packed-weight-stream kernel plus one finalize;
otherwise the sites run one after the other.  Either way every site's result must be what
`lq_linear_fwd` gives for it alone."""
import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import bf16_round, dev, host, reldev, seeded

pytestmark = pytest.mark.gpu


def _sites(k, outs, ranks, block=64):
    import loractl_b200 as lb

    sites, refs = [], []
    for i, (m, r) in enumerate(zip(outs, ranks)):
        w = seeded((m, k), 20 + i, 0.02)
        wq = lb.quantize_linear_weight(dev(w), 4, block)
        dq = O.dequantize(*O.quantize(w, block, 4), block)
        a = seeded((k, r), 30 + i, 1.0 / np.sqrt(k)) if r else None
        b = seeded((r, m), 40 + i, 0.01) if r else None
        sites.append((wq, dev(a) if r else None, dev(b) if r else None, 1.5))
        refs.append((dq, a, b))
    return sites, refs


@pytest.mark.parametrize("n", [1, 8, 16])
def test_group_of_stream_sites_matches_each_site_alone(n):
    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200 import quant as Q

    k = 512
    sites, refs = _sites(k, [256, 384, 1024, 136], [16, 8, 0, 32])
    x = bf16_round(seeded((n, k), 6))
    xd = dev(x, torch.bfloat16)
    lib = L.lib()
    before = lib.lq_kernel_launch_count()
    outs = Q.linear_fwd_grouped_raw(sites, xd)
    launches = lib.lq_kernel_launch_count() - before
    lb.check_device_status()
    assert launches == 2, launches  # one weight-stream launch over all four sites, one finalize
    for (wq, a, b, s), (dq, an, bn), (y, h) in zip(sites, refs, outs):
        y1, h1 = Q.linear_fwd_raw(wq, xd, a, b, s)
        oy, oh = O.lora_linear_fwd(x, dq, an, bn, s)
        assert reldev(host(y), oy) <= 6e-3
        assert reldev(host(y), host(y1)) <= 4e-3  # the joint k-split differs: at most a bf16 rounding apart
        if a is not None:
            assert torch.equal(h, h1) and reldev(host(h), oh) <= 6e-3


def test_group_beyond_the_stream_regime_runs_the_sites_in_turn():
    from loractl_b200 import quant as Q

    sites, _ = _sites(256, [256, 512], [8, 8])
    xd = dev(bf16_round(seeded((100, 256), 6)), torch.bfloat16)
    outs = Q.linear_fwd_grouped_raw(sites, xd)
    for (wq, a, b, s), (y, h) in zip(sites, outs):
        y1, h1 = Q.linear_fwd_raw(wq, xd, a, b, s)
        assert torch.equal(y, y1) and torch.equal(h, h1)


def test_site_group_autograd_equals_separate_sites():
    import loractl_b200 as lb
    from loractl_b200.adapters import LoraConfig, LoraSite, TargetSpec, build_adapters
    from loractl_b200.linear import site, site_group

    torch.manual_seed(0)
    bases = {n: lb.BaseLinear.quant(lb.QuantLinear.from_linear(torch.nn.Linear(256, m, bias=False).cuda(), 4, block=64))
             for n, m in (("wq", 256), ("wk", 128), ("wv", 128))}
    ad = build_adapters([LoraSite(f"blk.{n}", 256, b.d_out) for n, b in bases.items()],
                        LoraConfig(rank=4, alpha=8.0, targets=[TargetSpec(r"w(q|v)$")]), torch.device("cuda"))
    with torch.no_grad():
        for d in ad.deltas:
            d.lora_b.normal_(0, 0.02)
    x = dev(bf16_round(seeded((2, 6, 256), 3)), torch.bfloat16).requires_grad_(True)
    pairs = [(f"blk.{n}", b) for n, b in bases.items()]
    ys = site_group(ad, pairs, x)
    loss = sum((y.float() ** 2).mean() for y in ys)
    loss.backward()
    gx = x.grad.clone()
    ga = [(d.lora_a.grad.clone(), d.lora_b.grad.clone()) for d in ad.deltas]
    x.grad = None
    for d in ad.deltas:
        d.lora_a.grad = d.lora_b.grad = None
    ys2 = [site(ad, p, b, x) for p, b in pairs]
    loss2 = sum((y.float() ** 2).mean() for y in ys2)
    loss2.backward()
    assert abs(float(loss) - float(loss2)) <= 1e-2 * abs(float(loss2))
    assert reldev(host(gx), host(x.grad)) <= 1e-2
    for (a1, b1), d in zip(ga, ad.deltas):
        assert reldev(host(a1), host(d.lora_a.grad)) <= 1e-2 and reldev(host(b1), host(d.lora_b.grad)) <= 1e-2


def test_group_rejects_sites_of_different_width():
    from loractl_b200 import _lib as L
    from loractl_b200 import quant as Q

    s1, _ = _sites(256, [256], [0])
    s2, _ = _sites(512, [256], [0])
    xd = dev(bf16_round(seeded((4, 256), 6)), torch.bfloat16)
    with pytest.raises(L.LqError) as e:
        Q.linear_fwd_grouped_raw(s1 + s2, xd)
    assert e.value.status == L.LQ_ERR_INVALID

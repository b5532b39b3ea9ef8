"""GPU tests of the step glue and of block-checkpoint recompute.

AdamW and the finite check are floating-point kernels with no quantized arithmetic, so their
reference is plain PyTorch fp32 (torch.optim.AdamW implements the same decoupled-decay formula as
burn's AdamW); tolerance 1e-6 relative.  Checkpointed gradients must EQUAL the monolithic ones
bit for bit (crates/loractl-core/tests/block_ckpt.rs:236-283), which holds because every kernel
on the path is deterministic."""
import numpy as np
import pytest
import torch

from tests.util import dev, seeded

pytestmark = pytest.mark.gpu


def lb():
    import loractl_b200

    return loractl_b200


@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096, 1_000_003])
def test_nonfinite_flag(n):
    g = torch.randn(n, device="cuda")
    flag = torch.full((1,), 7, dtype=torch.int32, device="cuda")
    lb().nonfinite_flag(g, flag)
    assert int(flag) == 0
    for pos, val in ((0, float("nan")), (n - 1, float("inf")), (n // 2, float("-inf"))):
        g2 = g.clone()
        g2[pos] = val
        lb().nonfinite_flag(g2, flag)
        assert int(flag) == 1
    lb().nonfinite_flag(g, flag)
    assert int(flag) == 0  # cleared again


def make_adapters(device="cuda"):
    sites = [lb().LoraSite("blocks.0.w1", 64, 96), lb().LoraSite("blocks.0.w2", 96, 64),
             lb().LoraSite("blocks.1.w1", 64, 96)]
    ad = lb().build_adapters(sites, lb().LoraConfig(rank=4, alpha=8.0, targets=[lb().TargetSpec("blocks")]), device)
    with torch.no_grad():
        for d in ad.deltas:
            d.lora_b.normal_(0, 0.02)
    return ad


def test_flat_adapters_are_views_and_adamw_matches_torch():
    ad = make_adapters()
    ref_params = [p.detach().clone().requires_grad_(True) for d in ad.deltas for p in (d.lora_a, d.lora_b)]
    flat = lb().FlatAdapters(ad)
    ours = [p for d in ad.deltas for p in (d.lora_a, d.lora_b)]
    assert all(torch.equal(a, b) for a, b in zip(ours, ref_params))
    assert all(p.data_ptr() == flat.params.data_ptr() + 4 * o for p, o in zip(ours, flat.offsets))
    assert all(o % 64 == 0 for o in flat.offsets)
    opt = lb().AdamW(flat, weight_decay=1e-2)
    ref = torch.optim.AdamW(ref_params, lr=1e-2, betas=(0.9, 0.999), eps=1e-5, weight_decay=1e-2)
    g = torch.Generator(device="cuda").manual_seed(3)
    for step in range(5):
        flat.zero_grad()
        for p, rp in zip(ours, ref_params):
            gr = torch.randn(p.shape, device="cuda", generator=g)
            p.grad.copy_(gr)
            rp.grad = gr.clone()
        opt.step(1e-2)
        ref.step()
        for p, rp in zip(ours, ref_params):
            assert torch.allclose(p, rp, rtol=1e-6, atol=1e-7), step
    # grad_scale = 1/world folds the data-parallel mean into the update
    before = flat.params.clone()
    flat.grads.mul_(2.0)
    m0, v0 = flat.exp_avg.clone(), flat.exp_avg_sq.clone()
    opt.step(1e-2, grad_scale=0.5)
    a = flat.params.clone()
    flat.params.copy_(before); flat.exp_avg.copy_(m0); flat.exp_avg_sq.copy_(v0)
    flat.grads.mul_(0.5)
    opt.step(1e-2, grad_scale=1.0, count=False)
    assert torch.allclose(a, flat.params, rtol=1e-6, atol=1e-8)
    # a raised skip flag makes the step a no-op, decided on the device
    snap = (flat.params.clone(), flat.exp_avg.clone(), flat.exp_avg_sq.clone())
    flat.grads[5] = float("nan")
    lb().nonfinite_flag(flat.grads, flat.flag)
    opt.step(1e-2, skip_flag=flat.flag, count=False)
    assert torch.equal(flat.params, snap[0]) and torch.equal(flat.exp_avg, snap[1]) and torch.equal(flat.exp_avg_sq, snap[2])


class Block(torch.nn.Module):
    """x + w2(silu(w1(norm(x)))) with both linears as LoRA'd quantized sites."""

    def __init__(self, idx, adapters, dtype):
        super().__init__()
        l1, l2 = torch.nn.Linear(64, 96).cuda(), torch.nn.Linear(96, 64).cuda()
        self.w1 = lb().BaseLinear.quant(lb().QuantLinear.from_linear(l1, 4))
        self.w2 = lb().BaseLinear.quant(lb().QuantLinear.from_linear(l2, 4))
        self.idx, self.adapters, self.dtype = idx, adapters, dtype

    def forward(self, x):
        h = torch.nn.functional.layer_norm(x.float(), (64,)).to(self.dtype)
        h = lb().site(self.adapters, f"blocks.{self.idx}.w1", self.w1, h)
        h = torch.nn.functional.silu(h.float()).to(self.dtype)
        return x + lb().site(self.adapters, f"blocks.{self.idx}.w2", self.w2, h)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_checkpointed_step_equals_monolithic_exactly(dtype):
    torch.manual_seed(0)
    ad = make_adapters()
    blocks = [Block(0, ad, dtype), Block(1, ad, dtype)]
    params = [p for d in ad.deltas for p in (d.lora_a, d.lora_b)]
    x0 = dev(seeded((2, 24, 64), 6), dtype)
    target = dev(seeded((2, 24, 64), 7), torch.float32)
    head = lambda x: ((x.float() - target) ** 2).mean()
    scale = 128.0
    # monolithic
    for p in params:
        p.grad = None
    x = x0
    for b in blocks:
        x = b(x)
    loss = head(x)
    (loss * scale).backward()
    mono = [p.grad.clone() if p.grad is not None else torch.zeros_like(p) for p in params]
    # checkpointed
    loss_c, grads_c = lb().checkpointed_step(blocks, x0, head, params, scale)
    assert loss_c == float(loss)
    used = 0
    for gm, gc in zip(mono, grads_c):
        assert torch.equal(gm, gc)
        used += int(float(gc.abs().max()) > 0)
    assert used >= 5  # completeness: the sites that ran produced non-zero gradients
    assert all(torch.isfinite(g).all() for g in grads_c)

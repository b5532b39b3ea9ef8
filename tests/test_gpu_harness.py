"""GPU tests of the training harness around the hot path: a tiny double-stream block stack whose
linears are LoRA'd int4 sites, trained with block-checkpoint recompute, the flat gradient bucket,
the fused finite check and the fused AdamW.

Mirrors crates/loractl-core/tests/block_ckpt.rs:236-283 (checkpointed step == monolithic step,
exactly) and crates/loractl-core/tests/quant_trainer.rs:321-475 (finite, decreasing losses;
a non-finite gradient skips the update and halves the loss scale)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def make(n_blocks=2, dtype=torch.bfloat16):
    from loractl_b200.harness import BlockConfig, BlockStack

    cfg = BlockConfig(hidden=128, heads=4, mlp=256, img_tokens=64, txt_tokens=16, quant_bits=4, quant_block=64)
    return BlockStack(n_blocks, cfg, rank=4, alpha=8.0, device=torch.device("cuda"), seed=5, dtype=dtype), cfg


def batch(cfg, b=2, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x0 = torch.randn((b, cfg.img_tokens, cfg.hidden), generator=g, device="cuda")
    txt = torch.randn((b, cfg.txt_tokens, cfg.hidden), generator=g, device="cuda")
    cond = torch.randn((b, cfg.hidden), generator=g, device="cuda")
    t = torch.rand((b,), generator=g, device="cuda") * 0.9 + 0.05
    noise = torch.randn(x0.shape, generator=g, device="cuda")
    return x0, txt, cond, t, noise


def test_stack_sites_and_bucket():
    stack, cfg = make()
    assert len(stack.adapters.targets) == 20  # 2 blocks x 2 streams x 5 linears
    assert stack.adapters.targets[0] == "blocks.0.img.mod" and stack.adapters.targets[-1] == "blocks.1.txt.down"
    n = sum(p.numel() for p in stack.lora_parameters())
    assert stack.flat.numel >= n and all(p.data_ptr() >= stack.flat.params.data_ptr() for p in stack.lora_parameters())


def test_checkpointed_trainer_step_equals_monolithic_exactly():
    from loractl_b200.harness import Trainer

    x0, txt, cond, t, noise = batch(make()[1])
    grads, losses = [], []
    for ckpt in (True, False):
        stack, _ = make()
        tr = Trainer(stack, lr=0.0, weight_decay=0.0, grad_checkpointing=ckpt)  # lr 0: compare gradients only
        losses.append(tr.step(x0, txt, cond, t, noise))
        grads.append(stack.flat.grads.clone())
    assert losses[0] == losses[1]
    assert torch.equal(grads[0], grads[1])
    assert torch.isfinite(grads[0]).all() and float(grads[0].abs().max()) > 0


def test_training_reduces_the_loss_and_skips_on_nonfinite_gradients():
    from loractl_b200.harness import Trainer

    stack, cfg = make()
    tr = Trainer(stack, lr=2e-3, weight_decay=0.0)
    data = batch(cfg)
    losses = [tr.step(*data) for _ in range(8)]
    assert all(l == l and l < 1e6 for l in losses) and losses[-1] < losses[0]
    assert tr.optim.steps == 8 and tr.scaler.clean_streak == 8
    # poison the activations of one step: gradients become non-finite, the update must be skipped
    before = stack.flat.params.clone()
    x0, txt, cond, t, noise = data
    bad = x0.clone()
    bad[0, 0, 0] = float("inf")
    tr.scaler.loss_scale = 4.0
    tr.step(bad, txt, cond, t, noise)
    assert int(stack.flat.flag) == 1
    assert torch.equal(stack.flat.params, before)
    assert tr.scaler.loss_scale == 2.0 and tr.scaler.clean_streak == 0 and tr.optim.steps == 8
    # and the run continues afterwards
    l = tr.step(*data)
    assert l == l and tr.optim.steps == 9

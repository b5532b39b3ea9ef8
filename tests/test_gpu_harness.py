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


def test_weight_copy_modes_train_identically():
    """Resident bf16 weight copies and the two-arena prefetch one block ahead change where the bf16
    operand comes from, not its values: same loss, same gradients (the backward reads the copy as an
    MN-major operand, a different tile walk over the same products), and the prefetcher refills
    exactly the blocks the sweep has evicted."""
    from loractl_b200.harness import BlockConfig, BlockStack, Trainer

    cfg = BlockConfig(hidden=256, heads=4, mlp=512, img_tokens=256, txt_tokens=128, quant_bits=4, quant_block=64)
    data = batch(cfg, b=2)
    out = {}
    for mode in ("none", "resident", "block"):
        stack = BlockStack(4, cfg, rank=4, alpha=8.0, device=torch.device("cuda"), seed=5, weight_copies=mode)
        tr = Trainer(stack, lr=1e-3, weight_decay=0.0)
        losses = [tr.step(*data) for _ in range(3)]
        out[mode] = (losses, stack.flat.grads.clone(), stack.flat.params.clone())
        if mode == "block":
            # step 1: blocks 0..3 filled on the way up, 1 and 0 again on the way down; later steps
            # find 0 and 1 in place: 2, 3 up and 1, 0 down
            assert stack.prefetcher.fills == 6 + 4 + 4
            stack.prefetcher.release_all()
    import loractl_b200

    loractl_b200.check_device_status()
    ref_losses, ref_g, ref_p = out["none"]
    for mode in ("resident", "block"):
        losses, g, p = out[mode]
        assert all(abs(a - b) <= 1e-3 * abs(b) for a, b in zip(losses, ref_losses)), (mode, losses, ref_losses)
        assert float((g - ref_g).abs().max()) <= 2e-2 * float(ref_g.abs().max()), mode
        assert float((p - ref_p).abs().max()) <= 5e-3, mode  # lr 1e-3: each Adam step moves a parameter by at most ~lr
    # the two copy modes run the very same kernels on the same operand values; what is left is the
    # run-to-run noise of torch's attention backward (atomic adds), ~1e-6 of the gradient's peak
    assert out["resident"][0] == out["block"][0]
    assert float((out["resident"][1] - out["block"][1]).abs().max()) <= 1e-4 * float(ref_g.abs().max())


def test_graphed_sweep_trains_like_the_eager_sweep():
    """The checkpointed sweep replayed from CUDA graphs (one per block forward, one head, one per block
    replay + backward) runs the same kernels on the same values as the eager sweep: same losses, same
    gradients up to the noise of the attention backward's atomic adds, same parameters after three
    steps — with new data copied into the static buffers every step and a changed loss scale."""
    from loractl_b200.harness import BlockConfig, BlockStack, Trainer

    cfg = BlockConfig(hidden=256, heads=4, mlp=512, img_tokens=256, txt_tokens=128, quant_bits=4, quant_block=64)
    out = {}
    for graphs, mode in ((False, "none"), (True, "none"), (True, "resident"), (True, "block")):
        stack = BlockStack(5, cfg, rank=4, alpha=8.0, device=torch.device("cuda"), seed=5, weight_copies=mode)
        tr = Trainer(stack, lr=1e-3, weight_decay=0.0, graphs=graphs)
        losses = []
        for i in range(3):
            if i == 2:
                tr.scaler.loss_scale = 4.0
            losses.append(tr.step(*batch(cfg, b=2, seed=i)))
        out[(graphs, mode)] = (losses, stack.flat.grads.clone(), stack.flat.params.clone())
        assert tr.optim.steps == 3
    import loractl_b200

    loractl_b200.check_device_status()
    l0, g0, p0 = out[(False, "none")]
    assert l0[0] != l0[1]  # the data really changed between steps
    # same kernels, same values: graph replay against eager launches
    l1, g1, p1 = out[(True, "none")]
    assert all(abs(a - b) <= 1e-5 * abs(a) for a, b in zip(l0, l1)), (l0, l1)
    assert float((g0 - g1).abs().max()) <= 1e-4 * float(g0.abs().max())
    assert float((p0 - p1).abs().max()) <= 1e-5
    # weight copies: the backward walks the same products in another tile order
    for mode in ("resident", "block"):
        l1, g1, p1 = out[(True, mode)]
        assert all(abs(a - b) <= 1e-3 * abs(a) for a, b in zip(l0, l1)), (mode, l0, l1)
        assert float((g0 - g1).abs().max()) <= 2e-2 * float(g0.abs().max()), mode
        assert float((p0 - p1).abs().max()) <= 5e-3, mode
    # the block-ahead refill inside the graphs leaves exactly what the resident copies hold
    assert out[(True, "block")][0] == out[(True, "resident")][0]
    assert float((out[(True, "block")][1] - out[(True, "resident")][1]).abs().max()) <= 1e-4 * float(g0.abs().max())


@pytest.mark.parametrize("graphs", [False, True])
def test_text_and_image_chains_on_two_cuda_streams_change_nothing(graphs):
    """A block's text chain on a second CUDA stream beside the image chain (`two_cuda_streams`) is a
    scheduling change only: three training steps give the single-stream run's losses, gradients and
    parameters (up to the attention backward's atomic-add noise), eagerly and from CUDA graphs, and
    repeating the two-stream run reproduces itself to the same noise."""
    from loractl_b200.harness import BlockConfig, BlockStack, Trainer

    cfg = BlockConfig(hidden=256, heads=4, mlp=512, img_tokens=256, txt_tokens=128, quant_bits=4, quant_block=64)
    runs = []
    for two in (False, True, True):
        stack = BlockStack(3, cfg, rank=4, alpha=8.0, device=torch.device("cuda"), seed=5, two_cuda_streams=two)
        tr = Trainer(stack, lr=1e-3, weight_decay=0.0, graphs=graphs)
        losses = [tr.step(*batch(cfg, b=2, seed=i)) for i in range(3)]
        torch.cuda.synchronize()
        runs.append((losses, stack.flat.grads.clone(), stack.flat.params.clone()))
    import loractl_b200

    loractl_b200.check_device_status()
    (l0, g0, p0) = runs[0]
    for l1, g1, p1 in runs[1:]:
        assert all(abs(a - b) <= 1e-5 * abs(a) for a, b in zip(l0, l1)), (l0, l1)
        assert torch.isfinite(g1).all()
        assert float((g0 - g1).abs().max()) <= 1e-4 * float(g0.abs().max())
        assert float((p0 - p1).abs().max()) <= 1e-5

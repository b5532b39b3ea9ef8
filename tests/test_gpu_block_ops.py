"""GPU parity of the fused element-wise block ops against their plain PyTorch f32 composition
(crates/loractl-core/src/mmdit.rs:857-869: `(scale + 1) * norm(x) + shift`, `x + gate * f(x)`):
forward values and every gradient, f32 (summation-order tolerance) and bf16 (one rounding of the
output), several samples, token counts that do not divide the reduction chunk, and run-to-run
determinism of the token-axis sums."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

CASES = [(1, 1, 64), (2, 5, 96), (1, 300, 3072), (3, 129, 520), (1, 4608, 3072)]


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-30))


def inputs(b, t, h, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g, device="cuda")
    x, y, dout = mk(b, t, h) * 1.5 + 0.3, mk(b, t, h), mk(b, t, h)
    shift, scale, gate = mk(b, 1, h) * 0.5, mk(b, 1, h) * 0.5, mk(b, 1, h)
    return [v.to(dtype) for v in (x, y, dout, shift, scale, gate)]


@pytest.mark.parametrize("b,t,h", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_modulated_layer_norm_matches_torch(b, t, h, dtype):
    from loractl_b200.block_ops import modulated_layer_norm

    x, _, dout, shift, scale, _ = inputs(b, t, h, dtype)
    xs = [v.clone().requires_grad_(True) for v in (x, shift, scale)]
    out = modulated_layer_norm(*xs)
    out.backward(dout)
    ref_in = [v.float().clone().requires_grad_(True) for v in (x, shift, scale)]
    ref = F.layer_norm(ref_in[0], (h,)) * (1 + ref_in[2]) + ref_in[1]
    ref.backward(dout.float())
    tol = 2e-5 if dtype == torch.float32 else 8e-3
    assert out.dtype == dtype and rel(out, ref) <= tol
    for ours, theirs in zip(xs, ref_in):
        assert ours.grad.shape == ours.shape and ours.grad.dtype == dtype
        assert rel(ours.grad, theirs.grad) <= tol


@pytest.mark.parametrize("b,t,h", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_residual_matches_torch(b, t, h, dtype):
    from loractl_b200.block_ops import gated_residual

    x, y, dout, _, _, gate = inputs(b, t, h, dtype, seed=1)
    xs = [v.clone().requires_grad_(True) for v in (x, gate, y)]
    out = gated_residual(*xs)
    out.backward(dout)
    ref_in = [v.float().clone().requires_grad_(True) for v in (x, gate, y)]
    ref = ref_in[0] + ref_in[1] * ref_in[2]
    ref.backward(dout.float())
    tol = 2e-5 if dtype == torch.float32 else 8e-3
    assert rel(out, ref) <= tol
    for ours, theirs in zip(xs, ref_in):
        assert rel(ours.grad, theirs.grad) <= tol


def test_token_axis_sums_are_deterministic():
    from loractl_b200.block_ops import gated_residual, modulated_layer_norm

    x, y, dout, shift, scale, gate = inputs(2, 1000, 3072, torch.bfloat16, seed=2)
    grads = []
    for _ in range(2):
        a = [v.clone().requires_grad_(True) for v in (x, shift, scale)]
        modulated_layer_norm(*a).backward(dout)
        c = [v.clone().requires_grad_(True) for v in (x, gate, y)]
        gated_residual(*c).backward(dout)
        grads.append([v.grad for v in a + c])
    assert all(torch.equal(p, q) for p, q in zip(*grads))


def test_bad_shapes_are_loud():
    from loractl_b200.block_ops import gated_residual, modulated_layer_norm

    x = torch.randn(2, 4, 64, device="cuda")
    with pytest.raises(ValueError, match="shift must hold"):
        modulated_layer_norm(x, torch.zeros(1, 1, 64, device="cuda"), torch.zeros(2, 1, 64, device="cuda"))
    with pytest.raises(ValueError, match=r"expected \[b, tokens, h\]"):
        gated_residual(x[0], torch.zeros(2, 1, 64, device="cuda"), x[0])
    with pytest.raises(RuntimeError, match="CUDA"):
        modulated_layer_norm(x.cpu(), torch.zeros(2, 1, 64), torch.zeros(2, 1, 64))

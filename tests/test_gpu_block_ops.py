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


@pytest.mark.parametrize("shape", [(1, 1, 3), (2, 5, 96), (1, 4608, 512), (3, 129, 521), (8192 * 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["swiglu", "sigmoid_gate"])
def test_swiglu_and_sigmoid_gate_match_torch(shape, dtype, kind):
    """`silu(gate) * up` (crates/loractl-core/src/mmdit.rs:695-708) and `x * sigmoid(gate)`
    (mmdit.rs:659-664) as one kernel each way, against the PyTorch f32 composition: values and both
    input gradients; element counts that are not a multiple of the 16-byte vector."""
    from loractl_b200 import block_ops

    g = torch.Generator(device="cuda").manual_seed(3)
    shape = shape if isinstance(shape, tuple) else (shape,)
    a = (torch.randn(shape, generator=g, device="cuda") * 2).to(dtype)
    b = (torch.randn(shape, generator=g, device="cuda") * 2).to(dtype)
    dout = torch.randn(shape, generator=g, device="cuda").to(dtype)
    xs = [a.clone().requires_grad_(True), b.clone().requires_grad_(True)]
    out = getattr(block_ops, kind)(*xs)
    out.backward(dout)
    ref_in = [a.float().clone().requires_grad_(True), b.float().clone().requires_grad_(True)]
    ref = F.silu(ref_in[0]) * ref_in[1] if kind == "swiglu" else ref_in[0] * torch.sigmoid(ref_in[1])
    ref.backward(dout.float())
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    assert out.shape == a.shape and out.dtype == dtype and rel(out, ref) <= tol
    for ours, theirs in zip(xs, ref_in):
        assert ours.grad.shape == ours.shape and rel(ours.grad, theirs.grad) <= tol


def test_pair_activations_reject_mismatched_operands():
    from loractl_b200.block_ops import swiglu

    a = torch.zeros(4, 8, device="cuda")
    with pytest.raises(ValueError):
        swiglu(a, torch.zeros(4, 7, device="cuda"))
    with pytest.raises(ValueError):
        swiglu(a, torch.zeros(4, 8, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("shape", [(1, 1, 16), (2, 6, 33, 16), (3, 129, 96), (1, 4608, 3072), (2, 24, 300, 128)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_zrmsnorm_matches_torch(shape, dtype):
    """ZRmsNorm (crates/loractl-core/src/mmdit.rs:282-330) over the last axis, with a non-zero frozen
    scale, against the PyTorch f32 composition: values and the input gradient."""
    from loractl_b200.block_ops import zrmsnorm

    g = torch.Generator(device="cuda").manual_seed(4)
    x = (torch.randn(shape, generator=g, device="cuda") * 1.5 + 0.2).to(dtype)
    scale = torch.randn(shape[-1], generator=g, device="cuda") * 0.3
    dout = torch.randn(shape, generator=g, device="cuda").to(dtype)
    xs = x.clone().requires_grad_(True)
    out = zrmsnorm(xs, scale)
    out.backward(dout)
    xr = x.float().clone().requires_grad_(True)
    ref = xr / (xr.pow(2).mean(dim=-1, keepdim=True) + 1e-5).sqrt() * (scale + 1.0)
    ref.backward(dout.float())
    tol = 2e-5 if dtype == torch.float32 else 8e-3
    assert out.shape == x.shape and out.dtype == dtype
    assert rel(out, ref) <= tol and rel(xs.grad, xr.grad) <= tol

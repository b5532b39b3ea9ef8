"""Block-level parity at real widths: `harness.DoubleStreamBlock` (hidden 3072, 24 heads, MLP 12288,
every linear a LoRA'd int4 site through libloractl_b200, bf16 activations) against an f32 PyTorch
twin built from the DEQUANTIZED weights and the same LoRA factors, at a reduced token count.

What is compared: the block's output, the gradient with respect to its input, and every adapter
gradient (20 tensors).  The twin computes `x . dequant(W)^T + s (x . A) . B` with plain matmuls in
f32, torch's layer norm, attention and tanh-GELU, i.e. the reference's op sequence for a site
(crates/loractl-core/src/mmdit.rs:526-536, crates/loractl-core/src/lora.rs:199-203) around the same
block wiring; the bands are the bf16 bands of crates/loractl-core/tests/quant_mmdit.rs:165-226
widened for a ten-linear chain: output and dX within 3e-2 of their peak with cosine >= 0.999,
adapter gradients cosine >= 0.99."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def twin_forward(blk, state, cond, factors):
    """f32 restatement of `DoubleStreamBlock.forward`; `factors[path] = (A, B, scaling)` leaf tensors."""
    cfg = blk.cfg
    b, _, h = state.shape
    li = cfg.img_tokens

    def lin(stream, name, x):
        base = blk.bases[f"{stream}_{name}"]
        w = base.inner.weight.dequantize().float()  # [d_out, d_in]
        a, bb, s = factors[blk.path(stream, name)]
        return x @ w.t() + s * ((x @ a) @ bb)

    def ln_mod(x, shift, scale):
        return F.layer_norm(x, (h,)) * (1 + scale) + shift

    xs = {"img": state[:, :li], "txt": state[:, li:]}
    c = F.silu(cond)
    mods, qkvs = {}, {}
    for s_ in blk.STREAMS:
        mods[s_] = lin(s_, "mod", c).unsqueeze(1).chunk(6, dim=-1)
        shift, scale = mods[s_][0], mods[s_][1]
        qkvs[s_] = lin(s_, "qkv", ln_mod(xs[s_], shift, scale)).view(b, -1, 3, cfg.heads, h // cfg.heads)
    qkv = torch.cat([qkvs["img"], qkvs["txt"]], dim=1)
    q, k, v = (t.transpose(1, 2) for t in qkv.unbind(2))
    att = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, -1, h)
    atts = {"img": att[:, :li], "txt": att[:, li:]}
    outs = []
    for s_ in blk.STREAMS:
        _, _, gate1, shift2, scale2, gate2 = mods[s_]
        x = xs[s_] + gate1 * lin(s_, "out", atts[s_])
        xn = ln_mod(x, shift2, scale2)
        x = x + gate2 * lin(s_, "down", F.gelu(lin(s_, "up", xn), approximate="tanh"))
        outs.append(x)
    return torch.cat(outs, dim=1)


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-30))


def reldev(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def test_double_stream_block_matches_its_f32_twin_at_real_widths():
    import loractl_b200
    from loractl_b200.harness import BlockConfig, BlockStack

    cfg = BlockConfig(img_tokens=256, txt_tokens=64)  # hidden 3072, 24 heads, MLP 12288, int4 block 64
    dev = torch.device("cuda")
    stack = BlockStack(1, cfg, rank=16, alpha=16.0, device=dev, seed=5)
    blk = stack.blocks[0]
    g = torch.Generator(device=dev).manual_seed(3)
    b = 2
    state32 = torch.randn((b, cfg.img_tokens + cfg.txt_tokens, cfg.hidden), generator=g, device=dev)
    state32 = state32.to(torch.bfloat16).float()  # both sides start from the same bf16-representable values
    cond32 = torch.randn((b, cfg.hidden), generator=g, device=dev).to(torch.bfloat16).float()
    gout32 = torch.randn(state32.shape, generator=g, device=dev).to(torch.bfloat16).float()

    # ---- the library path: bf16 activations, fused LoRA-linear kernels ----
    stack.flat.zero_grad()
    x = state32.to(torch.bfloat16).requires_grad_(True)
    blk.cond = cond32.to(torch.bfloat16)
    out = blk(x)
    out.backward(gout32.to(torch.bfloat16))
    stack.flat.gather_autograd_grads()
    loractl_b200.check_device_status()
    got_grads = {d_path: (d.lora_a.grad.clone(), d.lora_b.grad.clone())
                 for d_path, d in zip(stack.adapters.targets, stack.adapters.deltas)}

    # ---- the f32 twin on dequantized weights ----
    factors = {}
    for path, d in zip(stack.adapters.targets, stack.adapters.deltas):
        a = d.lora_a.detach().clone().requires_grad_(True)
        bb = d.lora_b.detach().clone().requires_grad_(True)
        factors[path] = (a, bb, d.scaling)
    x32 = state32.clone().requires_grad_(True)
    ref = twin_forward(blk, x32, cond32, factors)
    ref.backward(gout32)

    assert torch.isfinite(out).all()
    assert reldev(out.float(), ref) <= 3e-2 and cosine(out.float(), ref) >= 0.999
    assert reldev(x.grad.float(), x32.grad) <= 3e-2 and cosine(x.grad.float(), x32.grad) >= 0.999
    worst = 1.0
    for path, (ga, gb) in got_grads.items():
        ra, rb = factors[path][0].grad, factors[path][1].grad
        for name, got, want in (("dA", ga, ra), ("dB", gb, rb)):
            c = cosine(got, want)
            worst = min(worst, c)
            assert c >= 0.99, (path, name, c)
            assert reldev(got, want) <= 8e-2, (path, name, reldev(got, want))
    assert worst >= 0.99

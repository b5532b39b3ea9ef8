"""The GPT-2-shaped caller of the hot path against the reference's tiny golden
(crates/loractl-core/tests/fixtures/gpt2_tiny_golden.json + tiny-gpt2/model.safetensors, pinned by
crates/loractl-core/tests/gpt2_lora_step.rs:94-172 and the gpt2 parity test at 1e-4).

  * CPU: the Plain model replays the golden's embed / block-0 / ln_f stages and logits within 1e-4,
    fused c_attn and split q/k/v alike; zero-initialised adapters on every site leave the logits
    bit-identical (gpt2_lora_step.rs:94-125); gradients reach A and B only.
  * GPU: with every projection quantized, the model equals its dequantized Plain twin to f32 noise,
    a zero-init attach is still a bit-identical no-op, and at the benchmark's widths (768 / 3072,
    int4 block 64, rank 8 on q/k/v/o, bf16) loss and adapter gradients match an f32 twin inside
    the bf16 band.
"""
import json
import pathlib

import numpy as np
import pytest
import torch
from safetensors.torch import load_file

from loractl_b200 import gpt2 as G
from loractl_b200.adapters import LoraConfig, TargetSpec, build_adapters

HERE = pathlib.Path(__file__).parent / "golden"


def golden():
    g = json.loads((HERE / "gpt2_tiny_golden.json").read_text())
    t = load_file(str(HERE / "gpt2_tiny.safetensors"))
    ids = torch.tensor(g["input_ids"], dtype=torch.long).reshape(1, -1)
    return g, t, ids


@pytest.mark.parametrize("split", [False, True])
def test_plain_model_replays_the_reference_golden_on_cpu(split):
    g, t, ids = golden()
    m = G.Gpt2.from_hf_tensors(G.Gpt2Config.tiny(), t, split_qkv=split)
    emb, b0, lnf = m.hidden_states(ids)
    shape = g["hidden_shape"]
    for name, got in (("hidden_after_embed", emb), ("hidden_after_block0", b0), ("hidden_after_lnf", lnf)):
        want = torch.tensor(g[name], dtype=torch.float32).reshape(shape)
        assert float((got[0] - want).abs().max()) <= 1e-4, name
    logits = m(ids)[0]
    want = torch.tensor(g["logits"], dtype=torch.float32).reshape(g["logits_shape"])
    assert float((logits - want).abs().max()) <= 1e-4
    assert int(logits[-1].argmax()) == int(want[-1].argmax())


def test_zero_init_attach_is_a_no_op_and_grads_route_to_the_adapters_on_cpu():
    g, t, ids = golden()
    m = G.Gpt2.from_hf_tensors(G.Gpt2Config.tiny(), t)
    sites = m.injectable_sites()
    assert [s.path.split(".", 3)[3] for s in sites[:4]] == ["attn.c_attn", "attn.c_proj", "mlp.c_fc", "mlp.c_proj"]
    assert len(sites) == 8 and (sites[0].d_in, sites[0].d_out) == (32, 96)
    ad = build_adapters(sites, LoraConfig(rank=4, alpha=8.0, targets=[TargetSpec(r"attn\.c_attn$")]), torch.device("cpu"))
    assert len(ad.deltas) == 2  # one per block
    base = m(ids)
    out = m(ids, ad)
    assert torch.equal(out, base)
    G.next_token_loss(out, ids).backward()
    assert all(not p.requires_grad for p in m.parameters())
    for d in ad.deltas:
        assert d.lora_b.grad is not None and float(d.lora_b.grad.abs().max()) > 0.0
        assert d.lora_a.grad is not None  # zero while B is zero, but routed


@pytest.mark.gpu
@pytest.mark.parametrize("split", [False, True])
def test_quantized_tiny_model_equals_its_dequantized_twin(split):
    g, t, ids = golden()
    ids = ids.cuda()
    q = G.Gpt2.from_hf_tensors(G.Gpt2Config.tiny(), t, split_qkv=split).cuda()
    done, left = q.into_quantized(8, block=32)
    assert left == 0 and done == (12 if split else 8)
    twin = G.Gpt2.from_hf_tensors(G.Gpt2Config.tiny(), t, split_qkv=split).cuda()
    with torch.no_grad():
        for (_, qb), (_, tb) in zip(q.base_linears(), twin.base_linears()):
            tb.as_plain().weight.copy_(qb.inner.dequantized_weight())
    a, b = q(ids), twin(ids)
    assert float((a - b).abs().max()) <= 2e-5 * float(b.abs().max())
    plain = G.Gpt2.from_hf_tensors(G.Gpt2Config.tiny(), t, split_qkv=split).cuda()
    ref = plain(ids)
    assert 0.0 < float((a - ref).abs().max()) <= 5e-2 * float(ref.abs().max())  # int8 band, quant_mmdit.rs:165-226
    ad = build_adapters(q.injectable_sites(), LoraConfig(rank=4, alpha=8.0, targets=[TargetSpec(r".*")]),
                        torch.device("cuda"))
    assert torch.equal(q(ids, ad), a)


@pytest.mark.gpu
def test_benchmark_width_stack_matches_an_f32_twin_in_the_bf16_band():
    """Two layers at the text benchmark's widths: int4 block-64 base, rank 8 on q/k/v/o, bf16
    activations, 2 x 256 tokens; the twin is Plain f32 on the dequantized weights with the same
    (non-zero) adapters."""
    import loractl_b200 as lb

    cfg = G.Gpt2Config(vocab_size=1000, n_positions=256, n_embd=768, n_layer=2, n_head=12, n_inner=3072)
    torch.manual_seed(3)
    m = G.Gpt2(cfg, split_qkv=True).cuda()
    with torch.no_grad():
        for _, base in m.base_linears():
            base.as_plain().weight.normal_(0, 0.02)
            base.as_plain().bias.normal_(0, 0.02)
        m.wte.weight.normal_(0, 0.02)
        m.wpe.weight.normal_(0, 0.01)
    twin = G.Gpt2(cfg, split_qkv=True).cuda()
    twin.load_state_dict(m.state_dict())
    assert m.into_quantized(4, block=64) == (12, 0)
    with torch.no_grad():
        for (_, qb), (_, tb) in zip(m.base_linears(), twin.base_linears()):
            tb.as_plain().weight.copy_(qb.inner.dequantized_weight())
    m = m.to(torch.bfloat16)
    lcfg = LoraConfig(rank=8, alpha=16.0, targets=[TargetSpec(r"attn\.(q|k|v|c_proj)$")])
    ad = build_adapters(m.injectable_sites(), lcfg, torch.device("cuda"))
    ad2 = build_adapters(twin.injectable_sites(), lcfg, torch.device("cuda"))
    assert len(ad.deltas) == 8
    g = torch.Generator(device="cuda").manual_seed(9)
    with torch.no_grad():
        for d, d2 in zip(ad.deltas, ad2.deltas):
            d.lora_b.copy_(torch.randn(d.lora_b.shape, generator=g, device="cuda") * 0.02)
            d2.lora_a.copy_(d.lora_a)
            d2.lora_b.copy_(d.lora_b)
    ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=g, device="cuda")
    loss = G.next_token_loss(m(ids, ad, dtype=torch.bfloat16), ids)
    loss.backward()
    lb.check_device_status()
    loss2 = G.next_token_loss(twin(ids, ad2), ids)
    loss2.backward()
    assert abs(float(loss) - float(loss2)) <= 2e-2 * abs(float(loss2))
    for d, d2 in zip(ad.deltas, ad2.deltas):
        for p, p2 in ((d.lora_a, d2.lora_a), (d.lora_b, d2.lora_b)):
            ga, gb = p.grad.float().cpu().numpy().ravel(), p2.grad.float().cpu().numpy().ravel()
            cos = float(ga @ gb / (np.linalg.norm(ga) * np.linalg.norm(gb) + 1e-30))
            assert cos >= 0.99, cos


@pytest.mark.gpu
def test_graphed_loss_step_replays_the_eager_step():
    """Forward + loss + backward of the text model captured as one CUDA graph (`GraphedLossStep`) over
    a fixed ids tensor and a flat gradient bucket: replaying it after copying new ids in gives the
    eager step's loss and adapter gradients (same kernels; the attention backward's atomic adds are
    the only noise), for two different batches."""
    import loractl_b200 as lb
    from loractl_b200.harness import GraphedLossStep
    from loractl_b200.optim import FlatAdapters

    cfg = G.Gpt2Config(vocab_size=512, n_positions=128, n_embd=256, n_layer=2, n_head=4, n_inner=1024)
    torch.manual_seed(3)
    m = G.Gpt2(cfg, split_qkv=True).cuda()
    with torch.no_grad():
        for _, base in m.base_linears():
            base.as_plain().weight.normal_(0, 0.02)
        m.wte.weight.normal_(0, 0.02)
        m.wpe.weight.normal_(0, 0.01)
    assert m.into_quantized(4, block=64) == (12, 0)
    m = m.to(torch.bfloat16)
    lcfg = LoraConfig(rank=8, alpha=16.0, targets=[TargetSpec(r"attn\.(q|k|v|c_proj)$")])
    ad = build_adapters(m.injectable_sites(), lcfg, torch.device("cuda"))
    g = torch.Generator(device="cuda").manual_seed(9)
    with torch.no_grad():
        for d in ad.deltas:
            d.lora_b.copy_(torch.randn(d.lora_b.shape, generator=g, device="cuda") * 0.02)
    flat = FlatAdapters(ad, torch.device("cuda"))
    flat.refresh_mirrors()
    ids = torch.randint(0, cfg.vocab_size, (4, 128), generator=g, device="cuda")
    fn = lambda: G.next_token_loss(m(ids, ad, dtype=torch.bfloat16), ids)
    step = GraphedLossStep(fn, torch.device("cuda"))
    for seed in (1, 2):
        new_ids = torch.randint(0, cfg.vocab_size, (4, 128), generator=torch.Generator(device="cuda").manual_seed(seed),
                                device="cuda")
        ids.copy_(new_ids)
        flat.zero_grad()
        loss_e = fn()
        loss_e.backward()
        flat.gather_autograd_grads()
        grads_e, le = flat.grads.clone(), float(loss_e)
        flat.zero_grad()
        lg = float(step.replay())
        flat.gather_autograd_grads()
        lb.check_device_status()
        assert abs(lg - le) <= 1e-5 * abs(le), (lg, le)
        assert float(grads_e.abs().max()) > 0
        assert float((flat.grads - grads_e).abs().max()) <= 1e-4 * float(grads_e.abs().max())

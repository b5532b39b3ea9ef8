"""GPU tests of streaming quantize-at-load (crates/loractl-core/src/diffusion_trainer.rs:1094-1267):
every quantizable weight of a checkpoint — f32, bf16, f16 and scaled fp8 with scalar or per-channel
`weight_scale` — must come out with exactly the codes and scales the oracle computes from the
decoded f32 values; sites with an unaligned d_in and 1-D tensors stay plain f32."""
import numpy as np
import pytest
import torch

from oracle import lq_oracle as O
from tests.util import host, seeded

pytestmark = pytest.mark.gpu


def make_checkpoint(path):
    from loractl_b200 import loader as LD

    t, f32vals = {}, {}

    def put_f32(name, a):
        t[name] = ("F32", a.shape, a.astype("<f4").tobytes())
        f32vals[name] = a.astype(np.float32)

    def put_half(name, a, tag):
        tt = torch.from_numpy(a).to(torch.bfloat16 if tag == "BF16" else torch.float16)
        t[name] = (tag, a.shape, tt.view(torch.int16).numpy().tobytes())
        f32vals[name] = tt.to(torch.float32).numpy()

    def put_fp8(name, a, per_channel):
        wb, sc = O.fp8_quantize(a, per_channel)
        t[name] = ("F8_E4M3", a.shape, wb.tobytes())
        t[name + "_scale"] = ("F32", sc.shape, np.asarray(sc, "<f4").tobytes())
        f32vals[name] = O.fp8_dequant(wb, sc)

    put_f32("blocks.0.attn.wq.weight", seeded((130, 128), 1, 0.02))
    put_half("blocks.0.attn.wk.weight", seeded((256, 320), 2, 0.02), "BF16")
    put_half("blocks.0.attn.wv.weight", seeded((64, 64), 3, 0.02), "F16")
    put_fp8("blocks.0.mlp.up.weight", seeded((264, 192), 4, 0.02), True)
    put_fp8("blocks.0.mlp.down.weight", seeded((192, 256), 5, 0.02), False)
    put_fp8("blocks.0.odd.weight", seeded((8, 72), 6, 0.02), True)       # d_in % 64 != 0: stays plain
    put_f32("blocks.0.norm.weight", seeded((128,), 7))                    # 1-D: plain
    put_f32("blocks.0.attn.wq.bias", seeded((130,), 8))
    LD.write_safetensors(path, t, {"format": "pt"})
    return f32vals


@pytest.mark.parametrize("bits,block", [(4, 64), (8, 32), (4, 32)])
def test_loaded_handles_are_bit_exact_against_the_oracle(tmp_path, bits, block):
    from loractl_b200 import loader as LD

    p = tmp_path / "ckpt.safetensors"
    vals = make_checkpoint(p)
    seen = []
    handles, plain, rep = LD.load_quant_module(p, torch.device("cuda"), bits=bits, block=block,
                                               progress=lambda n, i, tot: seen.append((n, i, tot)))
    quantized = {n for n, v in vals.items() if v.ndim == 2 and v.shape[1] % block == 0}
    assert set(handles) == quantized and set(plain) == set(vals) - quantized
    assert rep.quantized == len(quantized) and rep.left_plain == len(vals) - len(quantized) and rep.kept_fp8 == 0
    assert seen[-1] == ("", len(vals), len(vals)) and seen[0][1:] == (0, len(vals))
    for name in quantized:
        codes, scales = handles[name].unpack()
        oc, osc = O.quantize(vals[name], block, bits)
        assert np.array_equal(host(codes).astype(np.int8), oc), name
        assert np.array_equal(host(scales), osc), name
    for name in plain:
        assert np.array_equal(host(plain[name]), vals[name]), name
    assert rep.packed_bytes == sum(h.packed_bytes + h.scale_bytes for h in handles.values()) > 0


def test_keep_fp8_keeps_the_bytes_resident(tmp_path):
    from loractl_b200 import _lib as L
    from loractl_b200 import loader as LD

    p = tmp_path / "ckpt.safetensors"
    vals = make_checkpoint(p)
    handles, plain, rep = LD.load_quant_module(p, torch.device("cuda"), bits=4, block=64, keep_fp8=True)
    assert rep.kept_fp8 == 3 and handles["blocks.0.mlp.up.weight"].scheme == L.LQ_FP8_E4M3
    for name in ("blocks.0.mlp.up.weight", "blocks.0.mlp.down.weight", "blocks.0.odd.weight"):
        assert np.array_equal(host(handles[name].dequantize(torch.float32)), vals[name])
    assert handles["blocks.0.attn.wq.weight"].scheme == L.LQ_INT4


def test_requantize_from_fp8_equals_dequantize_then_quantize_at_site_size():
    """The fused kernel against the two-step route through an f32 tensor, 3072 x 3072."""
    import ctypes as C

    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200 import quant as Q

    dev = torch.device("cuda")
    w = torch.randn((3072, 3072), device=dev) * 0.02
    f8 = lb.fp8_quantize(w, True)
    wb, sc = f8.unpack()
    two_step = lb.quantize_linear_weight(f8.dequantize(torch.float32), 4, 64)
    out = C.c_void_p()
    L.check(L.lib().lq_quantize_from_fp8(wb.data_ptr(), sc.data_ptr(), L.LQ_SCALE_PER_CHANNEL, 3072, 3072, 64, 4,
                                         Q._stream_ptr(dev), C.byref(out)))
    fused = Q.QuantWeight(out.value, dev)
    c1, s1 = two_step.unpack()
    c2, s2 = fused.unpack()
    assert torch.equal(c1, c2) and torch.equal(s1, s2)


def test_bad_checkpoint_fails_before_any_upload(tmp_path):
    from loractl_b200 import loader as LD

    p = tmp_path / "bad.safetensors"
    LD.write_safetensors(p, {"a.weight": ("F8_E4M3", (4, 64), bytes(256))})
    with pytest.raises(LD.CheckpointError, match="sidecar"):
        LD.load_quant_module(p, torch.device("cuda"))

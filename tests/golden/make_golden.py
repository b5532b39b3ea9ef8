"""Regenerates the golden vectors under tests/golden/.

Run where the loractl reference checkout is available:

    python tests/golden/make_golden.py /path/to/loractl

It writes two kinds of fixtures, all small JSON:

1. Pass-through copies of the vectors the reference's own tests pin for this
   path (crates/loractl-core/tests/fixtures/quant_int4_golden.json,
   quant_int8_golden.json, fp8_lut_golden.json, fp8_dequant_golden.json and
   crates/loractl-core/tests/golden/lora_toy.json, lora_export.json,
   krea2_lora_keys.json), re-emitted unchanged, plus the
   fixed constants of reference/lora_reference.py:39-66 (W_BASE, A_INIT, X, T)
   that the toy replays.
2. Extra vectors produced by *importing the reference's Python generators*
   (reference/quant_int4_reference.py, reference/quant_reference.py) with the
   block size patched to 64 and larger seeded shapes, and by torch's own
   `float8_e4m3fn` cast following reference/fp8_reference.py:84-94 (that module
   itself needs `diffusers`, which is not installed, so its three-line
   `quantize` is restated here around the same torch cast).

The tests only read the JSON; they never import the reference.
"""
from __future__ import annotations

import importlib
import json
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent


def passthrough(ref: pathlib.Path) -> None:
    core = ref / "crates" / "loractl-core" / "tests"
    for rel in (
        "fixtures/quant_int4_golden.json",
        "fixtures/quant_int8_golden.json",
        "fixtures/fp8_lut_golden.json",
        "fixtures/fp8_dequant_golden.json",
        "golden/lora_toy.json",
        "golden/lora_export.json",
        "golden/krea2_lora_keys.json",
    ):
        data = json.loads((core / rel).read_text())
        (HERE / pathlib.Path(rel).name).write_text(json.dumps(data))
        print("copied", rel)


def lora_toy_inputs(ref: pathlib.Path) -> None:
    """The constants block of reference/lora_reference.py, evaluated as-is."""
    src = (ref / "reference" / "lora_reference.py").read_text()
    head = src.split("def run_torch", 1)[0]
    ns: dict = {}
    exec(compile(head, "lora_reference_constants", "exec"), ns)  # constants only, no RNG
    out = {
        "d_in": ns["D_IN"], "d_out": ns["D_OUT"], "rank": ns["RANK"], "alpha": ns["ALPHA"],
        "lr": ns["LR"], "steps": ns["STEPS"],
        "w_base": ns["W_BASE"].tolist(), "a_init": ns["A_INIT"].tolist(),
        "x": ns["X"].tolist(), "t": ns["T"].tolist(),
    }
    (HERE / "lora_toy_inputs.json").write_text(json.dumps(out))
    print("wrote lora_toy_inputs.json")


def quant_extra(ref: pathlib.Path) -> None:
    """dq / y from the reference generators at block 32 and 64 on wider shapes."""
    sys.path.insert(0, str(ref / "reference"))
    cases = []
    for modname, bits in (("quant_int4_reference", 4), ("quant_reference", 8)):
        mod = importlib.import_module(modname)
        for block, (m, k, n), seed in ((32, (16, 96, 5), 11), (64, (12, 128, 6), 12), (64, (8, 64, 3), 13)):
            mod.BLOCK = block
            s = seed
            while True:  # the generator asserts tie-freeness; walk seeds until it holds
                torch.manual_seed(s)
                w = torch.randn(m, k, dtype=torch.float32) * 0.02
                try:
                    dq = mod.quantize_per_block(w)
                    break
                except AssertionError:
                    s += 100
            torch.manual_seed(s + 1)
            x = torch.randn(n, k, dtype=torch.float32)
            y = x @ dq.T
            cases.append({
                "bits": bits, "block": block, "seed": s,
                "w": w.numpy().tolist(), "x": x.numpy().tolist(),
                "dq": dq.numpy().tolist(), "y": y.numpy().tolist(),
            })
        mod.BLOCK = 32
    (HERE / "quant_extra_golden.json").write_text(json.dumps({"cases": cases}))
    print("wrote quant_extra_golden.json", len(cases), "cases")


def fp8_encode() -> None:
    """torch's e4m3fn cast on seeded weights, scalar and per-channel scale."""
    fp8_max = 448.0
    g = torch.Generator().manual_seed(21)
    cases = []
    for per_channel, shape in ((False, (6, 16)), (True, (6, 16)), (True, (12, 32))):
        w = torch.randn(*shape, generator=g) * 0.02
        if per_channel:
            scale = (w.abs().amax(dim=1) / fp8_max).clamp(min=1e-12)
            q = (w / scale[:, None]).to(torch.float8_e4m3fn)
            dq = q.float() * scale[:, None]
        else:
            scale = (w.abs().amax() / fp8_max).clamp(min=1e-12)
            q = (w / scale).to(torch.float8_e4m3fn)
            dq = q.float() * scale
        cases.append({
            "per_channel": per_channel, "shape": list(shape),
            "w": w.numpy().tolist(),
            "scale": scale.to(torch.float32).numpy().tolist(),
            "bytes": q.view(torch.uint8).numpy().tolist(),
            "dq": dq.numpy().tolist(),
        })
    # every finite f32 that sits on or next to an e4m3 rounding boundary
    lut = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    pos = lut[:0x7F]
    mids = (pos[:-1] + pos[1:]) / 2
    probes = torch.cat([pos, mids, torch.nextafter(mids, torch.tensor(1e9)),
                        torch.nextafter(mids, torch.tensor(-1e9)), torch.tensor([455.9, 463.9])])
    probes = torch.cat([probes, -probes])
    enc = probes.to(torch.float8_e4m3fn).view(torch.uint8)
    cases_b = {"x": probes.numpy().astype(np.float32).tolist(), "bytes": enc.numpy().tolist()}
    (HERE / "fp8_encode_golden.json").write_text(json.dumps({"cases": cases, "boundaries": cases_b}))
    print("wrote fp8_encode_golden.json")


def mmdit_block0(ref: pathlib.Path) -> None:
    """Block 0 of the reference's tiny MMDiT trace, cut out of its golden: the stage tensors either
    side of the first trunk block (crates/loractl-core/tests/fixtures/mmdit_tiny_golden.json:
    after_first, after_txtmlp, tvec, pos, txtmask -> after_block0) and that block's tensors from
    tests/fixtures/tiny-mmdit/model.safetensors, as one small safetensors file (values unchanged,
    stored as f32)."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    fx = ref / "crates" / "loractl-core" / "tests" / "fixtures"
    g = json.loads((fx / "mmdit_tiny_golden.json").read_text())
    out = {}
    for name in ("after_first", "after_txtmlp", "tvec", "pos", "after_block0"):
        out[f"stage.{name}"] = torch.tensor(g[name], dtype=torch.float64).reshape(g[f"{name}_shape"]).to(torch.float32)
    out["stage.txtmask"] = torch.tensor(g["txtmask"], dtype=torch.float32)
    with safe_open(str(fx / "tiny-mmdit" / "model.safetensors"), "pt") as f:
        for k in f.keys():
            if k.startswith("blocks.0."):
                out[k] = f.get_tensor(k).to(torch.float32).contiguous()
    cfg = {k: str(g["config"][k]) for k in ("features", "heads", "kvheads", "multiplier")}
    save_file(out, str(HERE / "mmdit_tiny_block0.safetensors"), metadata=cfg)
    print("wrote mmdit_tiny_block0.safetensors", len(out), "tensors")


def gpt2_tiny(ref: pathlib.Path) -> None:
    """Pass-through of the reference's tiny GPT-2 fixture (weights and golden logits,
    crates/loractl-core/tests/fixtures/gpt2_tiny_golden.json, tiny-gpt2/model.safetensors)."""
    import shutil

    fx = ref / "crates" / "loractl-core" / "tests" / "fixtures"
    (HERE / "gpt2_tiny_golden.json").write_text(json.dumps(json.loads((fx / "gpt2_tiny_golden.json").read_text())))
    shutil.copyfile(fx / "tiny-gpt2" / "model.safetensors", HERE / "gpt2_tiny.safetensors")
    print("copied gpt2 tiny fixture")


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to the loractl checkout>")
    ref = pathlib.Path(sys.argv[1])
    passthrough(ref)
    mmdit_block0(ref)
    gpt2_tiny(ref)
    lora_toy_inputs(ref)
    quant_extra(ref)
    fp8_encode()


if __name__ == "__main__":
    main()

"""The reference arm of bench.py runs on the host alone: one JSON line with the keys the
measurement contract names, on the CPU restatement of the reference's op sequence."""
import json
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "cfg1",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip().startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["config"]["workload"] == "cfg1"
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "tokens" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_flop_model_matches_the_stated_figures():
    sys.path.insert(0, str(ROOT))
    import bench

    # 4NKM + 6Nr(K + M): the two headline workloads
    assert bench.step_flops(4096, 3072, 3072, 16) == 157_034_741_760
    assert bench.step_flops(8192, 3072, 12288, 32) == 1_261_109_772_288

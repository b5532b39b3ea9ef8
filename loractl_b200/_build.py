"""Builds libloractl_b200.so in-tree with nvcc for sm_100a.

Usage: `python -m loractl_b200._build` (or `__graft_entry__.build()`).  nvcc
cross-compiles without a GPU; the resulting `lib/libloractl_b200.so` is what
`loractl_b200._lib` loads.
"""
from __future__ import annotations

import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "libloractl_b200.so"
SOURCES = ["lq_api.cu", "lq_quant.cu", "lq_simt.cu", "lq_tc.cu", "lq_prof.cu", "lq_step.cu", "lq_fused.cu", "lq_block.cu"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "loractl_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not needs_build():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    LIB.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIB), *[str(CSRC / s) for s in SOURCES]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

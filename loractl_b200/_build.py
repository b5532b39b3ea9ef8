"""Builds libloractl_b200.so in-tree with nvcc for sm_100a.

Usage: `python -m loractl_b200._build` (or `__graft_entry__.build()`).  nvcc
cross-compiles without a GPU; the resulting `lib/libloractl_b200.so` is what
`loractl_b200._lib` loads.  Every translation unit is compiled to its own object
(in parallel, and only when it or a header changed), then linked; internal C++
symbols are hidden, only the C ABI of include/loractl_b200.h is exported.
"""
from __future__ import annotations

import concurrent.futures
import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "lib" / "obj"
LIB = PKG / "lib" / "libloractl_b200.so"
HEADER = PKG.parent / "include" / "loractl_b200.h"
SOURCES = ["lq_api.cu", "lq_quant.cu", "lq_simt.cu", "lq_tc.cu", "lq_w4.cu", "lq_prof.cu", "lq_step.cu", "lq_fused.cu", "lq_bwd_small.cu",
           "lq_block.cu"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _headers_mtime() -> float:
    return max(p.stat().st_mtime for p in [*CSRC.glob("*.cuh"), HEADER])


def _stale(out: pathlib.Path, deps_mtime: float) -> bool:
    return not out.exists() or out.stat().st_mtime < deps_mtime


def needs_build() -> bool:
    hdr = _headers_mtime()
    if _stale(LIB, hdr):
        return True
    return any((CSRC / s).stat().st_mtime > LIB.stat().st_mtime for s in SOURCES)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not needs_build():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    OBJ.mkdir(parents=True, exist_ok=True)
    hdr = _headers_mtime()

    def compile_one(src: str):
        obj = OBJ / (src[:-3] + ".o")
        if not force and not _stale(obj, max(hdr, (CSRC / src).stat().st_mtime)):
            return obj, ""
        cmd = [nvcc, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", "-o", str(obj), str(CSRC / src)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src} ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
        return obj, proc.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    if verbose:
        for _, log in results:
            if log:
                print(log)
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xlinker",
            f"--version-script={CSRC / 'exports.map'}", "-o", str(LIB), *[str(o) for o, _ in results]]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

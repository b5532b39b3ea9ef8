"""Builds the C oracle (test infrastructure) into oracle/_ref/liblq_oracle.so with gcc.

The reference itself is a Rust workspace on burn 0.21 with no C/C++ sources, and no Rust
toolchain exists here, so there is no reference binary to compile: `oracle/_ref/` holds only
this restatement's shared object."""
from __future__ import annotations

import pathlib
import shutil
import subprocess

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref" / "liblq_oracle.so"


def build(force: bool = False) -> pathlib.Path:
    src = HERE / "lq_oracle.c"
    if not force and OUT.exists() and OUT.stat().st_mtime >= src.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(parents=True, exist_ok=True)
    gcc = shutil.which("gcc") or "gcc"
    cmd = [gcc, "-O2", "-fno-fast-math", "-ffp-contract=off", "-shared", "-fPIC", "-o", str(OUT), str(src), "-lm"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"gcc failed:\n{proc.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(force=True))

"""Builds the C part of the oracle (oracle/w8a8_oracle.c) into oracle/_build/.

The reference's own native code for this path is CUDA compiled against ATen through
torch's JIT extension loader, so there is nothing under the reference tree that
gcc/g++ could compile into a CPU ``oracle/_ref``; the Python reference is used
instead to pin the oracle (tests/golden/make_golden.py).
"""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_build" / "libw8a8_oracle.so"


def build(force: bool = False) -> Path:
    src = HERE / "w8a8_oracle.c"
    if OUT.exists() and not force and OUT.stat().st_mtime >= src.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    subprocess.run(["gcc", "-O3", "-fopenmp", "-shared", "-fPIC", str(src), "-o", str(OUT)], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))

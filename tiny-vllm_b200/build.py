"""Builds libb200q.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Run as ``python tiny-vllm_b200/build.py`` or call :func:`build`.  The library is
written to ``tiny-vllm_b200/lib/libb200q.so``; a hash of the sources and flags is
kept beside it so that an up-to-date library is not rebuilt.  nvcc cross-compiles
for sm_100a without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libb200q.so"
HEADER = PKG_DIR.parent / "include" / "b200q.h"

SOURCES = ["api.cu", "act_quant.cu", "act_quant_fused.cu", "gemm_simt.cu", "gemm_umma.cu", "gemm_umma_w8a16.cu", "gemm_umma_w8a16_ts.cu",
           "gemm_umma_pair.cu", "gemm_mma_decode.cu", "gemm_bulk_decode.cu", "tp_allreduce.cu", "tp_reduce_norm_quant.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: set NVCC or add the CUDA toolkit to PATH")
    return cand


def _source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    files = sorted(CSRC.glob("*")) + [HEADER]
    for f in files:
        if f.is_file():
            h.update(f.name.encode())
            h.update(f.read_bytes())
    return h.hexdigest()


def is_current() -> bool:
    stamp = LIB_DIR / ".build_hash"
    return LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == _source_hash()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every .cu of csrc/ and links the shared library.  Returns its path."""
    if not force and is_current():
        return LIB_PATH
    nvcc = _nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(name: str) -> Path:
        obj = obj_dir / (Path(name).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(CSRC / name), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *[str(o) for o in objs],
           "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xlinker", "--no-undefined"]      # a launcher missing from every .cu fails the build
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link of libb200q.so failed")
    (LIB_DIR / ".build_hash").write_text(_source_hash())
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)

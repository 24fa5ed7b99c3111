"""Builds ``oracle/_ref/`` — the REFERENCE ITSELF for the quantized-linear path.  TEST INFRASTRUCTURE.

What this recipe does, from the reference checkout where it lies (first argument, else
``$NANOVLLM_REFERENCE``, else ``/root/reference``); nothing is written anywhere but
``oracle/_ref/``, which is git-ignored (it travels with a snapshot of the tree like every
other built artefact, so a machine without the checkout can still run it):

1. the reference's Python package ``nanovllm/`` (and its artifact tool ``scripts/quantize.py``)
   is mirrored to ``oracle/_ref/nanovllm/`` (``oracle/_ref/scripts/``) so
   that its own functions — ``quantize_int8_per_row_dynamic``, ``w8a8_linear_fallback``,
   ``int8_weight_only_linear_fallback``, ``apply_w8a8_linear``,
   ``apply_int8_weight_only_linear`` — can be imported unmodified;
2. the reference's two CUDA extensions (``quantization/csrc/w8a8_gemm.{cpp,cu}``,
   ``int8_weight_only_gemm.{cpp,cu}``) are compiled from those sources with torch's extension
   builder, the reference's own flags (``nanovllm/quantization/cuda.py:146-222``) plus the
   sm_100a code generation flag, into ``oracle/_ref/ext/<name>/<name>.so``.

:func:`load_reference` imports the mirrored package and points its lazy extension loaders at
the prebuilt libraries (the reference would otherwise JIT-compile the same sources on first
use).  Only ``tests/``, ``__graft_entry__`` and ``bench.py``'s reference legs use this module.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
EXTENSIONS = {
    "nanovllm_w8a8_cuda": ["w8a8_gemm.cpp", "w8a8_gemm.cu"],
    "nanovllm_int8_weight_only_cuda": ["int8_weight_only_gemm.cpp", "int8_weight_only_gemm.cu"],
}


def reference_checkout(where: str | None = None) -> Path | None:
    cand = where or os.environ.get("NANOVLLM_REFERENCE") or "/root/reference"
    p = Path(cand)
    return p if (p / "nanovllm" / "quantization" / "cuda.py").is_file() else None


def build(where: str | None = None, force: bool = False, verbose: bool = False) -> Path | None:
    """Mirrors the package and compiles the extensions.  Returns ``oracle/_ref`` or ``None``
    when no reference checkout is available (an existing ``oracle/_ref`` is left as it is)."""
    src = reference_checkout(where)
    if src is None:
        return REF_DIR if (REF_DIR / "nanovllm").is_dir() else None
    pkg = REF_DIR / "nanovllm"
    REF_DIR.mkdir(exist_ok=True)
    shutil.copytree(src / "nanovllm", pkg, dirs_exist_ok=True,
                    ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    if (src / "scripts" / "quantize.py").is_file():   # the reference's offline artifact tool
        (REF_DIR / "scripts").mkdir(exist_ok=True)
        shutil.copyfile(src / "scripts" / "quantize.py", REF_DIR / "scripts" / "quantize.py")
    for path in [pkg, *pkg.rglob("*")]:          # the checkout may be read-only; the mirror is not
        path.chmod(path.stat().st_mode | 0o200)
    from torch.utils.cpp_extension import load

    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    csrc = pkg / "quantization" / "csrc"
    for name, files in EXTENSIONS.items():
        out_dir = REF_DIR / "ext" / name
        lib = out_dir / f"{name}.so"
        sources = [csrc / f for f in files]
        if lib.exists() and not force and all(lib.stat().st_mtime >= s.stat().st_mtime for s in sources):
            continue
        out_dir.mkdir(parents=True, exist_ok=True)
        # flags of nanovllm/quantization/cuda.py:146-222, plus the target architecture
        load(name=name, sources=[str(s) for s in sources], extra_cflags=["-O3"],
             extra_cuda_cflags=["-O3", "--use_fast_math", "--expt-relaxed-constexpr",
                                "-gencode", "arch=compute_100a,code=sm_100a"],
             build_directory=str(out_dir), verbose=verbose)
    return REF_DIR


class Reference:
    """Handles to the reference's own functions (attributes are the reference's modules)."""

    def __init__(self, utils, cuda, native_w8a8: bool, native_w8a16: bool):
        self.utils = utils
        self.cuda = cuda
        self.native_w8a8 = native_w8a8        # its CUDA W8A8 extension is loaded
        self.native_w8a16 = native_w8a16      # its CUDA W8A16 extension is loaded


def _import_prebuilt(name: str):
    lib = REF_DIR / "ext" / name / f"{name}.so"
    if not lib.exists():
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(name, lib)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_cached: Reference | None = None


def load_reference(with_cuda_extensions: bool = False) -> Reference | None:
    """Imports the mirrored reference package (``None`` when ``oracle/_ref`` was never built).
    With ``with_cuda_extensions`` the reference's lazy extension loaders are replaced by
    functions returning the prebuilt libraries; everything else is the reference's code."""
    global _cached
    if not (REF_DIR / "nanovllm" / "quantization" / "cuda.py").is_file():
        return None
    if _cached is None:
        if str(REF_DIR) not in sys.path:
            sys.path.insert(0, str(REF_DIR))
        utils = importlib.import_module("nanovllm.quantization.utils")
        cuda = importlib.import_module("nanovllm.quantization.cuda")
        if Path(cuda.__file__).resolve().parent.parent.parent != REF_DIR.resolve():
            raise RuntimeError("another nanovllm package shadows oracle/_ref/nanovllm")
        _cached = Reference(utils, cuda, False, False)
    if with_cuda_extensions and not (_cached.native_w8a8 and _cached.native_w8a16):
        w8a8 = _import_prebuilt("nanovllm_w8a8_cuda")
        w8a16 = _import_prebuilt("nanovllm_int8_weight_only_cuda")
        if w8a8 is not None:
            _cached.cuda._load_w8a8_extension = lambda: w8a8
            _cached.native_w8a8 = True
        if w8a16 is not None:
            _cached.cuda._load_native_extension = lambda: w8a16
            _cached.native_w8a16 = True
    return _cached


if __name__ == "__main__":
    out = build(sys.argv[1] if len(sys.argv) > 1 else None, force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(out if out is not None else "no reference checkout found; oracle/_ref not built")

"""Installs this package under the reference's module names, so that the reference's own model
code, loader and runner use these layers without being edited.

``install_under_nanovllm()`` makes ``import nanovllm.layers.linear`` and
``import nanovllm.quantization`` (and its sub-modules ``base``, ``int8``, ``w8a8``, ``utils``,
``cuda``) resolve to the modules of this package, which export the same names with the same
constructors, attributes and loader hooks (``nanovllm/layers/linear.py:14-276``,
``nanovllm/quantization/*.py``).  Everything else of ``nanovllm`` — ``models/qwen3.py``, the
engine, ``utils/loader.py`` — is imported from the reference as it is.  Call it before the first
``import nanovllm`` in EVERY process (the reference spawns its tensor-parallel workers, which
import ``nanovllm`` again: ``nanovllm/engine/llm_engine.py:25-31``).
"""
from __future__ import annotations

import sys


def install_under_nanovllm(replace_loader: bool = False) -> list[str]:
    """Registers the aliases; returns the module names that were installed.  With
    ``replace_loader`` the reference's ``nanovllm.utils.loader`` is replaced too (same
    ``load_model`` call, but each rank reads only its own share of every weight)."""
    from . import quantization
    from .layers import linear
    from .quantization import base, cuda, int8, utils, w8a8
    from .utils import loader

    aliases = {
        "nanovllm.layers.linear": linear,
        "nanovllm.quantization": quantization,
        "nanovllm.quantization.base": base,
        "nanovllm.quantization.int8": int8,
        "nanovllm.quantization.w8a8": w8a8,
        "nanovllm.quantization.utils": utils,
        "nanovllm.quantization.cuda": cuda,
    }
    if replace_loader:
        aliases["nanovllm.utils.loader"] = loader
    already = [name for name in aliases if name in sys.modules and sys.modules[name] is not aliases[name]]
    if already:
        raise RuntimeError(f"the reference's modules are imported already: {already}; install the "
                           "aliases before the first `import nanovllm`")
    sys.modules.update(aliases)
    return sorted(aliases)

"""Import shim: makes the directory ``tiny-vllm_b200/`` importable as the package
``tiny_vllm_b200`` (a hyphen cannot appear in a Python module name).

``import tiny_vllm_b200`` from the repository root executes the package's
``__init__.py`` in this module's namespace and points ``__path__`` at the
directory, so ``tiny_vllm_b200.quantization`` etc. resolve to the files inside it.
"""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "tiny-vllm_b200")]
__file__ = _os.path.join(__path__[0], "__init__.py")
with open(__file__, "r", encoding="utf-8") as _f:
    exec(compile(_f.read(), __file__, "exec"))
del _f, _os

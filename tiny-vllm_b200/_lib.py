"""ctypes binding of ``libb200q.so`` — the C ABI declared in ``include/b200q.h``.

The library is loaded from ``tiny-vllm_b200/lib/`` (built in-tree by
``build.py``).  There is no other implementation behind these calls: if the
library is missing, :func:`lib` raises instead of degrading to a CPU path.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = _PKG_DIR / "lib" / "libb200q.so"

# error codes / enums of include/b200q.h
OK = 0
ERR_NULL_POINTER = 1
ERR_BAD_SHAPE = 2
ERR_UNSUPPORTED_SHAPE = 3
ERR_MISALIGNED = 4
ERR_WORKSPACE = 5
ERR_UNSUPPORTED_ARCH = 6
ERR_LAUNCH = 7
ERR_BAD_ARGUMENT = 8
ERR_DEVICE_TIMEOUT = 9
ERR_SCRATCH_LIMIT = 10
NOALLOC_SCRATCH_BYTES = 8 << 20

DTYPE_F16 = 0
DTYPE_BF16 = 1

OP_ACT_QUANT = 0
OP_W8A8 = 1
OP_W8A16 = 2

PATH_AUTO = 0
PATH_SIMT_STREAM = 1
PATH_UMMA = 2
PATH_UMMA_SWAP = 3
PATH_MMA_STREAM = 4

# every symbol include/b200q.h declares: name -> (restype, argtypes)
_c = ctypes
SIGNATURES = {
    "b200q_act_quant_i8": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int, _c.c_void_p, _c.c_void_p,
                                      _c.c_int, _c.c_int, _c.c_void_p]),
    "b200q_w8a8_gemm": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                   _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                   _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "b200q_w8a8_gemm_i32": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int,
                                       _c.c_int, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "b200q_w8a16_gemm": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                    _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p,
                                    _c.c_size_t, _c.c_void_p]),
    "b200q_workspace_bytes": (_c.c_size_t, [_c.c_int, _c.c_int, _c.c_int, _c.c_int]),
    "b200q_select_path": (_c.c_char_p, [_c.c_int, _c.c_int, _c.c_int, _c.c_int]),
    "b200q_strerror": (_c.c_char_p, [_c.c_int]),
    "b200q_last_cuda_error": (_c.c_int, []),
    "b200q_device_status": (_c.c_int, []),
    "b200q_version": (_c.c_int, []),
    "b200q_debug_force_path": (_c.c_int, [_c.c_int]),
    "b200q_launch_count": (_c.c_uint64, []),
    "b200q_tp_allreduce": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_size_t,
                                      _c.c_int, _c.c_void_p]),
    "b200q_w8a8_gemm_allreduce": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                             _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int,
                                             _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_size_t,
                                             _c.c_int, _c.c_int, _c.c_void_p]),
    "b200q_w8a16_gemm_allreduce": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                              _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                              _c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_int,
                                              _c.c_int, _c.c_void_p]),
    "b200q_w8a8_gemm_allreduce_tiled": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                                   _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int,
                                                   _c.c_int, _c.c_int, _c.c_void_p, _c.c_size_t,
                                                   _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p]),
    "b200q_add_rmsnorm_quant_i8": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_float,
                                              _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                              _c.c_int, _c.c_int, _c.c_int, _c.c_void_p]),
    "b200q_silu_mul_quant_i8": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p,
                                           _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p]),
    "b200q_tp_allreduce_multimem": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int,
                                               _c.c_size_t, _c.c_int, _c.c_void_p]),
    "b200q_tp_allreduce_pull": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int,
                                           _c.c_size_t, _c.c_int, _c.c_void_p]),
    "b200q_tp_allreduce_small": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_int,
                                            _c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_int,
                                            _c.c_int, _c.c_void_p]),
    "b200q_w8a8_gemm_noalloc": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                           _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int,
                                           _c.c_int, _c.c_void_p]),
}

_lock = threading.Lock()
_lib = None


class B200QError(RuntimeError):
    """A libb200q entry point returned a non-zero code."""

    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        text = lib().b200q_strerror(code).decode()
        msg = f"{where}: {text} (code {code})"
        if code == ERR_LAUNCH:
            msg += f", cudaError {lib().b200q_last_cuda_error()}"
        if detail:
            msg += f" [{detail}]"
        super().__init__(msg)


def lib() -> ctypes.CDLL:
    """Loads the shared library once and sets the prototypes.  Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python tiny-vllm_b200/build.py` "
                    "(there is no fallback implementation)")
            handle = ctypes.CDLL(str(LIB_PATH))
            for name, (restype, argtypes) in SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype = restype
                fn.argtypes = argtypes
            _lib = handle
    return _lib


def check(code: int, where: str, detail: str = "") -> None:
    if code != OK:
        raise B200QError(code, where, detail)

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

# debug knobs (B200Q_KNOB_*): settings are private to the calling thread, unset at load
KNOB_FORCE_PATH = 0
KNOB_FLAGS = 1
KNOB_BN = 2
KNOB_SPLITS = 3
KNOB_CLUSTER = 4
KNOB_NO_PAIR = 5
KNOB_NO_TS = 6
KNOB_TS_MIN_K = 7
KNOB_SIMT_MAX_M = 8
KNOB_TILED_ONLY = 9
KNOB_PAIR_EPILOGUE = 10
KNOB_W8A16_PAIR_MIN_M = 11
KNOB_NO_PDL = 12
KNOB_WAIT_CYCLES = 13
KNOB_PAIR_MIN_TILES = 14
KNOB_BULK_DECODE = 15
KNOB_BULK_SLOTS = 16
KNOB_BULK_WPP = 17

# B200Q_VERSION of include/b200q.h this binding was written for
ABI_VERSION = 2

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
    "b200q_debug_set": (_c.c_int, [_c.c_int, _c.c_int]),
    "b200q_debug_reset": (None, []),
    "b200q_check_status": (_c.c_int, [_c.POINTER(_c.c_int)]),
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
    "b200q_tp_reduce_rmsnorm_quant": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                                 _c.c_void_p, _c.c_float, _c.c_void_p, _c.c_void_p,
                                                 _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
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
            from . import build as _build
            if not _build.is_current():
                raise RuntimeError(
                    f"{LIB_PATH} was not built from the current csrc/ and include/b200q.h "
                    "(source hash differs): run `python tiny-vllm_b200/build.py`")
            handle = ctypes.CDLL(str(LIB_PATH))
            for name, (restype, argtypes) in SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype = restype
                fn.argtypes = argtypes
            if handle.b200q_version() != ABI_VERSION:
                raise RuntimeError(
                    f"{LIB_PATH} reports ABI version {handle.b200q_version()}, this binding expects "
                    f"{ABI_VERSION}: rebuild with `python tiny-vllm_b200/build.py`")
            _lib = handle
    return _lib


def check_device(where: str = "device status") -> None:
    """Synchronous: reads and clears the device status word of the current device and raises
    :class:`B200QError` (``ERR_DEVICE_TIMEOUT``) when a bounded device-side wait gave up since
    the last read.  Call it after synchronising the stream."""
    word = ctypes.c_int(0)
    rc = lib().b200q_check_status(ctypes.byref(word))
    if rc != OK:
        raise B200QError(rc, where, f"status word 0x{word.value & 0xFFFFFFFF:x}")


def check(code: int, where: str, detail: str = "") -> None:
    if code != OK:
        raise B200QError(code, where, detail)

"""Helpers of the GPU parity tests."""
import contextlib

import torch

import tiny_vllm_b200  # noqa: F401
from tiny_vllm_b200 import _lib

PATHS = {"simt": _lib.PATH_SIMT_STREAM, "umma": _lib.PATH_UMMA, "umma_swap": _lib.PATH_UMMA_SWAP,
         "mma": _lib.PATH_MMA_STREAM}


@contextlib.contextmanager
def forced_path(name):
    """Runs the body with one kernel family forced (``None`` = the library's own choice)."""
    L = _lib.lib()
    prev = L.b200q_debug_force_path(PATHS[name] if name else _lib.PATH_AUTO)
    try:
        yield
    finally:
        L.b200q_debug_force_path(prev)


@contextlib.contextmanager
def knobs(**settings):
    """Runs the body with debug knobs set for this thread, e.g. ``knobs(CLUSTER=1)``
    (names are the ``KNOB_*`` constants of ``_lib`` without the prefix); all knobs are unset
    again afterwards, a forced kernel family included."""
    L = _lib.lib()
    path = L.b200q_debug_force_path(_lib.PATH_AUTO)
    L.b200q_debug_force_path(path)
    for name, value in settings.items():
        assert L.b200q_debug_set(getattr(_lib, "KNOB_" + name), int(value)) == 0
    try:
        yield
    finally:
        L.b200q_debug_reset()
        L.b200q_debug_force_path(path)


def device_status_ok():
    torch.cuda.synchronize()
    return _lib.lib().b200q_device_status() == 0


def bits(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.int16) if t.element_size() == 2 else t

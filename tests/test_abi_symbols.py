"""The C-ABI library: builds, loads, exports every symbol include/b200q.h declares, and
rejects bad arguments before touching a GPU (no compute call needs a device here)."""
import ctypes
import re
from pathlib import Path

import pytest

import tiny_vllm_b200  # noqa: F401  (import shim)
from tiny_vllm_b200 import _lib, build as b200_build

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200q.h"


@pytest.fixture(scope="module")
def L():
    b200_build.build()
    return _lib.lib()


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_list_the_same_functions():
    assert declared_functions() == sorted(_lib.SIGNATURES)


def test_every_declared_symbol_is_exported(L):
    for name in declared_functions():
        assert hasattr(L, name), name


def test_version_and_strerror(L):
    assert L.b200q_version() == _lib.ABI_VERSION
    assert L.b200q_strerror(0) == b"ok"
    for code in range(1, 10):
        assert len(L.b200q_strerror(code)) > 3
    assert b"unknown" in L.b200q_strerror(1234)


def test_error_codes_match_header():
    text = HEADER.read_text()
    for name in ("OK", "ERR_NULL_POINTER", "ERR_BAD_SHAPE", "ERR_UNSUPPORTED_SHAPE", "ERR_MISALIGNED",
                 "ERR_WORKSPACE", "ERR_UNSUPPORTED_ARCH", "ERR_LAUNCH", "ERR_BAD_ARGUMENT",
                 "ERR_DEVICE_TIMEOUT"):
        m = re.search(rf"B200Q_{name}\s*=\s*(\d+)", text)
        assert m and int(m.group(1)) == getattr(_lib, name), name


def test_argument_validation_needs_no_device(L):
    buf = ctypes.create_string_buffer(4096 + 64)
    p = (ctypes.addressof(buf) + 63) & ~63  # 64-byte aligned host address, never dereferenced
    # null pointers
    assert L.b200q_act_quant_i8(None, 64, 1, p, p, 4, 64, None) == _lib.ERR_NULL_POINTER
    assert L.b200q_w8a8_gemm(p, p, None, p, None, p, 4, 8, 64, 1, None, 0, None) == _lib.ERR_NULL_POINTER
    assert L.b200q_w8a8_gemm_i32(p, p, None, 4, 8, 64, None, 0, None) == _lib.ERR_NULL_POINTER
    assert L.b200q_w8a16_gemm(None, p, p, None, p, 4, 8, 64, 1, None, 0, None) == _lib.ERR_NULL_POINTER
    # shapes
    assert L.b200q_w8a8_gemm(p, p, p, p, None, p, 0, 8, 64, 1, None, 0, None) == _lib.ERR_BAD_SHAPE
    assert L.b200q_w8a8_gemm(p, p, p, p, None, p, 4, 8, 24, 1, None, 0, None) == _lib.ERR_UNSUPPORTED_SHAPE
    assert L.b200q_w8a16_gemm(p, p, p, None, p, 4, 8, 40, 1, None, 0, None) == _lib.ERR_UNSUPPORTED_SHAPE
    assert L.b200q_act_quant_i8(p, 60, 1, p, p, 4, 64, None) == _lib.ERR_UNSUPPORTED_SHAPE
    assert L.b200q_act_quant_i8(p, 64, 1, p, p, 4, 72, None) == _lib.ERR_UNSUPPORTED_SHAPE
    # dtype ids
    assert L.b200q_w8a8_gemm(p, p, p, p, None, p, 4, 8, 64, 7, None, 0, None) == _lib.ERR_BAD_ARGUMENT
    assert L.b200q_act_quant_i8(p, 64, 5, p, p, 4, 64, None) == _lib.ERR_BAD_ARGUMENT
    # alignment
    assert L.b200q_w8a8_gemm(p + 4, p, p, p, None, p, 4, 8, 64, 1, None, 0, None) == _lib.ERR_MISALIGNED
    assert L.b200q_w8a16_gemm(p, p + 8, p, None, p, 4, 8, 64, 1, None, 0, None) == _lib.ERR_MISALIGNED


def test_peer_entry_points_validate_before_touching_a_device(L):
    buf = ctypes.create_string_buffer(8192 + 512)
    p = (ctypes.addressof(buf) + 255) & ~255  # 256-byte aligned host address, never dereferenced
    two = (ctypes.c_void_p * 2)(p, p + 1024)
    holes = (ctypes.c_void_p * 2)(p, None)
    odd = (ctypes.c_void_p * 2)(p, p + 1028)
    # two-shot, pull and one-trip all-reduce
    assert L.b200q_tp_allreduce(None, two, 0, 2, 64, 1, None) == _lib.ERR_NULL_POINTER
    assert L.b200q_tp_allreduce(two, two, 2, 2, 64, 1, None) == _lib.ERR_BAD_ARGUMENT
    assert L.b200q_tp_allreduce(two, two, 0, 9, 64, 1, None) == _lib.ERR_BAD_ARGUMENT
    assert L.b200q_tp_allreduce(two, two, 0, 2, 60, 1, None) == _lib.ERR_UNSUPPORTED_SHAPE
    assert L.b200q_tp_allreduce(holes, two, 0, 2, 64, 1, None) == _lib.ERR_NULL_POINTER
    assert L.b200q_tp_allreduce(odd, two, 0, 2, 64, 1, None) == _lib.ERR_MISALIGNED
    assert L.b200q_tp_allreduce_pull(two, two, None, 0, 2, 64, 1, None) == _lib.ERR_NULL_POINTER
    assert L.b200q_tp_allreduce_pull(two, two, p + 2048, 0, 2, 64, 3, None) == _lib.ERR_BAD_ARGUMENT
    assert L.b200q_tp_allreduce_pull(two, two, p, 0, 2, 64, 1, None) == _lib.ERR_BAD_ARGUMENT  # out aliases input
    assert L.b200q_tp_allreduce_pull(two, two, p + 2056, 0, 2, 64, 1, None) == _lib.ERR_MISALIGNED
    assert L.b200q_tp_allreduce_small(p, p, 60, 1, two, two, 4096, 0, 2, None) == _lib.ERR_UNSUPPORTED_SHAPE
    assert L.b200q_tp_allreduce_small(p, p, 4096, 1, two, two, 4096, 0, 2, None) == _lib.ERR_WORKSPACE
    assert L.b200q_tp_allreduce_small(p, p, 64, 1, None, two, 4096, 0, 2, None) == _lib.ERR_NULL_POINTER
    # fused decode GEMM + all-reduce
    args = (p, p, p, p, None, p)
    assert L.b200q_w8a8_gemm_allreduce(*args, 16, 64, 64, 1, two, two, 1 << 20, 0, 2, None) in (
        _lib.ERR_UNSUPPORTED_ARCH, _lib.ERR_LAUNCH)            # arguments fine, no B200 here
    assert L.b200q_w8a8_gemm_allreduce(*args, 16, 64, 64, 1, None, two, 1 << 20, 0, 2, None) in (
        _lib.ERR_NULL_POINTER, _lib.ERR_UNSUPPORTED_ARCH, _lib.ERR_LAUNCH)
    assert L.b200q_w8a8_gemm_allreduce(*args, 16, 64, 24, 1, two, two, 1 << 20, 0, 2, None) == _lib.ERR_UNSUPPORTED_SHAPE
    assert L.b200q_w8a16_gemm_allreduce(None, p, p, None, p, 16, 64, 64, 1, two, two, 1 << 20, 0, 2,
                                        None) == _lib.ERR_NULL_POINTER
    # fused prefill route
    assert L.b200q_w8a8_gemm_allreduce_tiled(p, p, p, p, None, two, 1000, 64, 64, 1, two, 1 << 20, two, 0,
                                             2, None) == _lib.ERR_UNSUPPORTED_SHAPE      # M % (2 * 256)
    assert L.b200q_w8a8_gemm_allreduce_tiled(p, p, p, p, None, two, 1024, 64, 64, 1, two, 1024, two, 0, 2,
                                             None) == _lib.ERR_WORKSPACE
    assert L.b200q_w8a8_gemm_allreduce_tiled(p, p, p, p, None, None, 1024, 64, 64, 1, two, 1 << 20, two, 0,
                                             2, None) == _lib.ERR_NULL_POINTER


def test_path_names_and_workspace_queries(L):
    assert L.b200q_select_path(_lib.OP_W8A8, 8192, 4096, 1024) == b"umma_i8_pair_tokens256"
    assert L.b200q_select_path(_lib.OP_W8A8, 300, 4096, 1024) == b"umma_i8_tokens128"
    assert L.b200q_select_path(_lib.OP_W8A8, 128, 4096, 1024) == b"umma_i8_tokens128"
    assert L.b200q_select_path(_lib.OP_W8A8, 1, 4096, 1024) == b"mma_stream_s8_splitk"
    assert L.b200q_select_path(_lib.OP_W8A8, 16, 4096, 1000) == b"unsupported_shape"
    assert L.b200q_select_path(99, 1, 1, 16) == b"invalid_op"
    assert L.b200q_workspace_bytes(_lib.OP_W8A8, 8192, 4096, 1024) == 0
    assert L.b200q_workspace_bytes(_lib.OP_W8A8, 128, 512, 8192) > 16384
    assert L.b200q_workspace_bytes(_lib.OP_ACT_QUANT, 16, 1024, 3072) == 0
    prev = L.b200q_debug_force_path(_lib.PATH_SIMT_STREAM)
    try:
        assert prev == _lib.PATH_AUTO
        assert L.b200q_select_path(_lib.OP_W8A8, 8192, 4096, 1024) == b"simt_stream_dp4a"
        assert L.b200q_debug_force_path(99) == -1
    finally:
        L.b200q_debug_force_path(_lib.PATH_AUTO)
    assert L.b200q_launch_count() == 0 or L.b200q_launch_count() > 0


def test_python_entry_points_refuse_cpu_tensors():
    import torch
    from tiny_vllm_b200.quantization.cuda import (apply_int8_weight_only_linear, apply_w8a8_linear,
                                                  quantize_activation_int8)
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    q = torch.zeros(8, 64, dtype=torch.int8)
    s = torch.ones(8)
    with pytest.raises(RuntimeError):
        apply_int8_weight_only_linear(x, q, s)
    with pytest.raises(RuntimeError):
        quantize_activation_int8(x)
    with pytest.raises(RuntimeError):
        apply_w8a8_linear(q[:4], torch.ones(4), q, s, out_dtype=torch.bfloat16)

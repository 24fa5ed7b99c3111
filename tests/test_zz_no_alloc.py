"""b200q_w8a8_gemm_noalloc: the W8A8 entry point for callers that cannot hand over scratch
memory (an embedder of the C ABI without a device allocator, or a server whose free HBM has
all gone to the KV cache).  It must give exactly what b200q_w8a8_gemm gives with a
caller-owned workspace, call after call, although its scratch is one array inside the
library that keeps the previous call's contents.

This file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test.  It also passes when run alone in a fresh process."""
import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import bits, forced_path
from tiny_vllm_b200 import _lib
from tiny_vllm_b200.quantization.cuda import apply_w8a8_linear

pytestmark = pytest.mark.gpu


def call_noalloc(xq, a_s, q, s, bias, dtype):
    M, K = xq.shape
    N = q.shape[0]
    y = torch.empty(M, N, dtype=dtype, device=xq.device)
    rc = _lib.lib().b200q_w8a8_gemm_noalloc(
        xq.data_ptr(), a_s.data_ptr(), q.data_ptr(), s.data_ptr(),
        None if bias is None else bias.data_ptr(), y.data_ptr(), M, N, K,
        _lib.DTYPE_BF16 if dtype == torch.bfloat16 else _lib.DTYPE_F16,
        torch.cuda.current_stream().cuda_stream)
    return rc, y


@pytest.mark.parametrize("M,N,K,with_bias", [(48, 256, 8192, False), (16, 512, 8192, True),
                                             (200, 256, 16384, False)])
def test_matches_the_workspace_entry_point_on_consecutive_calls(M, N, K, with_bias):
    L = _lib.lib()
    q, s = O.make_weight(N, K, seed=N + K)
    x = O.make_activation(M, K, seed=M)
    xq, a_s = O.quantize_per_row_dynamic(x)
    b = (torch.randn(N, generator=torch.Generator().manual_seed(3)) * 0.1).to(torch.bfloat16) \
        if with_bias else None
    gxq, gas, gq, gs = xq.cuda(), a_s.cuda(), q.cuda(), s.cuda()
    gb = None if b is None else b.cuda()
    with forced_path("umma_swap"):
        assert L.b200q_workspace_bytes(_lib.OP_W8A8, M, N, K) > 0   # this shape does use scratch
        expect = apply_w8a8_linear(gxq, gas, gq, gs, gb, out_dtype=torch.bfloat16)
    # a second problem in between leaves other data in the shared scratch array
    q2, s2 = O.make_weight(N, K, seed=7)
    for round_ in range(2):
        rc, y = call_noalloc(gxq, gas, gq, gs, gb, torch.bfloat16)
        assert rc == _lib.OK, L.b200q_strerror(rc)
        torch.cuda.synchronize()
        assert torch.equal(bits(y), bits(expect)), round_   # int32 sums are exact: identical bits
        rc, _ = call_noalloc(gxq, gas, q2.cuda(), s2.cuda(), None, torch.bfloat16)
        assert rc == _lib.OK
    # and it agrees with the CPU oracle, not only with the other entry point
    ref = O.w8a8_native_epilogue(O.w8a8_int32_accumulators(xq, q), a_s, s, b, torch.bfloat16)
    assert torch.equal(bits(y.cpu()), bits(ref))
    torch.cuda.synchronize()
    assert L.b200q_device_status() == 0


def test_prefill_sized_call_needs_no_scratch_and_matches():
    M, N, K = 4096, 1536, 512      # 192 output tiles: enough for every SM, so no split-K
    q, s = O.make_weight(N, K, seed=1)
    xq, a_s = O.quantize_per_row_dynamic(O.make_activation(M, K, seed=2))
    gxq, gas, gq, gs = xq.cuda(), a_s.cuda(), q.cuda(), s.cuda()
    expect = apply_w8a8_linear(gxq, gas, gq, gs, out_dtype=torch.float16)
    rc, y = call_noalloc(gxq, gas, gq, gs, None, torch.float16)
    assert rc == _lib.OK
    assert torch.equal(bits(y), bits(expect))


def test_refuses_problems_beyond_the_built_in_scratch_and_bad_arguments():
    L = _lib.lib()
    M, N, K = 256, 9216, 8192      # split-K partial tiles of this shape exceed 8 MiB
    xq = torch.zeros(M, K, dtype=torch.int8, device="cuda")
    q = torch.zeros(N, K, dtype=torch.int8, device="cuda")
    a_s = torch.ones(M, device="cuda")
    s = torch.ones(N, device="cuda")
    before = L.b200q_launch_count()
    rc, _ = call_noalloc(xq, a_s, q, s, None, torch.bfloat16)
    assert rc == _lib.ERR_SCRATCH_LIMIT
    assert b"scratch" in L.b200q_strerror(rc)
    assert L.b200q_launch_count() == before          # nothing was launched
    st = torch.cuda.current_stream().cuda_stream
    assert L.b200q_w8a8_gemm_noalloc(None, a_s.data_ptr(), q.data_ptr(), s.data_ptr(), None,
                                     xq.data_ptr(), M, N, K, 1, st) == _lib.ERR_NULL_POINTER
    assert L.b200q_w8a8_gemm_noalloc(xq.data_ptr(), a_s.data_ptr(), q.data_ptr(), s.data_ptr(), None,
                                     xq.data_ptr(), M, N, 1000, 1, st) == _lib.ERR_UNSUPPORTED_SHAPE

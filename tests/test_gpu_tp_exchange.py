"""The fused exchange after a row-parallel layer — sum over ranks + residual add + RMSNorm +
int8 quantisation + gather of the codes (``b200q_tp_reduce_rmsnorm_quant``) — on ONE GPU.

A rank's kernel only waits for flags, so its part of the exchange can be run alone when the
host plays the peers: their partial outputs are ordinary local tensors and the two flags a peer
would raise are written by the host before the launch.  Running the kernel once as every rank,
one after the other (never two waiting kernels at a time), assembles the complete result, which
must be bit-identical to what the reference's chain computes on the rank-ordered fp32 sum:
``dist.all_reduce`` -> ``RMSNorm(x, residual)`` -> ``quantize_int8_per_row_dynamic``
(nanovllm/layers/linear.py:274-275, layernorm.py:28-40, quantization/utils.py:28-32) — here
through ``b200q_add_rmsnorm_quant_i8``, whose parity with the reference modules is tested
elsewhere.  The multi-GPU run of the same entry point is in test_gpu_tp_allreduce.py."""
import ctypes

import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import bits, device_status_ok
from tiny_vllm_b200 import _lib
from tiny_vllm_b200.quantization.cuda import add_rmsnorm_quantize_int8

pytestmark = pytest.mark.gpu
SLOT_A, SLOT_B = 16, 32


def ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def run_as_every_rank(parts, residual, weight, eps, dtype):
    """Runs the exchange kernel once per rank on this GPU.  Returns per-rank code / scale
    buffers, the new residual and the normalised rows (both assembled from the owners)."""
    L = _lib.lib()
    world = len(parts)
    M, K = parts[0].shape
    rows = M // world
    xq = [torch.full((M, K), -128, dtype=torch.int8, device="cuda") for _ in range(world)]
    sc = [torch.full((M,), -1.0, dtype=torch.float32, device="cuda") for _ in range(world)]
    pads = [torch.zeros(1024, dtype=torch.int32, device="cuda") for _ in range(world)]
    new_res = torch.empty(M, K, dtype=dtype, device="cuda")
    normed = torch.empty(M, K, dtype=dtype, device="cuda")
    for rank in range(world):
        for peer in range(world):          # the host raises the peers' flags of call number 1
            if peer != rank:
                pads[rank][SLOT_A + peer] = 1
                pads[rank][SLOT_B + peer] = 1
        torch.cuda.synchronize()
        res_in = None if residual is None else residual[rank * rows:(rank + 1) * rows]
        rc = L.b200q_tp_reduce_rmsnorm_quant(
            ptrs(parts), ptrs(pads), None if res_in is None else res_in.data_ptr(),
            new_res[rank * rows:(rank + 1) * rows].data_ptr() if residual is not None else None,
            weight.data_ptr(), eps, ptrs(xq), ptrs(sc), normed[rank * rows:(rank + 1) * rows].data_ptr(),
            M, K, rank, world, _lib.DTYPE_BF16 if dtype == torch.bfloat16 else _lib.DTYPE_F16,
            torch.cuda.current_stream().cuda_stream)
        assert rc == _lib.OK, rc
        torch.cuda.synchronize()
        assert int(pads[rank][0].item()) == 1          # the rank's call counter
    return xq, sc, new_res, normed


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("M,K,dtype,with_residual", [(64, 1024, torch.bfloat16, True),
                                                      (8192, 1024, torch.bfloat16, True),
                                                      (48, 2048, torch.float16, False),
                                                      (16, 4096, torch.bfloat16, True),
                                                      (40, 272, torch.float16, True)])
def test_exchange_equals_allreduce_then_norm_quant(world, M, K, dtype, with_residual):
    if M % world:
        pytest.skip("rows must divide by the group size")
    g = torch.Generator().manual_seed(world * 1000 + M + K)
    parts_cpu = [(torch.randn(M, K, generator=g) * 1.5).to(dtype) for _ in range(world)]
    residual = (torch.randn(M, K, generator=g) * 2).to(dtype) if with_residual else None
    weight = (1.0 + 0.2 * torch.randn(K, generator=g)).to(dtype)
    eps = 1e-6
    total = torch.zeros(M, K)
    for p in parts_cpu:                     # the all-reduce: fp32, rank order, one rounding
        total += p.float()
    reduced = total.to(dtype)
    want_q, want_s, want_res, want_y = add_rmsnorm_quantize_int8(
        reduced.cuda(), weight.cuda(), eps, None if residual is None else residual.cuda(), return_normed=True)
    xq, sc, new_res, normed = run_as_every_rank([p.cuda() for p in parts_cpu],
                                                None if residual is None else residual.cuda(),
                                                weight.cuda(), eps, dtype)
    for r in range(world):                  # every rank holds all rows
        assert torch.equal(xq[r], want_q), (world, r)
        assert torch.equal(sc[r], want_s), (world, r)
    assert torch.equal(bits(normed), bits(want_y))
    if with_residual:
        assert torch.equal(bits(new_res), bits(want_res))
    # and against the oracle's restatement of the reference modules (tolerance of the norm:
    # two units in the last place in at most 2 % of the elements)
    y_ref, res_ref = O.add_rmsnorm(reduced, weight, eps, residual)
    d = (bits(normed.cpu()).int() - bits(y_ref).int()).abs()
    assert int(d.max()) <= 2 and float((d > 0).float().mean()) <= 0.02
    if with_residual:
        assert torch.equal(bits(new_res.cpu()), bits(res_ref))
    assert device_status_ok()


def test_exchange_rejects_bad_arguments():
    L = _lib.lib()
    t = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    q = torch.zeros(16, 64, dtype=torch.int8, device="cuda")
    s = torch.zeros(16, dtype=torch.float32, device="cuda")
    pad = torch.zeros(1024, dtype=torch.int32, device="cuda")
    w = torch.ones(64, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream

    def call(M=16, K=64, rank=0, world=1, parts=None):
        return L.b200q_tp_reduce_rmsnorm_quant(parts if parts is not None else ptrs([t] * world),
                                               ptrs([pad] * world), None, None, w.data_ptr(), 1e-6,
                                               ptrs([q] * world), ptrs([s] * world), None, M, K,
                                               rank, world, _lib.DTYPE_BF16, st)
    assert call(world=9) == _lib.ERR_BAD_ARGUMENT
    assert call(rank=2, world=2) == _lib.ERR_BAD_ARGUMENT
    assert call(M=15, world=2) == _lib.ERR_UNSUPPORTED_SHAPE       # rows do not divide
    assert call(K=40) == _lib.ERR_UNSUPPORTED_SHAPE
    assert call(parts=None, M=0) == _lib.ERR_BAD_SHAPE
    assert L.b200q_tp_reduce_rmsnorm_quant(None, ptrs([pad]), None, None, w.data_ptr(), 1e-6, ptrs([q]),
                                           ptrs([s]), None, 16, 64, 0, 1, _lib.DTYPE_BF16, st) == _lib.ERR_NULL_POINTER

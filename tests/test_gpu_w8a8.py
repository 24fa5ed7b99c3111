"""W8A8 GEMM kernels vs the CPU oracle.

* int32 accumulators: bit-exact against the integer oracle, for every kernel family;
* 16-bit outputs: bit-exact against the oracle's restatement of the fused epilogue
  ((acc * a_s) * w_s + bias, fp32, one rounding per operation), and within
  rel-L2 <= 1e-2, cosine >= 0.9999 of the reference's dequantize-then-matmul path.
"""
import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import bits, device_status_ok, forced_path, knobs
from tiny_vllm_b200 import _lib
from tiny_vllm_b200.quantization.cuda import (apply_w8a8_linear, quantize_activation_int8,
                                              select_path, w8a8_int32_accumulators)

pytestmark = pytest.mark.gpu

REL_L2_GATE = 1e-2
COSINE_GATE = 0.9999


def problem(M, N, K, seed=0, dtype=torch.bfloat16, bias=False):
    q, s = O.make_weight(N, K, seed=seed)
    x = O.make_activation(M, K, seed=seed, dtype=dtype)
    xq, a_s = O.quantize_per_row_dynamic(x)
    b = None
    if bias:
        b = (torch.randn(N, generator=torch.Generator().manual_seed(seed + 5)) * 0.1).to(dtype)
    return x, xq, a_s, q, s, b


SHAPES = [  # (M, N, K) — ragged tiles, single K block, K tail (K % 128 != 0), N % 8 != 0
    (1, 64, 128), (5, 96, 256), (16, 1024, 1024), (37, 192, 256), (64, 130, 512),
    (128, 256, 128), (130, 320, 1024), (200, 72, 48), (257, 512, 2048), (300, 1000, 1040),
    (512, 1024, 3072), (1000, 384, 272),
]


@pytest.mark.parametrize("path", ["simt", "umma", "umma_swap", "mma"])
@pytest.mark.parametrize("M,N,K", SHAPES + [(17, 68, 80), (48, 1024, 3072), (64, 6144, 1024), (40, 256, 8192), (300, 384, 12288)])
def test_int32_accumulators_bit_exact(path, M, N, K, oracle_c_lib):
    if path == "mma" and M > 64:
        pytest.skip("mma.sync streaming family is for M <= 64")
    if path == "simt" and M * N * K > 2e8:
        pytest.skip("SIMT family is for small token counts")
    if path == "umma_swap" and M > 512:
        pytest.skip("swap family is for decode-sized token counts")
    _, xq, _, q, _, _ = problem(M, N, K, seed=M + N)
    with forced_path(path):
        acc = w8a8_int32_accumulators(xq.cuda(), q.cuda())
    assert torch.equal(acc.cpu(), O.w8a8_int32_accumulators(xq, q)), (path, M, N, K)
    assert device_status_ok()


@pytest.mark.parametrize("path", ["simt", "umma", "umma_swap", "mma", None])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K,bias", [(5, 96, 256, True), (130, 320, 1024, False),
                                        (257, 512, 2048, True), (64, 1024, 3072, False),
                                        (33, 100, 272, True)])
def test_scaled_output(path, dtype, M, N, K, bias, oracle_c_lib):
    if path == "mma" and M > 64:
        pytest.skip("mma.sync streaming family is for M <= 64")
    x, xq, a_s, q, s, b = problem(M, N, K, seed=N, dtype=dtype, bias=bias)
    with forced_path(path):
        y = apply_w8a8_linear(xq.cuda(), a_s.cuda(), q.cuda(), s.cuda(),
                              None if b is None else b.cuda(), out_dtype=dtype)
    assert y.dtype == dtype and y.shape == (M, N)
    acc = O.w8a8_int32_accumulators(xq, q)
    expect = O.w8a8_native_epilogue(acc, a_s, s, b, dtype)
    assert torch.equal(bits(y.cpu()), bits(expect)), (path, dtype)
    ref = O.w8a8_dequant_matmul(xq, a_s, q, s, b, dtype)
    m = O.tensor_metrics(ref, y)
    assert m["relative_l2"] <= REL_L2_GATE and m["cosine_similarity"] >= COSINE_GATE, m
    assert device_status_ok()


def test_golden_cases(golden_cases):
    for c in golden_cases:
        for path in ("simt", "umma", "umma_swap", "mma"):
            if path == "mma" and c["M"] > 64:
                continue
            with forced_path(path):
                acc = w8a8_int32_accumulators(c["xq"].cuda(), c["q"].cuda())
                y = apply_w8a8_linear(c["xq"].cuda(), c["a_s"].cuda(), c["q"].cuda(), c["s"].cuda(),
                                      None if c["bias"] is None else c["bias"].cuda(),
                                      out_dtype=c["dtype"])
            assert torch.equal(acc.cpu(), c["acc_i32"]), (c["id"], path)
            m = O.tensor_metrics(c["y_w8a8"], y)
            assert m["relative_l2"] <= REL_L2_GATE and m["cosine_similarity"] >= COSINE_GATE, (c["id"], path, m)


def test_benchmark_decode_shape_against_reference_vectors(baseline_shape_golden):
    # W8A8, 16 tokens through 1024 -> 4096: the reference's own quantiser output, exact integer
    # accumulators and dequantize-then-matmul output (tests/golden/baseline_shapes_golden.npz)
    import numpy as np
    z = baseline_shape_golden
    M, K, N = (int(v) for v in z["w8a8_shape"])
    q, s = O.make_weight(N, K, seed=1)
    x = O.make_activation(M, K, seed=1)
    xq, a_s = quantize_activation_int8(x.cuda())
    assert torch.equal(xq.cpu(), torch.from_numpy(z["w8a8_xq"]))
    assert torch.equal(a_s.cpu(), torch.from_numpy(z["w8a8_a_s"]))
    want = torch.from_numpy(z["w8a8_y"].view(np.int16).copy()).view(torch.bfloat16)
    for path in ("simt", "umma", "umma_swap", "mma", None):
        with forced_path(path):
            acc = w8a8_int32_accumulators(xq, q.cuda())
            y = apply_w8a8_linear(xq, a_s, q.cuda(), s.cuda(), out_dtype=torch.bfloat16)
        assert torch.equal(acc.cpu(), torch.from_numpy(z["w8a8_acc_i32"])), path
        m = O.tensor_metrics(want, y)
        assert m["relative_l2"] <= REL_L2_GATE and m["cosine_similarity"] >= COSINE_GATE, (path, m)
    assert device_status_ok()


def test_quant_then_gemm_matches_reference_chain():
    # activation quantisation on the GPU feeding the GEMM: the whole W8A8QuantMethod.apply chain
    x, xq, a_s, q, s, _ = problem(300, 512, 1024, seed=21)
    gxq, gas = quantize_activation_int8(x.cuda())
    assert torch.equal(gxq.cpu(), xq) and torch.equal(gas.cpu(), a_s)
    y = apply_w8a8_linear(gxq, gas, q.cuda(), s.cuda(), out_dtype=torch.bfloat16, out_shape=(3, 100, 512))
    assert y.shape == (3, 100, 512)
    ref = O.w8a8_dequant_matmul(xq, a_s, q, s, None, torch.bfloat16)
    m = O.tensor_metrics(ref, y.view(300, 512))
    assert m["relative_l2"] <= REL_L2_GATE and m["cosine_similarity"] >= COSINE_GATE


@pytest.mark.parametrize("N,K", [(4096, 1024), (1024, 2048), (6144, 1024), (1024, 3072)])
def test_baseline_prefill_shapes_full_size(N, K, oracle_c_lib):
    # M = 8192 (the benchmark's workload), EVERY element: the CTA-pair kernel's raw int32
    # accumulators against the integer oracle, its 16-bit output — through both
    # output routes of its epilogue — against the oracle's restatement of the fused epilogue,
    # and the single-CTA kernel's accumulators as the independent second implementation.
    M = 8192
    x, xq, a_s, q, s, _ = problem(M, N, K, seed=K)
    gx, gq, gas, gs = xq.cuda(), q.cuda(), a_s.cuda(), s.cuda()
    assert select_path(_lib.OP_W8A8, M, N, K) == "umma_i8_pair_tokens256"
    ref_acc = O.w8a8_int32_accumulators(xq, q)
    acc = w8a8_int32_accumulators(gx, gq)
    assert torch.equal(acc.cpu(), ref_acc)
    with knobs(NO_PAIR=1):
        assert select_path(_lib.OP_W8A8, M, N, K) == "umma_i8_tokens128"
        assert torch.equal(w8a8_int32_accumulators(gx, gq).cpu(), ref_acc)
    # size-independent property: row sums of acc equal x_q @ (column sums of W) in int64
    assert torch.equal(acc.to(torch.int64).sum(dim=1).cpu(), xq.to(torch.int64) @ q.to(torch.int64).sum(dim=0))
    expect = bits(O.w8a8_native_epilogue(ref_acc, a_s, s, None, torch.bfloat16))
    # default output route (TMA stores), then the st.global route the row-parallel scatter uses
    for epilogue in (None, 0):
        with knobs(**({} if epilogue is None else {"PAIR_EPILOGUE": epilogue})):
            y = apply_w8a8_linear(gx, gas, gq, gs, out_dtype=torch.bfloat16)
        assert torch.equal(bits(y.cpu()), expect), epilogue
    rows = torch.arange(0, M, 331)
    ref = O.w8a8_dequant_matmul(xq[rows], a_s[rows], q, s, None, torch.bfloat16)
    m = O.tensor_metrics(ref, y[rows])
    assert m["relative_l2"] <= REL_L2_GATE and m["cosine_similarity"] >= COSINE_GATE
    assert device_status_ok()


@pytest.mark.parametrize("epilogue", [None, 0, 1])
@pytest.mark.parametrize("M,N,K,dtype,bias", [(2500, 2056, 272, torch.bfloat16, True),
                                              (2305, 2304, 1024, torch.float16, False),
                                              (9000, 520, 128, torch.bfloat16, False),
                                              (4700, 1288, 2064, torch.bfloat16, True)])
def test_cta_pair_kernel_ragged_edges(M, N, K, dtype, bias, epilogue, oracle_c_lib):
    # shapes the CTA-pair (cta_group::2) kernel takes, with M not a multiple of 256 (the second
    # CTA of the last pair is partly or wholly out of range), N not a multiple of 256 (nor of 16)
    # and a K tail; every output route of the epilogue, and the raw accumulators
    assert select_path(_lib.OP_W8A8, M, N, K) == "umma_i8_pair_tokens256"
    x, xq, a_s, q, s, b = problem(M, N, K, seed=M, dtype=dtype, bias=bias)
    ref_acc = O.w8a8_int32_accumulators(xq, q)
    # None = the library's own choice (TMA stores)
    with knobs(**({} if epilogue is None else {"PAIR_EPILOGUE": epilogue})):
        y = apply_w8a8_linear(xq.cuda(), a_s.cuda(), q.cuda(), s.cuda(), None if b is None else b.cuda(),
                              out_dtype=dtype)
    expect = O.w8a8_native_epilogue(ref_acc, a_s, s, b, dtype)
    assert torch.equal(bits(y.cpu()), bits(expect))
    if epilogue == 0:
        assert torch.equal(w8a8_int32_accumulators(xq.cuda(), q.cuda()).cpu(), ref_acc)
    assert device_status_ok()


def test_cta_pair_raw_accumulators_with_odd_channel_count(oracle_c_lib):
    # N % 4 != 0: the int32 rows are not 16-byte multiples, element-wise stores
    M, N, K = 2400, 2051, 144
    _, xq, _, q, _, _ = problem(M, N, K, seed=3)
    assert torch.equal(w8a8_int32_accumulators(xq.cuda(), q.cuda()).cpu(), O.w8a8_int32_accumulators(xq, q))
    assert device_status_ok()


@pytest.mark.parametrize("M", [1, 16, 128, 512])
@pytest.mark.parametrize("N,K", [(4096, 1024), (1024, 2048), (6144, 1024), (1024, 3072)])
def test_baseline_decode_shapes(M, N, K, oracle_c_lib):
    x, xq, a_s, q, s, _ = problem(M, N, K, seed=M + K)
    acc = w8a8_int32_accumulators(xq.cuda(), q.cuda())
    ref_acc = O.w8a8_int32_accumulators(xq, q)
    assert torch.equal(acc.cpu(), ref_acc)
    y = apply_w8a8_linear(xq.cuda(), a_s.cuda(), q.cuda(), s.cuda(), out_dtype=torch.bfloat16)
    assert torch.equal(bits(y.cpu()), bits(O.w8a8_native_epilogue(ref_acc, a_s, s, None, torch.bfloat16)))
    assert device_status_ok()


@pytest.mark.parametrize("M,N,K,dtype,bias", [(128, 1024, 2048, torch.bfloat16, False),
                                              (300, 1024, 3072, torch.bfloat16, True),
                                              (200, 1000, 1040, torch.float16, True),
                                              (100, 1000, 400, torch.bfloat16, False),
                                              (256, 4096, 1024, torch.bfloat16, False)])
def test_cluster_split_k(M, N, K, dtype, bias, oracle_c_lib):
    # decode batches of 64-512 tokens: K is split over a cluster of 2 or 4 CTAs and the leader
    # adds the peers' int32 partial tiles from its shared memory: exact, so nothing may change
    x, xq, a_s, q, s, b = problem(M, N, K, seed=M + K, dtype=dtype, bias=bias)
    dev = [t.cuda() for t in (xq, a_s, q, s)]
    bd = None if b is None else b.cuda()
    ref_acc = O.w8a8_int32_accumulators(xq, q)
    assert torch.equal(w8a8_int32_accumulators(dev[0], dev[2]).cpu(), ref_acc)
    y = apply_w8a8_linear(*dev, bias=bd, out_dtype=dtype)
    assert torch.equal(bits(y.cpu()), bits(O.w8a8_native_epilogue(ref_acc, a_s, s, b, dtype)))
    with knobs(CLUSTER=1):                                  # the same kernel without the cluster
        assert torch.equal(bits(apply_w8a8_linear(*dev, bias=bd, out_dtype=dtype)), bits(y))
    assert device_status_ok()


@pytest.mark.parametrize("M", [16, 300])
@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 12288)])
def test_qwen3_8b_shapes(M, N, K, oracle_c_lib):
    # the larger model of the engine configs: qkv (4096 -> 6144) and down (12288 -> 4096);
    # K = 12288 is the longest reduction (|acc| up to 1.98e8 < 2^31) and triggers split-K
    x, xq, a_s, q, s, _ = problem(M, N, K, seed=M + N)
    acc = w8a8_int32_accumulators(xq.cuda(), q.cuda())
    ref_acc = O.w8a8_int32_accumulators(xq, q)
    assert torch.equal(acc.cpu(), ref_acc)
    y = apply_w8a8_linear(xq.cuda(), a_s.cuda(), q.cuda(), s.cuda(), out_dtype=torch.bfloat16)
    assert torch.equal(bits(y.cpu()), bits(O.w8a8_native_epilogue(ref_acc, a_s, s, None, torch.bfloat16)))
    assert device_status_ok()


def test_saturated_inputs_reach_the_int32_extremes():
    # all +-127 codes: every accumulator is +-K * 127^2, the largest magnitude the path can see
    M, N, K = 130, 256, 12288
    xq = torch.full((M, K), 127, dtype=torch.int8)
    xq[::2] = -127
    q = torch.full((N, K), 127, dtype=torch.int8)
    q[1::2] = -127
    for path in ("umma", "umma_swap"):
        with forced_path(path):
            acc = w8a8_int32_accumulators(xq.cuda(), q.cuda())
        expect = (xq[:, :1].int() * q[:, :1].int().T) * K
        assert torch.equal(acc.cpu(), expect), path


def test_repeated_split_k_calls_leave_workspace_clean():
    # the split-K counters must return to zero: same call three times, same answer
    _, xq, a_s, q, s, _ = problem(48, 256, 8192, seed=9)
    expect = O.w8a8_int32_accumulators(xq, q)
    with forced_path("umma_swap"):
        assert _lib.lib().b200q_workspace_bytes(_lib.OP_W8A8, 48, 256, 8192) > 0
        for _ in range(3):
            assert torch.equal(w8a8_int32_accumulators(xq.cuda(), q.cuda()).cpu(), expect)


def test_workspace_too_small_is_an_error():
    _, xq, a_s, q, s, _ = problem(48, 256, 8192, seed=9)
    gx, gq = xq.cuda(), q.cuda()
    acc = torch.empty(48, 256, dtype=torch.int32, device="cuda")
    L = _lib.lib()
    with forced_path("umma_swap"):
        rc = L.b200q_w8a8_gemm_i32(gx.data_ptr(), gq.data_ptr(), acc.data_ptr(), 48, 256, 8192,
                                   None, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_WORKSPACE

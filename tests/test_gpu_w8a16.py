"""W8A16 GEMM vs the oracle: within rel-L2 1e-2 / cosine 0.9999 of the reference's
dequantize-then-matmul path, and much closer to the fp64 value of the same sum."""
import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import bits, device_status_ok, forced_path, knobs
from tiny_vllm_b200 import _lib
from tiny_vllm_b200.quantization.cuda import apply_int8_weight_only_linear, select_path

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("path", ["simt", "umma", "umma_swap", "mma", None])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K,bias", [(1, 64, 128, False), (5, 96, 256, True), (37, 192, 256, True),
                                        (130, 320, 1024, False), (256, 6144, 1024, False),
                                        (64, 1000, 1040, True), (300, 512, 2048, True), (40, 256, 8192, False),
                                        (513, 200, 48, False)])
def test_matches_reference_path(path, dtype, M, N, K, bias):
    if path == "mma" and M > 64:
        pytest.skip("mma.sync streaming family is for M <= 64")
    q, s = O.make_weight(N, K, seed=N)
    x = O.make_activation(M, K, seed=M, dtype=dtype, outliers=False)
    b = (torch.randn(N, generator=torch.Generator().manual_seed(1)) * 0.1).to(dtype) if bias else None
    with forced_path(path):
        y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda(), None if b is None else b.cuda())
    assert y.dtype == dtype and y.shape == (M, N)
    ref = O.w8a16_dequant_matmul(x, q, s, b)
    m = O.tensor_metrics(ref, y)
    assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, m
    exact = O.w8a16_native_reference(x, q, s, b)
    m = O.tensor_metrics(exact, y)
    assert m["relative_l2"] <= 4e-3, m
    assert device_status_ok()


def test_golden_cases(golden_cases):
    for c in golden_cases:
        for path in ("simt", "umma", "umma_swap", "mma"):
            if path == "mma" and c["M"] > 64:
                continue
            with forced_path(path):
                y = apply_int8_weight_only_linear(c["x"].cuda(), c["q"].cuda(), c["s"].cuda(),
                                                  None if c["bias"] is None else c["bias"].cuda())
            m = O.tensor_metrics(c["y_w8a16"], y)
            assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, (c["id"], path, m)


def test_benchmark_shape_against_reference_vectors(baseline_shape_golden):
    # single W8A16 linear 256 x 1024 -> 6144: sampled rows of the reference's own
    # dequantize-then-matmul output (tests/golden/baseline_shapes_golden.npz), every kernel family
    import numpy as np
    z = baseline_shape_golden
    M, K, N = (int(v) for v in z["w8a16_shape"])
    q, s = O.make_weight(N, K, seed=0)
    x = O.make_activation(M, K, seed=0, outliers=False)
    rows = torch.from_numpy(z["w8a16_rows"])
    want = torch.from_numpy(z["w8a16_y_rows"].view(np.int16).copy()).view(torch.bfloat16)
    for path in ("simt", "umma", "umma_swap", None):
        with forced_path(path):
            y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda())
        m = O.tensor_metrics(want, y[rows.cuda()])
        assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, (path, m)
    assert device_status_ok()


def test_all_int8_codes_expand_exactly():
    # every int8 value, -128 included, must reach the tensor cores unchanged: with x = identity
    # rows and unit scales the output is the weight matrix itself
    K = 256
    q = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8).repeat(128, 1)      # [128, 256]
    q = torch.stack([torch.roll(q[i], i) for i in range(128)])
    s = torch.ones(128)
    for dtype in (torch.bfloat16, torch.float16):
        x = torch.eye(K, dtype=dtype)
        for path in ("umma", "umma_swap"):
            with forced_path(path):
                y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda())
            assert torch.equal(y.float().cpu(), q.float().T), (dtype, path)
        with forced_path("mma"):   # 64 tokens at a time
            for r0 in range(0, K, 64):
                y = apply_int8_weight_only_linear(x[r0:r0 + 64].cuda(), q.cuda(), s.cuda())
                assert torch.equal(y.float().cpu(), q.float().T[r0:r0 + 64]), (dtype, r0)


@pytest.mark.parametrize("M,N,K,dtype,bias", [(2500, 2056, 272, torch.bfloat16, True),
                                              (2305, 2304, 1024, torch.float16, False)])
def test_prefill_kernel_ragged_edges(M, N, K, dtype, bias):
    q, s = O.make_weight(N, K, seed=N)
    x = O.make_activation(M, K, seed=M, dtype=dtype, outliers=False)
    b = (torch.randn(N, generator=torch.Generator().manual_seed(1)) * 0.1).to(dtype) if bias else None
    y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda(), None if b is None else b.cuda())
    m = O.tensor_metrics(O.w8a16_native_reference(x, q, s, b), y)
    assert m["relative_l2"] <= 4e-3 and m["cosine_similarity"] >= 0.9999, m
    assert device_status_ok()


@pytest.mark.parametrize("M,N,K,dtype,bias", [(2500, 2056, 272, torch.bfloat16, True),
                                              (2305, 2304, 1024, torch.float16, False),
                                              (5000, 1024, 2048, torch.bfloat16, False)])
def test_tensor_memory_weights_kernel(M, N, K, dtype, bias):
    # the variant that keeps the expanded weights in tensor memory (512 <= M < 1024 by default),
    # forced here for ragged M / N and a K tail as well
    with knobs(TS_MIN_K=16, W8A16_PAIR_MIN_M=1 << 30):
        assert select_path(_lib.OP_W8A16, M, N, K) == "umma_f16_tmem_weights_channels256"
        q, s = O.make_weight(N, K, seed=N)
        x = O.make_activation(M, K, seed=M, dtype=dtype, outliers=False)
        b = (torch.randn(N, generator=torch.Generator().manual_seed(1)) * 0.1).to(dtype) if bias else None
        y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda(), None if b is None else b.cuda())
        m = O.tensor_metrics(O.w8a16_native_reference(x, q, s, b), y)
        assert m["relative_l2"] <= 4e-3 and m["cosine_similarity"] >= 0.9999, m
        # every int8 code expands exactly: identity activations select weight columns
        Kc, Mc, Nc = 256, 2560, 2048
        qc = torch.stack([torch.roll(torch.arange(-128, 128, dtype=torch.int16).to(torch.int8), i)
                          for i in range(Nc)])
        xc = torch.eye(Kc, dtype=dtype).repeat(Mc // Kc, 1)
        yc = apply_int8_weight_only_linear(xc.cuda(), qc.cuda(), torch.ones(Nc).cuda())
        assert torch.equal(yc.float().cpu(), qc.float().T.repeat(Mc // Kc, 1))
    assert device_status_ok()


@pytest.mark.parametrize("epilogue", [0, 1])
@pytest.mark.parametrize("M,N,K,dtype,bias", [(2500, 2056, 272, torch.bfloat16, True),
                                              (2305, 2304, 1024, torch.float16, False),
                                              (5000, 1024, 2048, torch.bfloat16, False)])
def test_expand_once_pair_kernel(M, N, K, dtype, bias, epilogue):
    # prefill route: weights expanded to 16 bits once per call, then the CTA-pair kernel; both
    # output routes of its epilogue, ragged M / N and a K tail
    with knobs(PAIR_EPILOGUE=epilogue):
        assert select_path(_lib.OP_W8A16, M, N, K) == "umma_f16_pair_expand_once_tokens256"
        q, s = O.make_weight(N, K, seed=N)
        x = O.make_activation(M, K, seed=M, dtype=dtype, outliers=False)
        b = (torch.randn(N, generator=torch.Generator().manual_seed(1)) * 0.1).to(dtype) if bias else None
        y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda(), None if b is None else b.cuda())
        m = O.tensor_metrics(O.w8a16_native_reference(x, q, s, b), y)
        assert m["relative_l2"] <= 4e-3 and m["cosine_similarity"] >= 0.9999, m
        m = O.tensor_metrics(O.w8a16_dequant_matmul(x, q, s, b), y)
        assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, m
    assert device_status_ok()


def test_prefill_with_odd_channel_count_stays_on_the_shared_memory_kernel():
    # N % 8 != 0: no 16-byte output pieces, so neither the tensor-memory kernel nor the
    # full-line store path applies; element-wise stores of the shared-memory kernel
    M, N, K = 2600, 2052 + 2, 1040
    assert select_path(_lib.OP_W8A16, M, N, K) == "umma_f16_expand_tokens128"
    q, s = O.make_weight(N, K, seed=N)
    x = O.make_activation(M, K, seed=M, outliers=False)
    y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda())
    m = O.tensor_metrics(O.w8a16_native_reference(x, q, s), y)
    assert m["relative_l2"] <= 4e-3 and m["cosine_similarity"] >= 0.9999, m
    assert device_status_ok()


def test_prefill_kernel_expands_every_code_exactly():
    K, M, N = 256, 2560, 2048
    q = torch.stack([torch.roll(torch.arange(-128, 128, dtype=torch.int16).to(torch.int8), i)
                     for i in range(N)])
    s = torch.ones(N)
    for dtype in (torch.bfloat16, torch.float16):
        x = torch.eye(K, dtype=dtype).repeat(M // K, 1)        # row m selects weight column m % K
        y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda())
        assert torch.equal(y.float().cpu(), q.float().T.repeat(M // K, 1)), dtype


@pytest.mark.parametrize("N,K", [(4096, 1024), (1024, 2048), (6144, 1024), (1024, 3072)])
def test_baseline_prefill_shapes_full_size(N, K):
    # M = 8192: sampled rows against the oracle, all rows through linearity in x
    M = 8192
    q, s = O.make_weight(N, K, seed=K)
    x = O.make_activation(M, K, seed=K, outliers=False)
    y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda())
    rows = torch.arange(0, M, 331)
    m = O.tensor_metrics(O.w8a16_dequant_matmul(x[rows], q, s), y[rows])
    assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, m
    m = O.tensor_metrics(O.w8a16_native_reference(x[rows], q, s), y[rows])
    assert m["relative_l2"] <= 4e-3, m
    # checksum over all rows: sum_n y[m, n] == x[m, :] @ (sum_n s[n] * q[n, :])
    colsum = (q.double() * s.double()[:, None]).sum(dim=0)
    expect = x.double() @ colsum
    got = y.double().sum(dim=1).cpu()
    assert torch.allclose(got, expect, rtol=2e-2, atol=2e-2 * float(expect.abs().mean()))
    assert device_status_ok()


@pytest.mark.parametrize("M", [16, 300])
@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 12288)])
def test_qwen3_8b_shapes(M, N, K):
    q, s = O.make_weight(N, K, seed=N)
    x = O.make_activation(M, K, seed=M, outliers=False)
    y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda())
    m = O.tensor_metrics(O.w8a16_native_reference(x, q, s), y)
    assert m["relative_l2"] <= 4e-3 and m["cosine_similarity"] >= 0.9999, m
    m = O.tensor_metrics(O.w8a16_dequant_matmul(x, q, s), y)
    assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, m
    assert device_status_ok()


@pytest.mark.parametrize("M,N,K,dtype,bias", [(128, 1024, 2048, torch.bfloat16, False),
                                              (300, 1024, 3072, torch.bfloat16, True),
                                              (200, 1000, 1040, torch.float16, True),
                                              (256, 4096, 1024, torch.bfloat16, False)])
def test_cluster_split_k(M, N, K, dtype, bias):
    # decode batches of 64-512 tokens: K is split over a cluster of 2 or 4 CTAs and the leader
    # adds the peers' partial tiles from its shared memory; ragged M, N and a K tail included
    q, s = O.make_weight(N, K, seed=N + K)
    x = O.make_activation(M, K, seed=M, dtype=dtype, outliers=False)
    b = (torch.randn(N, generator=torch.Generator().manual_seed(2)) * 0.1).to(dtype) if bias else None
    args = (x.cuda(), q.cuda(), s.cuda(), None if b is None else b.cuda())
    y = apply_int8_weight_only_linear(*args)
    m = O.tensor_metrics(O.w8a16_native_reference(x, q, s, b), y)
    assert m["relative_l2"] <= 4e-3 and m["cosine_similarity"] >= 0.9999, m
    assert torch.equal(bits(y), bits(apply_int8_weight_only_linear(*args)))     # deterministic
    with knobs(CLUSTER=1):                                                      # same kernel, no cluster
        y1 = apply_int8_weight_only_linear(*args)
    assert O.tensor_metrics(y1, y)["relative_l2"] <= 2e-3
    assert device_status_ok()


def test_non_contiguous_activations_are_accepted():
    q, s = O.make_weight(64, 128)
    big = O.make_activation(24, 256).cuda()
    view = big[:, 64:192]                       # row pitch 256, offset 64
    y = apply_int8_weight_only_linear(view, q.cuda(), s.cuda())
    m = O.tensor_metrics(O.w8a16_native_reference(view.cpu(), q, s), y)
    assert m["relative_l2"] <= 4e-3, m


def test_leading_dimensions_are_kept():
    q, s = O.make_weight(64, 128)
    x = O.make_activation(24, 128).view(2, 3, 4, 128)
    y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda())
    assert y.shape == (2, 3, 4, 64)

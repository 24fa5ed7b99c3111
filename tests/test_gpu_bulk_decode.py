"""Persistent decode kernels fed by a shared-memory ring of bulk copies (large matrices, M <= 64).

They replace the register-streaming kernels inside the same kernel family, so the checks are:
the library picks them for large matrices only, W8A8 results are bit-identical to the oracle
and to the register-streaming kernel (knob BULK_DECODE = 1 turns the ring kernels off, 2 uses
them wherever they can run), W8A16 results are within the gates of the reference's
dequantize-then-matmul path and within rounding of the register-streaming kernel's, and ragged
shapes (K not a multiple of the 64-element block or of the 512-element stage, fewer channels
than CTAs, channel shares that are not multiples of 8, M across the 16-token tiles) are handled.
"""
import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import bits, device_status_ok, forced_path, knobs
from tiny_vllm_b200 import _lib
from tiny_vllm_b200.quantization.cuda import (apply_int8_weight_only_linear, apply_w8a8_linear,
                                              select_path, w8a8_int32_accumulators)

pytestmark = pytest.mark.gpu

SHAPES = [  # (M, N, K)
    (1, 1024, 2048), (7, 1029, 2064), (16, 512, 3072), (17, 260, 4096), (33, 1000, 5136),
    (48, 384, 8192), (64, 264, 12288), (5, 96, 17408), (64, 72, 25600), (3, 100, 48), (16, 20000, 528),
    (16, 6144, 4096), (2, 14800, 1024), (32, 520, 4224), (20, 300, 8192), (9, 4096, 12288),
]


def test_library_picks_the_staged_kernels_for_long_rows():
    assert select_path(_lib.OP_W8A8, 16, 6144, 4096) == "bulk_ring_s8_persistent"
    assert select_path(_lib.OP_W8A16, 16, 6144, 4096) == "bulk_ring_w8a16_persistent"
    assert select_path(_lib.OP_W8A8, 16, 6144, 1024) == "mma_stream_s8_splitk"
    with knobs(BULK_DECODE=1):
        assert select_path(_lib.OP_W8A8, 16, 6144, 4096) == "mma_stream_s8_splitk"
    with knobs(BULK_DECODE=2):
        assert select_path(_lib.OP_W8A8, 16, 6144, 1024) == "bulk_ring_s8_persistent"


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_w8a8_bit_exact(M, N, K, oracle_c_lib):
    g = torch.Generator().manual_seed(M + N + K)
    q, s = O.make_weight(N, K, seed=N)
    x = O.make_activation(M, K, seed=M, dtype=torch.bfloat16)
    xq, a_s = O.quantize_per_row_dynamic(x)
    b = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    dev = [t.cuda() for t in (xq, a_s, q, s)]
    ref_acc = O.w8a8_int32_accumulators(xq, q)
    with forced_path("mma"), knobs(BULK_DECODE=2):
        if M > 32:
            assert select_path(_lib.OP_W8A8, M, N, K).startswith("mma_stream")  # at most two token tiles
        else:
            assert select_path(_lib.OP_W8A8, M, N, K).startswith("bulk_ring")
        acc = w8a8_int32_accumulators(dev[0], dev[2])
        y = apply_w8a8_linear(*dev, bias=b.cuda(), out_dtype=torch.bfloat16)
    with forced_path("mma"), knobs(BULK_DECODE=1):
        assert select_path(_lib.OP_W8A8, M, N, K).startswith("mma_stream")
        y_regs = apply_w8a8_linear(*dev, bias=b.cuda(), out_dtype=torch.bfloat16)
    assert torch.equal(bits(y), bits(y_regs))
    with forced_path("mma"), knobs(BULK_DECODE=2, BULK_WPP=1):   # one consumer warp per ring
        assert torch.equal(bits(apply_w8a8_linear(*dev, bias=b.cuda(), out_dtype=torch.bfloat16)), bits(y))
    assert torch.equal(acc.cpu(), ref_acc)
    assert torch.equal(bits(y.cpu()), bits(O.w8a8_native_epilogue(ref_acc, a_s, s, b, torch.bfloat16)))
    assert device_status_ok()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_w8a16_within_the_gates(M, N, K, dtype):
    q, s = O.make_weight(N, K, seed=N)
    x = O.make_activation(M, K, seed=M, dtype=dtype, outliers=False)
    b = (torch.randn(N, generator=torch.Generator().manual_seed(1)) * 0.1).to(dtype)
    dev = [t.cuda() for t in (x, q, s, b)]
    with forced_path("mma"), knobs(BULK_DECODE=2):
        if M > 16:
            pytest.skip("the 16-bit ring kernel takes one token tile")
        assert select_path(_lib.OP_W8A16, M, N, K).startswith("bulk_ring")
        y = apply_int8_weight_only_linear(*dev)
    with forced_path("mma"), knobs(BULK_DECODE=1):
        y_regs = apply_int8_weight_only_linear(*dev)
    m = O.tensor_metrics(O.w8a16_dequant_matmul(x, q, s, b), y)
    assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, m
    m = O.tensor_metrics(O.w8a16_native_reference(x, q, s, b), y)
    assert m["relative_l2"] <= 4e-3, m
    # the two kernels cut K differently, so they differ in the last bits only
    m = O.tensor_metrics(y_regs, y)
    assert m["relative_l2"] <= 2e-3, m
    if M <= 8:
        # up to 8 tokens run the form with the channels on the 16-row side of the MMA; knob
        # BULK_WPP = 1 runs the 16-token form on the same problem
        with forced_path("mma"), knobs(BULK_DECODE=2, BULK_WPP=1):
            y_16 = apply_int8_weight_only_linear(*dev)
        m = O.tensor_metrics(y_16, y)
        assert m["relative_l2"] <= 2e-3, m
    assert device_status_ok()


def test_results_do_not_depend_on_the_launch(oracle_c_lib):
    M, N, K = 16, 6144, 4096
    q, s = O.make_weight(N, K, seed=3)
    x = O.make_activation(M, K, seed=4)
    dev = [t.cuda() for t in (x, q, s)]
    assert select_path(_lib.OP_W8A16, M, N, K).startswith("bulk_ring")
    first = apply_int8_weight_only_linear(*dev)
    for _ in range(5):
        assert torch.equal(bits(apply_int8_weight_only_linear(*dev)), bits(first))
    assert device_status_ok()

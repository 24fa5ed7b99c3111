"""W8A16 GEMM vs the oracle: within rel-L2 1e-2 / cosine 0.9999 of the reference's
dequantize-then-matmul path, and much closer to the fp64 value of the same sum."""
import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import device_status_ok
from tiny_vllm_b200.quantization.cuda import apply_int8_weight_only_linear

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K,bias", [(1, 64, 128, False), (5, 96, 256, True), (37, 192, 256, True),
                                        (130, 320, 1024, False), (256, 6144, 1024, False),
                                        (64, 1000, 1040, True)])
def test_matches_reference_path(dtype, M, N, K, bias):
    q, s = O.make_weight(N, K, seed=N)
    x = O.make_activation(M, K, seed=M, dtype=dtype, outliers=False)
    b = (torch.randn(N, generator=torch.Generator().manual_seed(1)) * 0.1).to(dtype) if bias else None
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
        y = apply_int8_weight_only_linear(c["x"].cuda(), c["q"].cuda(), c["s"].cuda(),
                                          None if c["bias"] is None else c["bias"].cuda())
        m = O.tensor_metrics(c["y_w8a16"], y)
        assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, (c["id"], m)


def test_leading_dimensions_are_kept():
    q, s = O.make_weight(64, 128)
    x = O.make_activation(24, 128).view(2, 3, 4, 128)
    y = apply_int8_weight_only_linear(x.cuda(), q.cuda(), s.cuda())
    assert y.shape == (2, 3, 4, 64)

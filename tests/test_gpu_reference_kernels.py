"""This library against the REFERENCE ITSELF on the GPU, same inputs.

``oracle/build_ref.py`` mirrors the reference's ``nanovllm`` package into the git-ignored
``oracle/_ref/`` and compiles its two CUDA extensions (``nanovllm/quantization/csrc``) for
sm_100a; here its own public functions run unmodified next to ours:

* ``quantize_int8_per_row_dynamic`` (``nanovllm/quantization/utils.py:28-32``) on CUDA tensors
  vs ``b200q_act_quant_i8``: scales within one unit in the last place (torch evaluates the
  division by the constant 127 differently on CUDA and on CPU; the kernel follows the CPU form,
  which is what the golden vectors pin), codes equal except where a tie flips;
* ``native_w8a8_linear`` (``nanovllm/quantization/cuda.py:434-452``: what ``apply_w8a8_linear``
  runs, without its silent fall-back to dequantize + matmul when the extension fails) vs
  ``b200q_w8a8_gemm``: bit-identical without bias (both evaluate ``(float(acc) * a_s) * w_s``
  with one rounding per product); with a bias fewer than 2 % of the outputs may differ in the
  last place (the reference is built with fast-math, which may fuse the last multiply with
  the bias add);
* ``native_int8_weight_only_linear`` (``cuda.py:262-274``) vs ``b200q_w8a16_gemm``: rel-L2 <= 1e-2
  and cosine >= 0.9999 (the reference rounds ``q * s`` to 16 bits before the contraction, this
  library applies ``s`` to the fp32 sum).

Skipped when ``oracle/_ref`` has not been built (no reference checkout was available).
"""
import pytest
import torch

from oracle import build_ref
from oracle import quant_linear_oracle as O
from gpu_util import bits, device_status_ok
from tiny_vllm_b200.quantization.cuda import (apply_int8_weight_only_linear, apply_w8a8_linear,
                                              quantize_activation_int8)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    r = build_ref.load_reference(with_cuda_extensions=True)
    if r is None or not (r.native_w8a8 and r.native_w8a16):
        pytest.skip("oracle/_ref (the reference's package and CUDA extensions) has not been built")
    return r


@pytest.mark.parametrize("M,K", [(1, 1024), (300, 2048), (8192, 3072)])
def test_activation_quantiser_against_the_reference_on_the_gpu(ref, M, K):
    # On CPU tensors the reference's quantiser and b200q_act_quant_i8 agree bit for bit (golden
    # vectors).  On CUDA tensors the reference's `amax.div(127.0)` is evaluated by torch as a
    # multiplication by fl(1 / 127) — a different rounding of the same quotient — so its own GPU
    # result differs from its own CPU result in the last bit of a few scales, and a code that sat
    # on a rounding tie follows.  Bit-identity is therefore shown against the same torch code with
    # a true division; against the multiply form scales are within one unit in the last place.
    x = O.make_activation(M, K, seed=M).cuda()
    q, s = quantize_activation_int8(x)
    xf = x.float()
    s_div = (xf.abs().amax(dim=1) / torch.full((M,), 127.0, device="cuda")).clamp_min(1e-8)
    q_div = torch.round(xf / s_div.unsqueeze(1)).clamp(-127, 127).to(torch.int8)
    assert torch.equal(s, s_div) and torch.equal(q, q_div)
    rq, rs = ref.utils.quantize_int8_per_row_dynamic(x)
    ulp = (s.view(torch.int32) - rs.view(torch.int32)).abs()
    assert int(ulp.max()) <= 1
    assert int((q.int() - rq.int()).abs().max()) <= 1
    assert float((q != rq).float().mean()) < 1e-3


@pytest.mark.parametrize("M", [16, 512, 8192])
@pytest.mark.parametrize("N,K", [(4096, 1024), (1024, 2048), (6144, 1024), (1024, 3072)])
def test_w8a8_matches_the_reference_kernel(ref, M, N, K):
    q, s = O.make_weight(N, K, seed=K)
    x = O.make_activation(M, K, seed=M + K).cuda()
    xq, a_s = ref.utils.quantize_int8_per_row_dynamic(x)
    qd, sd = q.cuda(), s.cuda()
    assert ref.cuda._load_w8a8_extension().select_path(xq, qd) == "wmma_int8_cp_async"
    want = ref.cuda.native_w8a8_linear(xq, a_s, qd, sd, None, torch.bfloat16)
    got = apply_w8a8_linear(xq, a_s, qd, sd, None, torch.bfloat16)
    torch.cuda.synchronize()
    assert torch.equal(bits(got), bits(want))
    assert device_status_ok()


def test_w8a8_with_bias_and_fp16_against_the_reference_kernel(ref):
    M, N, K = 300, 512, 1024
    q, s = O.make_weight(N, K, seed=5)
    for dtype in (torch.bfloat16, torch.float16):
        x = O.make_activation(M, K, seed=9, dtype=dtype).cuda()
        bias = (torch.randn(N, generator=torch.Generator().manual_seed(2)) * 0.1).to(dtype).cuda()
        xq, a_s = ref.utils.quantize_int8_per_row_dynamic(x)
        want = ref.cuda.native_w8a8_linear(xq, a_s, q.cuda(), s.cuda(), bias, dtype)
        got = apply_w8a8_linear(xq, a_s, q.cuda(), s.cuda(), bias, dtype)
        torch.cuda.synchronize()
        assert float((bits(got) != bits(want)).float().mean()) < 0.02, dtype
        m = O.tensor_metrics(want, got)
        assert m["relative_l2"] <= 1e-3 and m["cosine_similarity"] >= 0.9999, m


@pytest.mark.parametrize("M,N,K", [(256, 6144, 1024), (16, 4096, 1024), (2048, 1024, 3072)])
def test_w8a16_within_tolerance_of_the_reference_kernel(ref, M, N, K):
    q, s = O.make_weight(N, K, seed=N)
    x = O.make_activation(M, K, seed=M, outliers=False).cuda()
    want = ref.cuda.native_int8_weight_only_linear(x, q.cuda(), s.cuda(), None)
    got = apply_int8_weight_only_linear(x, q.cuda(), s.cuda(), None)
    torch.cuda.synchronize()
    m = O.tensor_metrics(want, got)
    assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, m
    assert device_status_ok()

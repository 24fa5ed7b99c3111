"""Quantisation fused into its producers (add-RMSNorm, SiLU-mul) vs the oracle.

Two claims per kernel: (1) the 16-bit value the kernel forms is the reference's (restated in
the oracle; summation order and exp differ from torch's CPU code, so a small fraction of
elements may sit one unit in the last place away); (2) the int8 codes and scales are
bit-identical to quantising exactly the 16-bit values the kernel formed."""
import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import bits, device_status_ok
from tiny_vllm_b200.quantization.cuda import (add_rmsnorm_quantize_int8, apply_w8a8_linear,
                                              silu_mul_quantize_int8)

pytestmark = pytest.mark.gpu


def _ulp_report(got, ref):
    d = (bits(got.cpu()).int() - bits(ref).int()).abs()
    return int(d.max()), float((d > 0).float().mean())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K", [(1, 1024), (37, 1024), (300, 2048), (64, 4096), (5, 272), (16, 12288)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_add_rmsnorm_quant(dtype, M, K, with_residual):
    g = torch.Generator().manual_seed(M + K)
    x = O.make_activation(M, K, seed=M, dtype=dtype)
    res = (torch.randn(M, K, generator=g) * 2).to(dtype) if with_residual else None
    w = (1.0 + 0.2 * torch.randn(K, generator=g)).to(dtype)
    eps = 1e-6
    xq, a_s, new_res, y = add_rmsnorm_quantize_int8(
        x.cuda(), w.cuda(), eps, None if res is None else res.cuda(), return_normed=True)
    y_ref, res_ref = O.add_rmsnorm(x, w, eps, res)
    # n = T(s * rsqrt(var)) can sit one unit off (the mean is summed in another order), and the
    # 16-bit multiply by the weight can carry that to two units in a handful of elements
    worst, frac = _ulp_report(y, y_ref)
    assert worst <= 2 and frac <= 0.02, (worst, frac)
    assert O.tensor_metrics(y_ref, y)["relative_l2"] <= 1e-3
    if with_residual:
        assert torch.equal(bits(new_res.cpu()), bits(res_ref))          # fp32 add, one rounding: exact
    else:
        assert new_res is None
    xq_ref, as_ref = O.quantize_per_row_dynamic(y.cpu())                 # of the kernel's own y
    assert torch.equal(xq.cpu(), xq_ref) and torch.equal(a_s.cpu(), as_ref)
    # the unfused route on the GPU gives the same codes when fed the same y
    xq2, a_s2, _, none_y = add_rmsnorm_quantize_int8(x.cuda(), w.cuda(), eps,
                                                      None if res is None else res.cuda())
    assert none_y is None and torch.equal(xq2, xq) and torch.equal(a_s2, a_s)
    assert device_status_ok()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,I", [(1, 3072), (37, 3072), (300, 1024), (8, 12288), (5, 272)])
def test_silu_mul_quant(dtype, M, I):
    g = torch.Generator().manual_seed(M + I)
    gate_up = (torch.randn(M, 2 * I, generator=g) * 2).to(dtype)
    xq, a_s, y = silu_mul_quantize_int8(gate_up.cuda(), return_act=True)
    y_ref = O.silu_mul(gate_up)
    worst, frac = _ulp_report(y, y_ref)
    assert worst <= 1 and frac <= 0.02, (worst, frac)
    xq_ref, as_ref = O.quantize_per_row_dynamic(y.cpu())
    assert torch.equal(xq.cpu(), xq_ref) and torch.equal(a_s.cpu(), as_ref)
    assert device_status_ok()


def test_kernels_against_the_reference_modules(fused_producer_cases):
    """The kernels' 16-bit values against outputs of the reference's own RMSNorm / SiluAndMul
    modules (tests/golden/fused_producers_golden.npz, run operation by operation on CPU).
    Norm: the residual sum is bit-identical; y within 2 units in the last place in <= 2 % of the
    elements (the mean is summed in another order).  Activation: the kernel rounds
    silu(gate) * up once, as the module's compiled form does, while the fixture rounds silu(gate)
    first: never more than one unit apart, in under 30 % of the elements."""
    norm, silu = fused_producer_cases
    for c in norm:
        xq, a_s, new_res, y = add_rmsnorm_quantize_int8(
            c["x"].cuda(), c["w"].cuda(), c["eps"], None if c["res"] is None else c["res"].cuda(),
            return_normed=True)
        worst, frac = _ulp_report(y, c["y"])
        assert worst <= 2 and frac <= 0.02, (c["id"], worst, frac)
        if c["res"] is not None:
            assert torch.equal(bits(new_res.cpu()), bits(c["new_res"])), c["id"]
    for c in silu:
        _, _, y = silu_mul_quantize_int8(c["gate_up"].cuda(), return_act=True)
        worst, frac = _ulp_report(y, c["y"])
        assert worst <= 1 and frac <= 0.30, (c["id"], worst, frac)
        worst, frac = _ulp_report(y, O.silu_mul(c["gate_up"]))
        assert worst <= 1 and frac <= 0.02, (c["id"], worst, frac)
    assert device_status_ok()


def test_fused_producers_feed_the_w8a8_layers():
    """An MLP block the way the reference's model runs it (qwen3.py:117-122,160-166), with the
    two quantisers fused into the norm and the activation, against the oracle's path."""
    from tiny_vllm_b200.layers.linear import MergedColumnParallelLinear, RowParallelLinear
    M, H, I = 48, 1024, 3072
    g = torch.Generator().manual_seed(3)
    hidden = O.make_activation(M, H, seed=1)
    residual = (torch.randn(M, H, generator=g)).to(torch.bfloat16)
    norm_w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    q_gu, s_gu = O.make_weight(2 * I, H, seed=4)
    q_dn, s_dn = O.make_weight(H, I, seed=5)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    with torch.device("cuda"):
        gate_up = MergedColumnParallelLinear(H, [I, I], quantization="w8a8")
        down = RowParallelLinear(I, H, quantization="w8a8")
    torch.set_default_dtype(prev)
    gate_up.qweight.weight_loader(gate_up.qweight, q_gu)
    gate_up.w_scales.weight_loader(gate_up.w_scales, s_gu)
    down.qweight.weight_loader(down.qweight, q_dn)
    down.w_scales.weight_loader(down.w_scales, s_dn)
    # fused: norm+quant -> GEMM -> silu-mul+quant -> GEMM
    xq, a_s, new_res, _ = add_rmsnorm_quantize_int8(hidden.cuda(), norm_w.cuda(), 1e-6, residual.cuda())
    gu = gate_up.quant_method.apply_quantized(xq, a_s, gate_up, torch.bfloat16)
    xq2, a_s2, _ = silu_mul_quantize_int8(gu)
    out = down.quant_method.apply_quantized(xq2, a_s2, down, torch.bfloat16)
    # oracle: the same chain on the CPU
    y_ref, res_ref = O.add_rmsnorm(hidden, norm_w, 1e-6, residual)
    rq, ra = O.quantize_per_row_dynamic(y_ref)
    gu_ref = O.w8a8_native_epilogue(O.w8a8_int32_accumulators(rq, q_gu), ra, s_gu, None, torch.bfloat16)
    aq, aa = O.quantize_per_row_dynamic(O.silu_mul(gu_ref))
    out_ref = O.w8a8_native_epilogue(O.w8a8_int32_accumulators(aq, q_dn), aa, s_dn, None, torch.bfloat16)
    m = O.tensor_metrics(out_ref, out)
    assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, m
    assert torch.equal(bits(new_res.cpu()), bits(res_ref))
    # and equals the layers' own (unfused) forward on the same normalised input, bit for bit
    y_gpu = add_rmsnorm_quantize_int8(hidden.cuda(), norm_w.cuda(), 1e-6, residual.cuda(),
                                      return_normed=True)[3]
    assert torch.equal(bits(gate_up(y_gpu)), bits(gu))
    assert device_status_ok()

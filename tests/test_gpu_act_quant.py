"""Activation-quant kernel vs the CPU oracle: int8 codes and fp32 scales bit-identical."""
import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import device_status_ok
from tiny_vllm_b200.quantization.cuda import quantize_activation_int8
from tiny_vllm_b200.quantization.utils import quantize_int8_per_row_dynamic

pytestmark = pytest.mark.gpu


def check(x_cpu):
    xq, a_s = quantize_activation_int8(x_cpu.cuda())
    eq, es = O.quantize_per_row_dynamic(x_cpu)
    assert torch.equal(a_s.cpu(), es)
    assert torch.equal(xq.cpu(), eq)


@pytest.mark.parametrize("M,K", [(1, 16), (3, 48), (7, 256), (33, 512), (130, 1024), (65, 2048),
                                 (19, 3072), (9, 4096), (5, 12288), (3, 16384), (2, 20480)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_matches_oracle(M, K, dtype):
    check(O.make_activation(M, K, seed=M + K, dtype=dtype))


def test_golden_cases(golden_cases):
    for c in golden_cases:
        xq, a_s = quantize_activation_int8(c["x"].cuda())
        assert torch.equal(xq.cpu(), c["xq"]) and torch.equal(a_s.cpu(), c["a_s"])


def test_edge_values_and_ties():
    x = torch.zeros(6, 64, dtype=torch.bfloat16)
    x[1, 3] = -7.0                       # lone negative maximum -> -127
    x[2] = 1e-30                         # below the eps clamp
    x[3, :] = torch.linspace(-4, 4, 64)  # includes rounding ties after division
    x[4, 0] = 3.0e38                     # near the top of the bf16 range
    x[5, 1::2] = 0.5
    x[5, 0] = 127.0                      # scale exactly 1: 0.5 is a tie -> rounds to even (0)
    check(x)


def test_strided_rows_and_empty():
    big = O.make_activation(40, 256, seed=3).cuda()
    view = big[:, :128]                  # row pitch 256, K = 128: handled without a copy
    xq, a_s = quantize_activation_int8(view)
    eq, es = O.quantize_per_row_dynamic(view.cpu())
    assert torch.equal(xq.cpu(), eq) and torch.equal(a_s.cpu(), es)
    xq, a_s = quantize_int8_per_row_dynamic(torch.empty(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert xq.shape == (0, 64) and a_s.shape == (0,)


def test_full_size_properties():
    # the benchmark's prefill size (8192 tokens, widest input): codes bounded, scale * 127 reproduces the row maximum, idempotent
    x = O.make_activation(8192, 3072, seed=11).cuda()
    xq, a_s = quantize_activation_int8(x)
    assert int(xq.abs().max()) == 127 and int(xq.min()) >= -127
    amax = x.float().abs().amax(dim=1)
    assert torch.equal(a_s, torch.clamp_min(amax / 127.0, 1e-8)) or \
        torch.allclose(a_s, amax / 127.0, rtol=1e-6)
    assert torch.equal(xq.abs().amax(dim=1), torch.full((8192,), 127, dtype=torch.int8, device="cuda"))
    rows = torch.arange(0, 8192, 257)
    eq, es = O.quantize_per_row_dynamic(x[rows].cpu())
    assert torch.equal(xq[rows].cpu(), eq) and torch.equal(a_s[rows].cpu(), es)
    assert device_status_ok()

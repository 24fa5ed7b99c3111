"""W8A16: int8 weights with one fp32 scale per output channel, 16-bit activations.

Mirrors ``Int8WeightOnlyQuantMethod`` of the reference
(``nanovllm/quantization/int8.py:8-29``): parameters ``qweight`` int8 ``[N, K]`` and
``scales`` fp32 ``[N]``.
"""
from __future__ import annotations

import torch
from torch import nn

from .base import QuantMethod, frozen
from .cuda import apply_int8_weight_only_linear


class Int8WeightOnlyQuantMethod(QuantMethod):

    def create_weights(self, layer: nn.Module, input_size: int, output_size: int) -> None:
        layer.qweight = frozen((output_size, input_size), torch.int8)
        layer.scales = frozen((output_size,), torch.float32)

    def quantize_activation(self, x: torch.Tensor) -> None:
        return None

    def apply(self, x: torch.Tensor, layer: nn.Module,
              bias: torch.Tensor | None = None) -> torch.Tensor:
        chosen_bias = bias if bias is not None else layer.bias
        return apply_int8_weight_only_linear(x, layer.qweight, layer.scales, chosen_bias)

    def apply_row_parallel(self, x: torch.Tensor, layer: nn.Module, bias, comm):
        """Multiply and sum over the tensor-parallel ranks in one GEMM kernel (decode-sized
        batches); ``None`` when the fused kernel does not take the shape."""
        n_out = layer.qweight.shape[0]
        tokens = x.numel() // x.shape[-1]
        if not comm.fused_fits(tokens, n_out) or x.dtype not in (torch.float16, torch.bfloat16):
            return None
        chosen = bias if bias is not None else layer.bias
        x_2d = x.contiguous().view(-1, x.shape[-1])
        y = comm.fused_w8a16(x_2d, layer.qweight, layer.scales, chosen)
        return None if y is None else y.view(*x.shape[:-1], n_out)

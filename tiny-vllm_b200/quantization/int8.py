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

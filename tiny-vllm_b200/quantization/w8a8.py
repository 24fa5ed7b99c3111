"""W8A8: int8 weights (fp32 scale per output channel) and per-token dynamically
quantised int8 activations, int32 accumulation.

Mirrors ``W8A8QuantMethod`` of the reference (``nanovllm/quantization/w8a8.py:9-40``):
parameters ``qweight`` int8 ``[N, K]`` and ``w_scales`` fp32 ``[N]``; ``apply`` flattens
the tokens, quantises them, and runs the int8 GEMM with the fused scale epilogue.
"""
from __future__ import annotations

import torch
from torch import nn

from .base import QuantMethod, frozen
from .cuda import apply_w8a8_linear, quantize_activation_int8


class W8A8QuantMethod(QuantMethod):

    def create_weights(self, layer: nn.Module, input_size: int, output_size: int) -> None:
        layer.qweight = frozen((output_size, input_size), torch.int8)
        layer.w_scales = frozen((output_size,), torch.float32)

    def quantize_activation(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        tokens = x.reshape(-1, x.shape[-1])
        return quantize_activation_int8(tokens)

    def apply(self, x: torch.Tensor, layer: nn.Module,
              bias: torch.Tensor | None = None) -> torch.Tensor:
        x_q, a_scales = self.quantize_activation(x)
        n_out = layer.qweight.shape[0]
        return apply_w8a8_linear(
            x_q, a_scales, layer.qweight, layer.w_scales,
            bias=layer.bias if bias is None else bias,
            out_dtype=x.dtype,
            out_shape=(*x.shape[:-1], n_out),
        )

    def apply_quantized(self, x_q: torch.Tensor, a_scales: torch.Tensor, layer: nn.Module,
                        out_dtype: torch.dtype, bias: torch.Tensor | None = None,
                        out_shape: tuple[int, ...] | None = None,
                        out: torch.Tensor | None = None) -> torch.Tensor:
        """The linear on activations that are already quantised — by
        ``add_rmsnorm_quantize_int8`` / ``silu_mul_quantize_int8`` fused into the producer of
        ``x``, or by ``quantize_activation``.  (No counterpart in the reference, whose ``apply``
        always quantises itself: ``nanovllm/quantization/w8a8.py:25-40``.)  ``out``: a
        contiguous ``[tokens, out_features]`` tensor to write into, e.g. ``comm.buffer(...)`` of
        the tensor-parallel communicator when ``comm.reduce_rmsnorm_quant`` consumes the result."""
        return apply_w8a8_linear(x_q, a_scales, layer.qweight, layer.w_scales,
                                 bias=layer.bias if bias is None else bias,
                                 out_dtype=out_dtype, out_shape=out_shape, out=out)

    def apply_row_parallel(self, x: torch.Tensor, layer: nn.Module, bias, comm):
        """Quantise, multiply and sum over the tensor-parallel ranks with the exchange fused
        into the GEMM: one kernel for decode-sized batches, GEMM + reduce-scatter under the
        main loop followed by a sum-and-gather kernel for prefill-sized ones.  ``None`` when
        neither takes the shape."""
        n_out = layer.qweight.shape[0]
        tokens = x.numel() // x.shape[-1]
        small = comm.fused_fits(tokens, n_out)
        large = not small and getattr(comm, "tiled_fits", lambda *_: False)(tokens, n_out)
        if not (small or large) or x.dtype not in (torch.float16, torch.bfloat16):
            return None
        x_q, a_scales = self.quantize_activation(x)
        chosen = layer.bias if bias is None else bias
        if chosen is not None:
            chosen = chosen.contiguous()
        fused = comm.fused_w8a8 if small else comm.fused_w8a8_tiled
        y = fused(x_q, a_scales, layer.qweight, layer.w_scales, chosen, x.dtype)
        return None if y is None else y.view(*x.shape[:-1], n_out)

"""Plug-in interface of a linear-layer quantization scheme.

Same three hooks as the reference's ``QuantMethod`` (``nanovllm/quantization/base.py:7-24``):
a layer asks its method to register the weight parameters, and routes every
forward through ``apply``.
"""
from __future__ import annotations

import abc

import torch
from torch import nn


class QuantMethod(abc.ABC):
    """How a linear layer stores its weight and computes ``x @ W.T + b``."""

    @abc.abstractmethod
    def create_weights(self, layer: nn.Module, input_size: int, output_size: int) -> None:
        """Registers the (frozen) weight parameters on ``layer``."""

    @abc.abstractmethod
    def apply(self, x: torch.Tensor, layer: nn.Module,
              bias: torch.Tensor | None = None) -> torch.Tensor:
        """Runs the linear.  An explicit ``bias`` wins over ``layer.bias``."""

    @abc.abstractmethod
    def quantize_activation(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor] | None:
        """Returns ``(x_q, a_scales)`` or ``None`` when activations stay in 16 bit."""

    def apply_row_parallel(self, x: torch.Tensor, layer: nn.Module, bias, comm):
        """Optional: the linear and the sum over tensor-parallel ranks in one kernel, through
        ``comm`` (``layers.tp_comm.PeerAllReduce``).  ``None`` = not available for this call;
        the layer then runs ``apply`` followed by an all-reduce.  (No counterpart in the
        reference, which always runs the two steps: ``nanovllm/layers/linear.py:265-276``.)"""
        return None


def frozen(shape: tuple[int, ...], dtype: torch.dtype) -> nn.Parameter:
    """An uninitialised parameter that takes no gradient."""
    return nn.Parameter(torch.empty(*shape, dtype=dtype), requires_grad=False)

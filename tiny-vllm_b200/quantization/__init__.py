"""Quantization plug-ins of the linear layers (reference: ``nanovllm/quantization``)."""
from .base import QuantMethod
from .int8 import Int8WeightOnlyQuantMethod
from .w8a8 import W8A8QuantMethod

__all__ = ["QuantMethod", "Int8WeightOnlyQuantMethod", "W8A8QuantMethod"]

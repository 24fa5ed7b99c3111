"""Layers on the quantized-linear path (reference: ``nanovllm/layers/linear.py``)."""
from .linear import (ColumnParallelLinear, LinearBase, MergedColumnParallelLinear,
                     QKVParallelLinear, ReplicatedLinear, RowParallelLinear)

__all__ = ["LinearBase", "ReplicatedLinear", "ColumnParallelLinear",
           "MergedColumnParallelLinear", "QKVParallelLinear", "RowParallelLinear"]

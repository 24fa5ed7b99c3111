"""Quantisation helpers shared by the offline artifact tool and the W8A8 method.

Counterpart of ``nanovllm/quantization/utils.py``.
"""
from __future__ import annotations

from pathlib import Path

import torch

from .cuda import quantize_activation_int8

# HF parameter-name endings of the Qwen3 projections that get quantised
# (reference: nanovllm/quantization/utils.py:6-18).
QWEN3_INT8_WEIGHT_SUFFIXES = tuple(
    f".{block}.{proj}.weight"
    for block, projs in (("self_attn", ("q_proj", "k_proj", "v_proj", "o_proj")),
                         ("mlp", ("gate_proj", "up_proj", "down_proj")))
    for proj in projs
)


def is_qwen3_int8_target_weight(name: str) -> bool:
    return name.endswith(QWEN3_INT8_WEIGHT_SUFFIXES)


def quantize_int8_per_channel(weight: torch.Tensor, eps: float = 1e-8) -> tuple[torch.Tensor, torch.Tensor]:
    """Offline symmetric weight quantisation, one scale per output channel (row).

    ``scale = max(absmax(row) / 127, eps)``; ``q = clamp(round_half_even(w / scale), ±127)``.
    Runs with torch ops on whatever device holds ``weight`` — it is artifact
    tooling, not part of the per-token path
    (reference: nanovllm/quantization/utils.py:21-25).
    """
    w32 = weight.to(torch.float32)
    scales = (w32.abs().amax(dim=1) / 127.0).clamp_min(eps)
    q = (w32 / scales[:, None]).round_().clamp_(-127, 127).to(torch.int8)
    return q, scales


def quantize_int8_per_row_dynamic(x: torch.Tensor, eps: float = 1e-8) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token dynamic activation quantisation (reference: utils.py:28-32), done by
    one CUDA kernel.  ``x`` must be a 2-D fp16/bf16 CUDA tensor; ``eps`` is fixed at
    1e-8 inside the kernel."""
    if eps != 1e-8:
        raise ValueError("the CUDA kernel implements eps = 1e-8 only")
    return quantize_activation_int8(x)


def iter_model_files(model_path: Path):
    """Files of a model directory that are not tensor shards."""
    for entry in Path(model_path).iterdir():
        if entry.is_file() and entry.suffix != ".safetensors":
            yield entry

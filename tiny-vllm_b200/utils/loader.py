"""Loads safetensors weights (plain HF checkpoints or quantized artifacts) into a model.

Counterpart of ``nanovllm/utils/loader.py:44-68`` with the same contract:

1. a stored tensor whose name is exactly a model parameter is handed to that
   parameter's ``weight_loader`` (this is how ``...qkv_proj.qweight`` /
   ``...gate_up_proj.scales`` of a quantized artifact arrive, already packed);
2. otherwise the model's ``packed_modules_mapping`` (HF name fragment ->
   (packed parameter fragment, shard id)) routes unpacked HF tensors such as
   ``q_proj.weight`` into their slice of the packed parameter;
3. after loading, a quantized model must have received every ``.qweight`` and every
   scale tensor (``.scales`` for ``"int8"``, ``.w_scales`` for ``"w8a8"``) —
   reference lines 27-41.

The exact-name test comes first on purpose: ``up_proj`` is a substring of
``gate_up_proj``, so fragment matching alone would misroute packed artifact names.
"""
from __future__ import annotations

import os
from glob import glob

import torch
from safetensors import safe_open
from torch import nn

_SCALE_SUFFIX = {"int8": ".scales", "w8a8": ".w_scales"}


def default_weight_loader(param: nn.Parameter, loaded_weight: torch.Tensor):
    param.data.copy_(loaded_weight)


def _lookup(model: nn.Module, name: str) -> nn.Parameter | None:
    try:
        return model.get_parameter(name)
    except AttributeError:
        return None


def _deliver(model: nn.Module, name: str, tensor: torch.Tensor, done: set[str], *shard):
    param = model.get_parameter(name)
    getattr(param, "weight_loader", default_weight_loader)(param, tensor, *shard)
    done.add(name)


def _route(model: nn.Module, stored_name: str, tensor: torch.Tensor, packed: dict, done: set[str]):
    if _lookup(model, stored_name) is not None:
        _deliver(model, stored_name, tensor, done)
        return
    for fragment, (target, shard_id) in packed.items():
        if fragment in stored_name:
            _deliver(model, stored_name.replace(fragment, target), tensor, done, shard_id)
            return
    _deliver(model, stored_name, tensor, done)  # raises AttributeError for unknown names


def _require_quantized_tensors(model: nn.Module, done: set[str], quantization: str):
    suffix = _SCALE_SUFFIX[quantization]
    wanted = {n for n, _ in model.named_parameters() if n.endswith(".qweight") or n.endswith(suffix)}
    missing = sorted(wanted - done)
    if missing:
        shown = ", ".join(missing[:8])
        if len(missing) > 8:
            shown += f", ... ({len(missing)} missing total)"
        label = "INT8" if quantization == "int8" else "W8A8"
        raise RuntimeError(
            f"Missing {label} quantized tensors. Expected qweight/{suffix[1:]} for quantized "
            f"linear layers, but did not load: {shown}")


def load_model(model: nn.Module, path: str, quantization: str | None = None):
    packed = getattr(model, "packed_modules_mapping", {})
    files = sorted(glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"No safetensors files found in {path}")
    done: set[str] = set()
    for file in files:
        with safe_open(file, "pt", "cpu") as f:
            for stored_name in f.keys():
                _route(model, stored_name, f.get_tensor(stored_name), packed, done)
    if quantization in _SCALE_SUFFIX:
        _require_quantized_tensors(model, done, quantization)

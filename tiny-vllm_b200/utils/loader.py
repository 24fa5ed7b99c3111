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

Unlike the reference, which reads every full tensor on every rank and lets the
``weight_loader`` throw most of it away (reference lines 50-64), a parameter that carries a
``shard_plan`` hook (all layers of ``layers.linear``) is filled from slices of the stored
tensor: only this rank's rows or columns are read from disk (1 / tp of the weight bytes), and
no full tensor is ever materialised — the 8B checkpoint's largest matrix is 200 MB in 16 bit.
``load_model(..., sharded_reads=False)`` keeps to the ``weight_loader`` hooks.
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


def _deliver(model: nn.Module, name: str, handle, stored_name: str, done: set[str], sharded: bool,
             stats: dict, *shard):
    """Fills parameter ``name`` from the stored tensor ``stored_name`` of the open file."""
    param = model.get_parameter(name)
    plan = getattr(param, "shard_plan", None) if sharded else None
    if plan is not None:
        view = handle.get_slice(stored_name)
        for dst_index, src_index in plan(view.get_shape(), *shard):
            piece = view[src_index]
            param.data[dst_index].copy_(piece)
            stats["bytes_read"] += piece.numel() * piece.element_size()
    else:
        tensor = handle.get_tensor(stored_name)
        getattr(param, "weight_loader", default_weight_loader)(param, tensor, *shard)
        stats["bytes_read"] += tensor.numel() * tensor.element_size()
    done.add(name)


def _route(model: nn.Module, handle, stored_name: str, packed: dict, done: set[str], sharded: bool,
           stats: dict):
    if _lookup(model, stored_name) is not None:
        _deliver(model, stored_name, handle, stored_name, done, sharded, stats)
        return
    for fragment, (target, shard_id) in packed.items():
        if fragment in stored_name:
            _deliver(model, stored_name.replace(fragment, target), handle, stored_name, done, sharded,
                     stats, shard_id)
            return
    # raises AttributeError for unknown names
    _deliver(model, stored_name, handle, stored_name, done, sharded, stats)


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


def load_model(model: nn.Module, path: str, quantization: str | None = None,
               sharded_reads: bool = True) -> dict:
    """Same call as the reference's ``load_model``.  Returns ``{"bytes_read": n}``: the tensor
    bytes this rank fetched from the files."""
    packed = getattr(model, "packed_modules_mapping", {})
    files = sorted(glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"No safetensors files found in {path}")
    done: set[str] = set()
    stats = {"bytes_read": 0}
    for file in files:
        with safe_open(file, "pt", "cpu") as f:
            for stored_name in f.keys():
                _route(model, f, stored_name, packed, done, sharded_reads, stats)
    if quantization in _SCALE_SUFFIX:
        _require_quantized_tensors(model, done, quantization)
    return stats

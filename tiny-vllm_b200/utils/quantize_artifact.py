"""Offline tool: turns a Hugging Face Qwen3 checkpoint directory into the quantized
artifact layout the loader expects.

Layout (identical to what ``scripts/quantize.py:79-139`` of the reference writes):

* ``<layer>.self_attn.qkv_proj.qweight``  int8  ``[q+k+v rows, hidden]`` — q, k, v
  weights concatenated along dim 0 in that order, then quantised per output channel;
* ``<layer>.mlp.gate_up_proj.qweight``    int8  — gate then up, same treatment;
* ``<layer>.self_attn.o_proj.qweight`` / ``<layer>.mlp.down_proj.qweight`` — quantised as is;
* beside every ``.qweight`` one fp32 ``[rows]`` tensor named ``.scales`` (mode ``int8``)
  or ``.w_scales`` (mode ``w8a8``);
* q/k/v and gate/up biases, when present, concatenated the same way, kept in 16 bit;
* every other tensor copied unchanged; one ``model.safetensors`` (several numbered shards
  when the output exceeds ``--shard-gib``; the loader reads every ``*.safetensors``);
  non-tensor files (config, tokenizer) copied beside it.

The checkpoint is streamed: tensors are read one at a time from the source shards and at most
one output shard is held in memory.

Usage: ``python -m tiny_vllm_b200.utils.quantize_artifact --model SRC --output DST
--quantization int8|w8a8 [--overwrite]``
"""
from __future__ import annotations

import argparse
import shutil
from pathlib import Path

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from ..quantization.utils import quantize_int8_per_channel

# packed name -> ordered member projections
_PACKS = {"qkv_proj": ("q_proj", "k_proj", "v_proj"), "gate_up_proj": ("gate_proj", "up_proj")}
_DIRECT = ("o_proj", "down_proj")


def _split(name: str) -> tuple[str, str, str] | None:
    """'a.b.q_proj.weight' -> ('a.b.', 'q_proj', 'weight'); None if not of that form."""
    parts = name.rsplit(".", 2)
    if len(parts) != 3 or parts[2] not in ("weight", "bias"):
        return None
    return parts[0] + ".", parts[1], parts[2]


class _Source:
    """Name -> tensor access to a checkpoint without holding it: an in-memory dict, or an index
    of which safetensors file stores which name (tensors are read one at a time on demand)."""

    def __init__(self, tensors: dict[str, torch.Tensor] | None = None, model_dir: Path | None = None):
        self._tensors = tensors
        self._where: dict[str, Path] = {}
        if tensors is None:
            shards = sorted(Path(model_dir).glob("*.safetensors"))
            if not shards:
                raise FileNotFoundError(f"No safetensors files found in {model_dir}")
            for shard in shards:
                with safe_open(shard, "pt", "cpu") as f:
                    for name in f.keys():
                        if name in self._where:
                            raise ValueError(f"Duplicate tensor name across safetensors files: {name}")
                        self._where[name] = shard

    def names(self):
        return list(self._tensors) if self._tensors is not None else list(self._where)

    def get(self, name: str) -> torch.Tensor:
        if self._tensors is not None:
            return self._tensors[name]
        with safe_open(self._where[name], "pt", "cpu") as f:
            return f.get_tensor(name)


def _quantize(weight: torch.Tensor, device: torch.device | None):
    """Per-channel quantisation of one matrix.  On a CUDA device a 16-bit matrix goes through
    the activation-quantiser kernel, whose arithmetic per row is the same as the per-channel
    rule (absmax / 127, clamp, divide, round half to even): bit-identical to the CPU result."""
    if device is not None and device.type == "cuda" and weight.dtype in (torch.float16, torch.bfloat16) \
            and weight.shape[1] % 16 == 0:
        from ..quantization.cuda import quantize_activation_int8
        q, s = quantize_activation_int8(weight.to(device))
        return q.cpu(), s.cpu()
    return quantize_int8_per_channel(weight)


def iter_quantized_tensors(source: _Source, quantization: str, device: torch.device | None = None):
    """Yields ``(name, tensor)`` of the artifact one tensor at a time: at most the members of one
    packed projection are in memory together."""
    scale_name = {"int8": "scales", "w8a8": "w_scales"}[quantization]
    member_to_pack = {m: p for p, members in _PACKS.items() for m in members}
    seen_groups: set[tuple[str, str, str]] = set()
    names = source.names()
    present = set(names)
    for name in names:
        parsed = _split(name)
        if parsed and parsed[1] in member_to_pack:
            prefix, proj, kind = parsed
            pack = member_to_pack[proj]
            if (prefix, pack, kind) in seen_groups:
                continue
            seen_groups.add((prefix, pack, kind))
            members = [f"{prefix}{m}.{kind}" for m in _PACKS[pack]]
            absent = [m for m, full in zip(_PACKS[pack], members) if full not in present]
            if absent:
                raise ValueError(f"Missing {pack} {kind} shards for {prefix}: {absent}")
            stacked = torch.cat([source.get(full) for full in members], dim=0)
            if kind == "weight":
                q, s = _quantize(stacked, device)
                yield f"{prefix}{pack}.qweight", q.contiguous()
                yield f"{prefix}{pack}.{scale_name}", s.contiguous()
            else:
                yield f"{prefix}{pack}.bias", stacked.contiguous()
        elif parsed and parsed[1] in _DIRECT and parsed[2] == "weight":
            q, s = _quantize(source.get(name), device)
            yield f"{parsed[0]}{parsed[1]}.qweight", q.contiguous()
            yield f"{parsed[0]}{parsed[1]}.{scale_name}", s.contiguous()
        else:
            yield name, source.get(name).contiguous()


def build_quantized_tensors(tensors: dict[str, torch.Tensor], quantization: str) -> dict[str, torch.Tensor]:
    """The whole artifact of an in-memory checkpoint as a dict (small models, tests)."""
    return dict(iter_quantized_tensors(_Source(tensors=tensors), quantization))


def copy_model_files(model_dir: Path, output_dir: Path):
    """Everything of the model directory that is not a tensor shard (config, tokenizer, ...)."""
    for entry in Path(model_dir).iterdir():
        is_shard = entry.suffix == ".safetensors" or entry.name.endswith(".safetensors.index.json")
        if entry.is_dir():
            shutil.copytree(entry, output_dir / entry.name, dirs_exist_ok=True,
                            ignore=shutil.ignore_patterns("*.safetensors"))
        elif not is_shard:
            shutil.copy2(entry, output_dir / entry.name)


def quantize_directory(model: Path, output: Path, quantization: str, overwrite: bool = False,
                       shard_bytes: int = 4 << 30, device: str | None = None) -> list[Path]:
    """Streams the checkpoint through the quantiser.  Output tensors are collected up to
    ``shard_bytes`` and written as ``model.safetensors`` (one shard) or
    ``model-0000i.safetensors`` (several): peak memory is one output shard plus one packed
    projection, whatever the model size (the 8B checkpoint is 16 GB in 16 bit).  ``device``:
    ``"cuda"`` quantises on the GPU.  Returns the files written."""
    model, output = Path(model), Path(output)
    if not model.is_dir():
        raise NotADirectoryError(model)
    if output.exists() and overwrite:
        shutil.rmtree(output)
    output.mkdir(parents=True, exist_ok=True)
    copy_model_files(model, output)
    dev = torch.device(device) if device else None
    pending: dict[str, torch.Tensor] = {}
    pending_bytes, written = 0, []

    def flush():
        nonlocal pending, pending_bytes
        if pending:
            path = output / f"model-{len(written):05d}.safetensors"
            save_file(pending, path)
            written.append(path)
            pending, pending_bytes = {}, 0

    for name, tensor in iter_quantized_tensors(_Source(model_dir=model), quantization, dev):
        size = tensor.numel() * tensor.element_size()
        if pending and pending_bytes + size > shard_bytes:
            flush()
        pending[name] = tensor
        pending_bytes += size
    flush()
    if len(written) == 1:       # the single-file name the reference's tool writes
        single = output / "model.safetensors"
        written[0].rename(single)
        written = [single]
    return written


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, type=Path)
    ap.add_argument("--output", required=True, type=Path)
    ap.add_argument("--quantization", default="int8", choices=["int8", "w8a8"])
    ap.add_argument("--overwrite", action="store_true")
    ap.add_argument("--device", default=None, help="'cuda' quantises on the GPU (same bits)")
    ap.add_argument("--shard-gib", type=float, default=4.0, help="largest output shard in GiB")
    args = ap.parse_args()
    quantize_directory(args.model, args.output, args.quantization, args.overwrite,
                       shard_bytes=int(args.shard_gib * (1 << 30)), device=args.device)
    print(f"Wrote {args.quantization.upper()} quantized model to {args.output}")


if __name__ == "__main__":
    main()

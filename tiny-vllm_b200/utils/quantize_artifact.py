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
* every other tensor copied unchanged; everything in one ``model.safetensors``;
  non-tensor files (config, tokenizer) copied beside it.

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


def build_quantized_tensors(tensors: dict[str, torch.Tensor], quantization: str) -> dict[str, torch.Tensor]:
    scale_name = {"int8": "scales", "w8a8": "w_scales"}[quantization]
    member_to_pack = {m: p for p, members in _PACKS.items() for m in members}
    out: dict[str, torch.Tensor] = {}
    groups: dict[tuple[str, str, str], dict[str, torch.Tensor]] = {}

    def emit_quantized(stem: str, weight: torch.Tensor):
        q, s = quantize_int8_per_channel(weight)
        out[f"{stem}.qweight"] = q.contiguous()
        out[f"{stem}.{scale_name}"] = s.contiguous()

    for name, tensor in tensors.items():
        parsed = _split(name)
        if parsed and parsed[1] in member_to_pack:
            prefix, proj, kind = parsed
            groups.setdefault((prefix, member_to_pack[proj], kind), {})[proj] = tensor
        elif parsed and parsed[1] in _DIRECT and parsed[2] == "weight":
            emit_quantized(parsed[0] + parsed[1], tensor)
        else:
            out[name] = tensor.contiguous()

    for (prefix, pack, kind), members in groups.items():
        absent = [m for m in _PACKS[pack] if m not in members]
        if absent:
            raise ValueError(f"Missing {pack} {kind} shards for {prefix}: {absent}")
        stacked = torch.cat([members[m] for m in _PACKS[pack]], dim=0)
        if kind == "weight":
            emit_quantized(prefix + pack, stacked)
        else:
            out[f"{prefix}{pack}.bias"] = stacked.contiguous()
    return out


def load_tensors(model_dir: Path) -> dict[str, torch.Tensor]:
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"No safetensors files found in {model_dir}")
    tensors: dict[str, torch.Tensor] = {}
    for file in files:
        with safe_open(file, "pt", "cpu") as f:
            for name in f.keys():
                if name in tensors:
                    raise ValueError(f"Duplicate tensor name across safetensors files: {name}")
                tensors[name] = f.get_tensor(name)
    return tensors


def copy_model_files(model_dir: Path, output_dir: Path):
    for src in Path(model_dir).iterdir():
        if src.is_dir():
            shutil.copytree(src, output_dir / src.name,
                            ignore=shutil.ignore_patterns("*.safetensors"), dirs_exist_ok=True)
        elif src.suffix != ".safetensors" and not src.name.endswith(".safetensors.index.json"):
            shutil.copy2(src, output_dir / src.name)


def quantize_directory(model: Path, output: Path, quantization: str, overwrite: bool = False):
    model, output = Path(model), Path(output)
    if not model.is_dir():
        raise NotADirectoryError(model)
    if output.exists() and overwrite:
        shutil.rmtree(output)
    output.mkdir(parents=True, exist_ok=True)
    copy_model_files(model, output)
    save_file(build_quantized_tensors(load_tensors(model), quantization), output / "model.safetensors")


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, type=Path)
    ap.add_argument("--output", required=True, type=Path)
    ap.add_argument("--quantization", default="int8", choices=["int8", "w8a8"])
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args()
    quantize_directory(args.model, args.output, args.quantization, args.overwrite)
    print(f"Wrote {args.quantization.upper()} quantized model to {args.output}")


if __name__ == "__main__":
    main()

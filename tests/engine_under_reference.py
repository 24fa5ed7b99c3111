"""Runs the REFERENCE'S OWN ENGINE — ``LLM`` / ``LLMEngine`` / ``ModelRunner`` / scheduler /
CUDA-graph capture / attention, unmodified, from the mirror ``oracle/build_ref.py`` keeps in
``oracle/_ref`` — over a random-initialised Qwen3-architecture model, either with the
reference's own quantized linears (its CUDA extensions, prebuilt for sm_100a by the same
recipe) or with THIS package's layers installed under the reference's module names
(``tiny_vllm_b200.integration.install_under_nanovllm``).  Test infrastructure: the engine is the
harness, the linear layers are what differs between the two arms.

What it exercises of the drop-in contract (``nanovllm/engine/model_runner.py:18-60,216-251,
298-335``, ``nanovllm/utils/loader.py:44-68``): the model is built from the layer classes by
``nanovllm/models/qwen3.py``, filled by the reference's ``load_model`` from the quantized
artifact, warmed up at ``max_num_batched_tokens``, and one CUDA graph per decode batch size of
the runner's list (1, 2, 4, 8, 16, 32 ... 512) is captured and replayed; prefill runs eagerly.

Sub-commands:
  make   --dir D [--layers L ...]     writes D/hf (config, tokenizer stub, random bf16 weights)
                                      and D/int8, D/w8a8 (artifacts, ``utils/quantize_artifact``)
  run    --dir D --mode bf16|int8|w8a8 --impl reference|ours [--tp N] [--seqs ...]   prints one JSON line

The workload is the reference's own throughput benchmark in miniature (random token ids, fixed
output length with ``ignore_eos``, ``bench_quant.py:166-190``); the tokens-per-second
definitions are the engine's (``llm_engine.py:151-162``).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF_DIR = ROOT / "oracle" / "_ref"

QWEN3_06B = dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=128, vocab_size=151936)
QWEN3_8B = dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, vocab_size=151936)


def make(args) -> None:
    """Random-initialised checkpoint with Hugging Face names + tokenizer stub + both artifacts."""
    import torch
    from safetensors.torch import save_file
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    sys.path.insert(0, str(ROOT))
    import tiny_vllm_b200  # noqa: F401
    from tiny_vllm_b200.utils import quantize_artifact as QA

    arch = dict(QWEN3_8B if args.arch == "8b" else QWEN3_06B)
    if args.layers:
        arch["num_hidden_layers"] = args.layers
    if args.vocab:
        arch["vocab_size"] = args.vocab
    root = Path(args.dir)
    hf = root / "hf"
    hf.mkdir(parents=True, exist_ok=True)
    config = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
              "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000,
              "tie_word_embeddings": True, "torch_dtype": "bfloat16", "dtype": "bfloat16",
              "attention_bias": False, **arch}
    (hf / "config.json").write_text(json.dumps(config, indent=1))
    vocab = {f"t{i}": i for i in range(arch["vocab_size"] - 1)}
    vocab["<eos>"] = arch["vocab_size"] - 1
    tok = Tokenizer(WordLevel(vocab, unk_token="t0"))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(hf / "tokenizer.json"))
    (hf / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<eos>", "unk_token": "t0",
         "model_max_length": 40960}))

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator(device=dev).manual_seed(0)
    H, I = arch["hidden_size"], arch["intermediate_size"]
    q_rows, kv_rows = arch["num_attention_heads"] * arch["head_dim"], arch["num_key_value_heads"] * arch["head_dim"]

    def w(*shape, std=0.02):
        return (torch.randn(*shape, generator=g, device=dev) * std).to(torch.bfloat16).cpu()

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16)

    shard, index, part = {}, 0, 0

    def flush():
        nonlocal shard, part
        if shard:
            save_file(shard, str(hf / f"model-{part:05d}.safetensors"))
            part += 1
            shard = {}

    shard["model.embed_tokens.weight"] = w(arch["vocab_size"], H)
    shard["model.norm.weight"] = ones(H)
    for i in range(arch["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shard[p + "self_attn.q_proj.weight"] = w(q_rows, H)
        shard[p + "self_attn.k_proj.weight"] = w(kv_rows, H)
        shard[p + "self_attn.v_proj.weight"] = w(kv_rows, H)
        shard[p + "self_attn.o_proj.weight"] = w(H, q_rows)
        shard[p + "self_attn.q_norm.weight"] = ones(arch["head_dim"])
        shard[p + "self_attn.k_norm.weight"] = ones(arch["head_dim"])
        shard[p + "mlp.gate_proj.weight"] = w(I, H)
        shard[p + "mlp.up_proj.weight"] = w(I, H)
        shard[p + "mlp.down_proj.weight"] = w(H, I)
        shard[p + "input_layernorm.weight"] = ones(H)
        shard[p + "post_attention_layernorm.weight"] = ones(H)
        index += 1
        if index % 4 == 0:      # a few layers per file: the whole model is never held at once
            flush()
    flush()
    for mode in ("int8", "w8a8"):
        QA.quantize_directory(hf, root / mode, mode, device=dev if dev == "cuda" else None)
    print(json.dumps({"made": str(root), "arch": arch}))


def _install(impl: str, quantized: bool) -> None:
    """Makes ``import nanovllm`` resolve to the mirror, with this package's layers under the
    reference's module names (``ours``) or with the reference's prebuilt CUDA extensions
    (``reference``).  Runs in the parent and again in every spawned tensor-parallel worker."""
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    if impl == "ours":
        import tiny_vllm_b200  # noqa: F401
        from tiny_vllm_b200 import integration
        if "nanovllm.layers.linear" not in sys.modules:
            integration.install_under_nanovllm()
        if str(REF_DIR) not in sys.path:
            sys.path.insert(0, str(REF_DIR))
    else:
        from oracle import build_ref
        ref = build_ref.load_reference(with_cuda_extensions=quantized)
        if quantized and not (ref.native_w8a16 and ref.native_w8a8):
            raise SystemExit("the reference's CUDA extensions are not in oracle/_ref/ext")


if __name__ == "__mp_main__":
    # A spawned tensor-parallel worker imports this file first and only then unpickles the
    # engine's arguments, which imports ``nanovllm``: the aliases must be in place by then.
    import os as _os
    if "ENGINE_HARNESS_IMPL" in _os.environ:
        _install(_os.environ["ENGINE_HARNESS_IMPL"], _os.environ["ENGINE_HARNESS_QUANTIZED"] == "1")


def _runner_entry(config, rank, event):
    """Stands in for ``ModelRunner`` in ``nanovllm/engine/llm_engine.py:27-33``: the engine
    spawns its tensor-parallel workers with this function as the process target (a spawned
    child imports ``nanovllm`` afresh, so the module aliases have to be installed there too)
    and calls it directly for rank 0."""
    import os
    _install(os.environ["ENGINE_HARNESS_IMPL"], os.environ["ENGINE_HARNESS_QUANTIZED"] == "1")
    from nanovllm.engine.model_runner import ModelRunner
    if os.environ.get("ENGINE_HARNESS_PEER") != "1":
        return ModelRunner(config, rank, event)

    class PeerRunner(ModelRunner):
        """Installs this package's peer-memory communicator (fused decode GEMM + all-reduce,
        one-trip / two-shot all-reduce kernels) once the process group exists and before the
        first forward pass; everything else is the reference's runner."""

        def warmup_model(self):
            from tiny_vllm_b200.layers import linear as our_linear
            from tiny_vllm_b200.layers.tp_comm import PeerAllReduce
            hidden = self.config.hf_config.hidden_size
            our_linear.set_tp_all_reduce(PeerAllReduce(max_bytes=self.config.max_num_batched_tokens * hidden * 2))
            super().warmup_model()

    return PeerRunner(config, rank, event)


def run(args) -> None:
    import os

    import torch

    if not (REF_DIR / "nanovllm" / "engine" / "llm_engine.py").is_file():
        raise SystemExit("oracle/_ref holds no mirror of the reference (run oracle/build_ref.py)")
    ours = args.impl == "ours"
    os.environ["ENGINE_HARNESS_IMPL"] = args.impl          # read by the spawned workers
    os.environ["ENGINE_HARNESS_QUANTIZED"] = "1" if args.mode != "bf16" else "0"
    os.environ["ENGINE_HARNESS_PEER"] = "1" if (args.peer and ours and args.tp > 1) else "0"
    _install(args.impl, args.mode != "bf16")
    if ours:
        from tiny_vllm_b200 import _lib
    from nanovllm import LLM, SamplingParams      # the reference's engine, unmodified
    import nanovllm.engine.llm_engine as engine_mod
    import nanovllm.engine.model_runner as runner_mod
    assert Path(runner_mod.__file__).resolve().is_relative_to(REF_DIR.resolve())
    if args.tp > 1:
        engine_mod.ModelRunner = _runner_entry

    root = Path(args.dir)
    kw = dict(enforce_eager=args.eager, max_model_len=args.max_model_len, tensor_parallel_size=args.tp,
              max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens)
    if args.mode != "bf16":
        kw.update(quantization=args.mode, quantized_model_path=str(root / args.mode))
    t0 = time.perf_counter()
    llm = LLM(str(root / "hf"), **kw)
    init_s = time.perf_counter() - t0
    model = llm.model_runner.model
    layer0 = model.model.layers[0]
    linear_module = type(layer0.mlp.down_proj).__module__
    if ours:
        assert linear_module.startswith("tiny_vllm_b200"), linear_module
        assert layer0.self_attn.qkv_proj.quant_method is None or \
            type(layer0.self_attn.qkv_proj.quant_method).__module__.startswith("tiny_vllm_b200")
        launches0 = _lib.lib().b200q_launch_count()
    else:
        assert linear_module.startswith("nanovllm"), linear_module

    g = torch.Generator().manual_seed(1)
    vocab = model.model.embed_tokens.weight.shape[0]

    def prompts(n):
        lens = torch.randint(args.in_min, args.in_max + 1, (n,), generator=g).tolist()
        return [torch.randint(0, vocab - 1, (k,), generator=g).tolist() for k in lens]

    sp = SamplingParams(temperature=0.6, max_tokens=args.out, ignore_eos=True)
    llm.generate_with_stats(prompts(min(16, args.seqs)), SamplingParams(temperature=0.6, max_tokens=8, ignore_eos=True))
    outputs, stats = llm.generate_with_stats(prompts(args.seqs), sp)
    torch.cuda.synchronize()
    ok = len(outputs) == args.seqs and all(len(o["token_ids"]) == args.out for o in outputs)
    line = {"impl": args.impl, "mode": args.mode, "tp": args.tp, "peer_allreduce": bool(args.peer and ours and args.tp > 1),
            "ok": ok, "linear_module": linear_module,
            "graphs": 0 if args.eager else len(getattr(llm.model_runner, "graphs", {})),
            "graph_batch_sizes": None if args.eager else sorted(getattr(llm.model_runner, "graph_bs", [])),
            "init_seconds": round(init_s, 1), "seqs": args.seqs, "in": [args.in_min, args.in_max], "out": args.out,
            "prefill_tokens_per_second": round(stats["prefill_tokens_per_second"], 1),
            "decode_tokens_per_second": round(stats["decode_tokens_per_second"], 1),
            "prefill_tokens": stats["prefill_tokens"], "decode_tokens": stats["decode_tokens"],
            "wall_seconds": round(stats["wall_time_seconds"], 2),
            "after_load_gib": round(llm.model_runner.memory_snapshots["after_model_load"]["memory_allocated"] / 2**30, 2)}
    if ours:
        line["b200q_launches"] = int(_lib.lib().b200q_launch_count() - launches0)
        line["device_status"] = int(_lib.lib().b200q_device_status())
        ok = ok and line["b200q_launches"] > 0 and line["device_status"] == 0
        line["ok"] = ok
    print("ENGINE " + json.dumps(line), flush=True)
    llm.exit()
    if not ok:
        raise SystemExit(1)


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    m = sub.add_parser("make")
    m.add_argument("--dir", required=True)
    m.add_argument("--arch", default="0.6b", choices=["0.6b", "8b"])
    m.add_argument("--layers", type=int, default=0)
    m.add_argument("--vocab", type=int, default=0)
    r = sub.add_parser("run")
    r.add_argument("--dir", required=True)
    r.add_argument("--mode", default="w8a8", choices=["bf16", "int8", "w8a8"])
    r.add_argument("--impl", default="ours", choices=["reference", "ours"])
    r.add_argument("--seqs", type=int, default=64)
    r.add_argument("--in-min", type=int, default=16)
    r.add_argument("--in-max", type=int, default=128)
    r.add_argument("--out", type=int, default=32)
    r.add_argument("--max-model-len", type=int, default=2048)
    r.add_argument("--max-num-seqs", type=int, default=512)
    r.add_argument("--max-num-batched-tokens", type=int, default=16384)
    r.add_argument("--eager", action="store_true")
    r.add_argument("--peer", action="store_true",
                   help="with --impl ours --tp N: this package's peer-memory all-reduce instead of NCCL")
    r.add_argument("--tp", type=int, default=1, help="tensor-parallel ranks (the engine spawns tp - 1 workers)")
    args = ap.parse_args()
    make(args) if args.cmd == "make" else run(args)


if __name__ == "__main__":
    main()

"""Drop-in proof under the REFERENCE'S OWN model code, two CPU ranks over gloo.

In every rank ``tiny_vllm_b200.integration.install_under_nanovllm()`` puts this package's
``layers.linear`` and ``quantization`` in place of the reference's modules; then the reference's
unmodified ``Qwen3ForCausalLM`` (``nanovllm/models/qwen3.py:195-224``) is built from a toy
two-layer config — which constructs our ``QKVParallelLinear`` / ``MergedColumnParallelLinear`` /
``RowParallelLinear`` with the arguments of ``qwen3.py:43-56,103-114`` — and is loaded with the
reference's unmodified ``load_model`` (``nanovllm/utils/loader.py:44-68``) from

* an artifact written by the reference's own ``scripts/quantize.py:93-139``, and
* an artifact written by ``tiny_vllm_b200.utils.quantize_artifact``,

and with this package's loader (sharded reads) from the first.  Every parameter must be equal
across the three, the two artifacts must be identical tensor for tensor, and each rank's
``qweight`` / scale shards must be exactly the rows / columns the sharding rules of
``nanovllm/layers/linear.py:101-113,139-171,209-244,259-267`` give.

Needs the reference's Python sources: the mirror ``oracle/build_ref.py`` keeps under
``oracle/_ref`` (or a checkout named by NANOVLLM_REFERENCE); skipped when neither exists.
"""
import importlib.util
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
HIDDEN, LAYERS, HEADS, KV_HEADS, HEAD_DIM, INTER, VOCAB = 64, 2, 4, 2, 16, 96, 128


def reference_dir():
    for cand in (os.environ.get("NANOVLLM_REFERENCE"), str(ROOT / "oracle" / "_ref"), "/root/reference"):
        if cand and (Path(cand) / "nanovllm" / "models" / "qwen3.py").is_file() \
                and (Path(cand) / "scripts" / "quantize.py").is_file():
            return cand
    return None


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def hf_checkpoint(seed=0):
    """Tensors named like a Hugging Face Qwen3 checkpoint, 16 bit."""
    g = torch.Generator().manual_seed(seed)

    def w(*shape):
        return (torch.randn(*shape, generator=g) * 0.05).to(torch.bfloat16)

    t = {"model.embed_tokens.weight": w(VOCAB, HIDDEN), "model.norm.weight": w(HIDDEN) + 1,
         "lm_head.weight": w(VOCAB, HIDDEN)}
    for i in range(LAYERS):
        p = f"model.layers.{i}."
        t[p + "self_attn.q_proj.weight"] = w(HEADS * HEAD_DIM, HIDDEN)
        t[p + "self_attn.k_proj.weight"] = w(KV_HEADS * HEAD_DIM, HIDDEN)
        t[p + "self_attn.v_proj.weight"] = w(KV_HEADS * HEAD_DIM, HIDDEN)
        t[p + "self_attn.o_proj.weight"] = w(HIDDEN, HEADS * HEAD_DIM)
        t[p + "self_attn.q_norm.weight"] = w(HEAD_DIM) + 1
        t[p + "self_attn.k_norm.weight"] = w(HEAD_DIM) + 1
        t[p + "mlp.gate_proj.weight"] = w(INTER, HIDDEN)
        t[p + "mlp.up_proj.weight"] = w(INTER, HIDDEN)
        t[p + "mlp.down_proj.weight"] = w(HIDDEN, INTER)
        t[p + "input_layernorm.weight"] = w(HIDDEN) + 1
        t[p + "post_attention_layernorm.weight"] = w(HIDDEN) + 1
    return t


def _worker(rank, world, port, ref_dir, work_dir, mode):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    notes, ok = [], True
    try:
        import tiny_vllm_b200  # noqa: F401
        from tiny_vllm_b200 import integration
        from tiny_vllm_b200.layers import linear as our_linear
        from tiny_vllm_b200.utils import quantize_artifact as QA
        from tiny_vllm_b200.utils.loader import load_model as our_load_model
        integration.install_under_nanovllm()
        sys.path.insert(0, ref_dir)
        from safetensors.torch import load_file, save_file
        from transformers import Qwen3Config
        from nanovllm.models.qwen3 import Qwen3ForCausalLM          # the reference's model code
        from nanovllm.utils.loader import load_model as ref_load_model  # and its loader
        import nanovllm.layers.linear as seen_linear
        assert seen_linear is our_linear
        assert Path(sys.modules["nanovllm.models.qwen3"].__file__).is_relative_to(ref_dir)

        work = Path(work_dir)
        if rank == 0:
            (work / "hf").mkdir()
            save_file(hf_checkpoint(), work / "hf" / "model.safetensors")
            (work / "hf" / "config.json").write_text("{}")
            # the reference's own artifact tool, imported from its file
            spec = importlib.util.spec_from_file_location("ref_quantize", Path(ref_dir) / "scripts" / "quantize.py")
            ref_tool = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(ref_tool)
            (work / "by_reference").mkdir()
            tensors = ref_tool.load_tensors(work / "hf")
            save_file(ref_tool.build_quantized_tensors(tensors, mode), work / "by_reference" / "model.safetensors")
            QA.quantize_directory(work / "hf", work / "by_ours", mode)
        dist.barrier()
        art_ref = load_file(work / "by_reference" / "model.safetensors")
        art_ours = load_file(work / "by_ours" / "model.safetensors")
        ok = ok and set(art_ref) == set(art_ours)
        for k in art_ref:
            if not torch.equal(art_ref[k], art_ours[k]):
                ok = False
                notes.append(f"artifacts differ at {k}")

        config = Qwen3Config(hidden_size=HIDDEN, num_hidden_layers=LAYERS, num_attention_heads=HEADS,
                             num_key_value_heads=KV_HEADS, head_dim=HEAD_DIM, intermediate_size=INTER,
                             vocab_size=VOCAB, max_position_embeddings=256, tie_word_embeddings=False)
        config.nanovllm_quantization = mode
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            models = [Qwen3ForCausalLM(config) for _ in range(3)]
        finally:
            torch.set_default_dtype(prev)
        ref_load_model(models[0], str(work / "by_reference"), mode)
        ref_load_model(models[1], str(work / "by_ours"), mode)
        stats = our_load_model(models[2], str(work / "by_reference"), mode)
        layer0 = models[0].model.layers[0]
        ok = ok and isinstance(layer0.self_attn.qkv_proj, our_linear.QKVParallelLinear) \
            and isinstance(layer0.self_attn.o_proj, our_linear.RowParallelLinear) \
            and isinstance(layer0.mlp.gate_up_proj, our_linear.MergedColumnParallelLinear) \
            and layer0.self_attn.qkv_proj.tp_size == world and layer0.self_attn.qkv_proj.tp_rank == rank
        names = [n for n, _ in models[0].named_parameters()]
        for other in models[1:]:
            for (na, pa), (nb, pb) in zip(models[0].named_parameters(), other.named_parameters()):
                if na != nb or not torch.equal(pa.data, pb.data):
                    ok = False
                    notes.append(f"parameter {na} differs between loads")
        # the shards themselves, from the sharding rules
        scale = "w_scales" if mode == "w8a8" else "scales"
        for i in range(LAYERS):
            p = f"model.layers.{i}."
            full = art_ref[p + "self_attn.qkv_proj.qweight"]
            q_rows, kv_rows = HEADS * HEAD_DIM, KV_HEADS * HEAD_DIM
            want = torch.cat([full[:q_rows].chunk(world)[rank],
                              full[q_rows:q_rows + kv_rows].chunk(world)[rank],
                              full[q_rows + kv_rows:].chunk(world)[rank]])
            lay = models[0].model.layers[i]
            checks = [
                (lay.self_attn.qkv_proj.qweight, want),
                (lay.self_attn.o_proj.qweight, art_ref[p + "self_attn.o_proj.qweight"].chunk(world, dim=1)[rank]),
                (getattr(lay.self_attn.o_proj, scale), art_ref[p + f"self_attn.o_proj.{scale}"]),
                (lay.mlp.gate_up_proj.qweight,
                 torch.cat([art_ref[p + "mlp.gate_up_proj.qweight"][:INTER].chunk(world)[rank],
                            art_ref[p + "mlp.gate_up_proj.qweight"][INTER:].chunk(world)[rank]])),
                (getattr(lay.mlp.gate_up_proj, scale),
                 torch.cat([art_ref[p + f"mlp.gate_up_proj.{scale}"][:INTER].chunk(world)[rank],
                            art_ref[p + f"mlp.gate_up_proj.{scale}"][INTER:].chunk(world)[rank]])),
                (lay.mlp.down_proj.qweight, art_ref[p + "mlp.down_proj.qweight"].chunk(world, dim=1)[rank]),
            ]
            for param, expect in checks:
                if not torch.equal(param.data, expect):
                    ok = False
                    notes.append(f"layer {i}: a shard is not what the sharding rules give")
        notes.append(f"{len(names)} parameters, sharded loader read {stats['bytes_read']} bytes")
    except Exception:  # noqa: BLE001
        import traceback
        ok = False
        notes.append(traceback.format_exc())
    torch.save({"ok": ok, "notes": notes}, os.path.join(work_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["w8a8", "int8"])
def test_reference_model_builds_and_loads_over_these_layers(tmp_path, mode):
    ref_dir = reference_dir()
    if ref_dir is None:
        pytest.skip("the reference's Python sources are not available (oracle/_ref was never built)")
    mp.spawn(_worker, args=(2, _free_port(), ref_dir, str(tmp_path), mode), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"r{r}.pt")
        print(r, res["notes"])
        assert res["ok"], res["notes"]

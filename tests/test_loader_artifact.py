"""Quantized-artifact layout and loader contract, on CPU with a toy Qwen3-shaped model."""
import pytest
import torch
from safetensors.torch import load_file, save_file
from torch import nn

import tiny_vllm_b200  # noqa: F401
from oracle import quant_linear_oracle as O
from tiny_vllm_b200.layers import linear as L
from tiny_vllm_b200.utils import quantize_artifact as QA
from tiny_vllm_b200.utils.loader import load_model

HIDDEN, HD, NH, NKV, INTER = 32, 8, 4, 2, 48


class Attn(nn.Module):
    def __init__(self, quant):
        super().__init__()
        self.qkv_proj = L.QKVParallelLinear(HIDDEN, HD, NH, NKV, quantization=quant)
        self.o_proj = L.RowParallelLinear(NH * HD, HIDDEN, quantization=quant)


class Mlp(nn.Module):
    def __init__(self, quant):
        super().__init__()
        self.gate_up_proj = L.MergedColumnParallelLinear(HIDDEN, [INTER, INTER], quantization=quant)
        self.down_proj = L.RowParallelLinear(INTER, HIDDEN, quantization=quant)


class Layer(nn.Module):
    def __init__(self, quant):
        super().__init__()
        self.self_attn = Attn(quant)
        self.mlp = Mlp(quant)
        self.input_layernorm = nn.LayerNorm(HIDDEN, bias=False)


class Toy(nn.Module):
    # same mapping as the reference model (nanovllm/models/qwen3.py:195-201)
    packed_modules_mapping = {
        "q_proj": ("qkv_proj", "q"), "k_proj": ("qkv_proj", "k"), "v_proj": ("qkv_proj", "v"),
        "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1),
    }

    def __init__(self, quant=None, n_layers=2):
        super().__init__()
        self.layers = nn.ModuleList(Layer(quant) for _ in range(n_layers))


def hf_tensors(n_layers=2, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = {}
    for i in range(n_layers):
        p = f"layers.{i}."
        t[p + "self_attn.q_proj.weight"] = torch.randn(NH * HD, HIDDEN, generator=g) * 0.02
        t[p + "self_attn.k_proj.weight"] = torch.randn(NKV * HD, HIDDEN, generator=g) * 0.02
        t[p + "self_attn.v_proj.weight"] = torch.randn(NKV * HD, HIDDEN, generator=g) * 0.02
        t[p + "self_attn.o_proj.weight"] = torch.randn(HIDDEN, NH * HD, generator=g) * 0.02
        t[p + "mlp.gate_proj.weight"] = torch.randn(INTER, HIDDEN, generator=g) * 0.02
        t[p + "mlp.up_proj.weight"] = torch.randn(INTER, HIDDEN, generator=g) * 0.02
        t[p + "mlp.down_proj.weight"] = torch.randn(HIDDEN, INTER, generator=g) * 0.02
        t[p + "input_layernorm.weight"] = torch.rand(HIDDEN, generator=g)
    return t


@pytest.fixture
def tp(monkeypatch):
    def set_tp(rank, size):
        monkeypatch.setattr(L, "_tp_coordinates", lambda: (rank, size))
    return set_tp


@pytest.mark.parametrize("mode,scale", [("int8", "scales"), ("w8a8", "w_scales")])
def test_artifact_layout(tmp_path, mode, scale):
    src = tmp_path / "hf"
    src.mkdir()
    tensors = hf_tensors()
    save_file(tensors, src / "model.safetensors")
    (src / "config.json").write_text("{}")
    out = tmp_path / "q"
    QA.quantize_directory(src, out, mode)
    assert (out / "config.json").exists()
    art = load_file(out / "model.safetensors")
    for i in range(2):
        p = f"layers.{i}."
        for stem, rows in ((p + "self_attn.qkv_proj", (NH + 2 * NKV) * HD), (p + "self_attn.o_proj", HIDDEN),
                           (p + "mlp.gate_up_proj", 2 * INTER), (p + "mlp.down_proj", HIDDEN)):
            assert art[stem + ".qweight"].dtype == torch.int8 and art[stem + ".qweight"].shape[0] == rows
            assert art[stem + "." + scale].dtype == torch.float32 and art[stem + "." + scale].shape == (rows,)
        packed = torch.cat([tensors[p + f"self_attn.{n}_proj.weight"] for n in "qkv"])
        q, s = O.quantize_per_channel(packed)       # oracle quantiser on the packed matrix
        assert torch.equal(art[p + "self_attn.qkv_proj.qweight"], q)
        assert torch.equal(art[p + "self_attn.qkv_proj." + scale], s)
        assert torch.equal(art[p + "input_layernorm.weight"], tensors[p + "input_layernorm.weight"])
        assert p + "self_attn.q_proj.weight" not in art and p + "mlp.up_proj.weight" not in art
    other = "w_scales" if scale == "scales" else "scales"
    assert not any(k.endswith("." + other) for k in art)


def test_artifact_requires_complete_groups():
    t = hf_tensors(1)
    del t["layers.0.self_attn.k_proj.weight"]
    with pytest.raises(ValueError):
        QA.build_quantized_tensors(t, "int8")


@pytest.mark.parametrize("size", [1, 2])
def test_load_plain_and_quantized(tmp_path, tp, size):
    src = tmp_path / "hf"
    src.mkdir()
    tensors = hf_tensors()
    save_file(tensors, src / "model.safetensors")
    out = tmp_path / "q"
    QA.quantize_directory(src, out, "w8a8")
    art = load_file(out / "model.safetensors")
    for rank in range(size):
        tp(rank, size)
        plain = Toy(None)
        load_model(plain, str(src))
        w = plain.layers[1].self_attn.qkv_proj.weight.data
        exp = torch.cat([tensors[f"layers.1.self_attn.{n}_proj.weight"].chunk(size)[rank] for n in "qkv"])
        assert torch.equal(w, exp)

        qm = Toy("w8a8")
        load_model(qm, str(out), "w8a8")
        full = art["layers.0.mlp.gate_up_proj.qweight"]
        exp = torch.cat([full[:INTER].chunk(size)[rank], full[INTER:].chunk(size)[rank]])
        assert torch.equal(qm.layers[0].mlp.gate_up_proj.qweight.data, exp)
        assert torch.equal(qm.layers[0].mlp.down_proj.qweight.data,
                           art["layers.0.mlp.down_proj.qweight"].chunk(size, dim=1)[rank])
        assert torch.equal(qm.layers[0].mlp.down_proj.w_scales.data, art["layers.0.mlp.down_proj.w_scales"])


def test_loader_errors(tmp_path, tp):
    tp(0, 1)
    with pytest.raises(FileNotFoundError):
        load_model(Toy(None), str(tmp_path))
    # an int8 artifact cannot satisfy a w8a8 model: the w_scales are missing
    src = tmp_path / "hf"
    src.mkdir()
    save_file(hf_tensors(), src / "model.safetensors")
    out = tmp_path / "q8"
    QA.quantize_directory(src, out, "int8")
    art = load_file(out / "model.safetensors")
    art = {k: v for k, v in art.items() if not k.endswith(".scales")}
    bad = tmp_path / "bad"
    bad.mkdir()
    save_file(art, bad / "model.safetensors")
    with pytest.raises(RuntimeError, match="Missing INT8 quantized tensors"):
        load_model(Toy("int8"), str(bad), "int8")


@pytest.mark.parametrize("size", [1, 2, 4, 8])
@pytest.mark.parametrize("mode", [None, "int8", "w8a8"])
def test_sharded_reads_equal_whole_tensor_loads(tmp_path, tp, size, mode):
    # every rank of every group size: parameters filled from slices of the stored tensors equal
    # those filled by the reference-style weight_loader hooks, and only this rank's share of the
    # column- / row-split matrices is read
    src = tmp_path / "hf"
    src.mkdir()
    tensors = hf_tensors()
    if size > 2:        # the toy model has 2 KV heads: give it 8 so that they split 8 ways
        g = torch.Generator().manual_seed(5)
        for i in range(2):
            for n in "kv":
                tensors[f"layers.{i}.self_attn.{n}_proj.weight"] = torch.randn(8 * HD, HIDDEN, generator=g) * 0.02
            tensors[f"layers.{i}.self_attn.q_proj.weight"] = torch.randn(8 * HD, HIDDEN, generator=g) * 0.02
            tensors[f"layers.{i}.self_attn.o_proj.weight"] = torch.randn(HIDDEN, 8 * HD, generator=g) * 0.02
    save_file(tensors, src / "model.safetensors")
    path = src
    if mode is not None:
        path = tmp_path / "q"
        QA.quantize_directory(src, path, mode)

    heads, kv_heads = (8, 8) if size > 2 else (NH, NKV)

    class WideAttn(nn.Module):
        def __init__(self, quant):
            super().__init__()
            self.qkv_proj = L.QKVParallelLinear(HIDDEN, HD, heads, kv_heads, quantization=quant)
            self.o_proj = L.RowParallelLinear(heads * HD, HIDDEN, quantization=quant)

    class WideLayer(nn.Module):
        def __init__(self, quant):
            super().__init__()
            self.self_attn = WideAttn(quant)
            self.mlp = Mlp(quant)
            self.input_layernorm = nn.LayerNorm(HIDDEN, bias=False)

    class Wide(Toy):
        def __init__(self, quant):
            nn.Module.__init__(self)
            self.layers = nn.ModuleList(WideLayer(quant) for _ in range(2))

    whole_bytes = None
    for rank in range(size):
        tp(rank, size)
        a, b = Wide(mode), Wide(mode)
        sa = load_model(a, str(path), mode)                          # sliced reads
        sb = load_model(b, str(path), mode, sharded_reads=False)     # whole tensors + weight_loader
        for (na, pa), (nb, pb) in zip(a.named_parameters(), b.named_parameters()):
            assert na == nb and torch.equal(pa.data, pb.data), (rank, na)
        whole_bytes = sb["bytes_read"]
        assert sa["bytes_read"] <= sb["bytes_read"]
        if size > 1:
            # the split matrices dominate the toy checkpoint: close to 1 / size of the bytes
            assert sa["bytes_read"] < sb["bytes_read"] * (1.0 / size + 0.15), (sa, sb)
    assert whole_bytes > 0


def test_streaming_artifact_writes_shards_and_matches_in_memory_builder(tmp_path, tp):
    tp(0, 1)
    src = tmp_path / "hf"
    src.mkdir()
    tensors = hf_tensors()
    # source split over two shard files, members of one packed projection in different files
    names = sorted(tensors)
    save_file({n: tensors[n] for n in names[::2]}, src / "model-00001-of-00002.safetensors")
    save_file({n: tensors[n] for n in names[1::2]}, src / "model-00002-of-00002.safetensors")
    out = tmp_path / "q"
    files = QA.quantize_directory(src, out, "w8a8", shard_bytes=4096)   # tiny shards: several files
    assert len(files) > 1 and all(f.name.startswith("model-") for f in files)
    merged = {}
    for f in files:
        part = load_file(f)
        assert not set(part) & set(merged)
        merged.update(part)
    want = QA.build_quantized_tensors(tensors, "w8a8")
    assert set(merged) == set(want)
    for k in want:
        assert torch.equal(merged[k], want[k]), k
    model = Toy("w8a8")
    load_model(model, str(out), "w8a8")                                 # the loader reads every shard
    assert torch.equal(model.layers[1].mlp.down_proj.qweight.data, want["layers.1.mlp.down_proj.qweight"])
    # duplicate names across source shards are refused
    save_file({names[0]: tensors[names[0]]}, src / "model-00003-of-00003.safetensors")
    with pytest.raises(ValueError, match="Duplicate tensor name"):
        QA.quantize_directory(src, tmp_path / "q2", "w8a8")

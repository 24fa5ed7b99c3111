"""Host logic of the tensor-parallel linear layers, on CPU: constructor contract,
per-rank shard loaders for tp in {1,2,4,8}, unquantized forward, bias choice.
The expected shards are recomputed here by plain slicing of the full matrices."""
import pytest
import torch
from torch import nn

import tiny_vllm_b200  # noqa: F401
from tiny_vllm_b200.layers import linear as L
from tiny_vllm_b200.quantization import Int8WeightOnlyQuantMethod, QuantMethod, W8A8QuantMethod


@pytest.fixture
def tp(monkeypatch):
    def set_tp(rank, size):
        monkeypatch.setattr(L, "_tp_coordinates", lambda: (rank, size))
    return set_tp


def chunk(t, size, rank, dim=0):
    return t.chunk(size, dim)[rank]


def test_rejects_unknown_quantization(tp):
    tp(0, 1)
    with pytest.raises(NotImplementedError):
        L.ReplicatedLinear(16, 16, quantization="int4_awq")


@pytest.mark.parametrize("quant,scale_name,cls", [("int8", "scales", Int8WeightOnlyQuantMethod),
                                                   ("w8a8", "w_scales", W8A8QuantMethod)])
def test_parameter_registration(tp, quant, scale_name, cls):
    tp(0, 1)
    layer = L.ColumnParallelLinear(64, 32, bias=True, quantization=quant)
    assert isinstance(layer.quant_method, cls) and isinstance(layer.quant_method, QuantMethod)
    names = dict(layer.named_parameters())
    assert set(names) == {"qweight", scale_name, "bias"}
    assert names["qweight"].dtype == torch.int8 and names["qweight"].shape == (32, 64)
    assert names[scale_name].dtype == torch.float32 and names[scale_name].shape == (32,)
    assert not names["qweight"].requires_grad
    for p in names.values():
        assert callable(p.weight_loader)
    plain = L.ColumnParallelLinear(64, 32)
    assert set(dict(plain.named_parameters())) == {"weight"} and plain.bias is None
    assert plain.quant_method is None


@pytest.mark.parametrize("size", [1, 2, 4, 8])
def test_column_and_row_loaders(tp, size):
    full_w = torch.arange(64 * 32, dtype=torch.float32).view(64, 32)
    full_q = torch.randint(-127, 128, (64, 32), dtype=torch.int8)
    full_s = torch.rand(64)
    for rank in range(size):
        tp(rank, size)
        col = L.ColumnParallelLinear(32, 64, bias=True)
        assert (col.tp_rank, col.tp_size, col.tp_dim) == (rank, size, 0)
        col.weight.weight_loader(col.weight, full_w)
        assert torch.equal(col.weight.data, chunk(full_w, size, rank))
        col.bias.weight_loader(col.bias, full_s)
        assert torch.equal(col.bias.data, chunk(full_s, size, rank))
        colq = L.ColumnParallelLinear(32, 64, quantization="int8")
        colq.qweight.weight_loader(colq.qweight, full_q)
        colq.scales.weight_loader(colq.scales, full_s)
        assert torch.equal(colq.qweight.data, chunk(full_q, size, rank))
        assert torch.equal(colq.scales.data, chunk(full_s, size, rank))

        row = L.RowParallelLinear(32, 64, quantization="w8a8")
        assert row.tp_dim == 1 and row.qweight.shape == (64, 32 // size)
        row.qweight.weight_loader(row.qweight, full_q)
        row.w_scales.weight_loader(row.w_scales, full_s)
        assert torch.equal(row.qweight.data, chunk(full_q, size, rank, dim=1))
        assert torch.equal(row.w_scales.data, full_s)  # replicated


@pytest.mark.parametrize("size", [1, 2, 4, 8])
def test_merged_column_loaders(tp, size):
    sizes = [48, 48]
    K = 16
    gate = torch.randn(48, K)
    up = torch.randn(48, K)
    packed_q = torch.randint(-127, 128, (96, K), dtype=torch.int8)
    packed_s = torch.rand(96)
    for rank in range(size):
        tp(rank, size)
        m = L.MergedColumnParallelLinear(K, sizes, bias=True)
        assert m.output_sizes == sizes and m.weight.shape == (96 // size, K)
        m.weight.weight_loader(m.weight, gate, 0)
        m.weight.weight_loader(m.weight, up, 1)
        expect = torch.cat([chunk(gate, size, rank), chunk(up, size, rank)])
        assert torch.equal(m.weight.data, expect)
        # packed bias (no shard id) and per-shard bias
        m.bias.weight_loader(m.bias, packed_s)
        eb = torch.cat([chunk(packed_s[:48], size, rank), chunk(packed_s[48:], size, rank)])
        assert torch.equal(m.bias.data, eb)
        m.bias.weight_loader(m.bias, packed_s[48:], 1)
        assert torch.equal(m.bias.data[48 // size:], chunk(packed_s[48:], size, rank))

        mq = L.MergedColumnParallelLinear(K, sizes, quantization="w8a8")
        mq.qweight.weight_loader(mq.qweight, packed_q)
        mq.w_scales.weight_loader(mq.w_scales, packed_s)
        eq = torch.cat([chunk(packed_q[:48], size, rank), chunk(packed_q[48:], size, rank)])
        assert torch.equal(mq.qweight.data, eq)
        assert torch.equal(mq.w_scales.data, eb)


@pytest.mark.parametrize("size", [1, 2, 4, 8])
def test_qkv_loaders(tp, size):
    hidden, hd, nh, nkv = 32, 8, 16, 8
    q = torch.randn(nh * hd, hidden)
    k = torch.randn(nkv * hd, hidden)
    v = torch.randn(nkv * hd, hidden)
    packed = torch.cat([q, k, v])
    packed_q = torch.randint(-127, 128, packed.shape, dtype=torch.int8)
    packed_s = torch.rand(packed.shape[0])
    for rank in range(size):
        tp(rank, size)
        layer = L.QKVParallelLinear(hidden, hd, nh, nkv)
        assert (layer.num_heads, layer.num_kv_heads, layer.head_size) == (nh // size, nkv // size, hd)
        for sid, t in (("q", q), ("k", k), ("v", v)):
            layer.weight.weight_loader(layer.weight, t, sid)
        expect = torch.cat([chunk(q, size, rank), chunk(k, size, rank), chunk(v, size, rank)])
        assert torch.equal(layer.weight.data, expect)
        shards = layer.qkv_shards()
        assert sum(s[1] for s in shards) == layer.weight.shape[0]
        assert sum(s[3] for s in shards) == packed.shape[0]

        lq = L.QKVParallelLinear(hidden, hd, nh, nkv, bias=True, quantization="int8")
        lq.qweight.weight_loader(lq.qweight, packed_q)
        lq.scales.weight_loader(lq.scales, packed_s)
        lq.bias.weight_loader(lq.bias, packed_s)
        nq, nk = nh * hd, nkv * hd
        split = lambda t: torch.cat([chunk(t[:nq], size, rank), chunk(t[nq:nq + nk], size, rank),
                                     chunk(t[nq + nk:], size, rank)])
        assert torch.equal(lq.qweight.data, split(packed_q))
        assert torch.equal(lq.scales.data, split(packed_s))
        assert torch.equal(lq.bias.data, split(packed_s))
    tp(0, 1)
    assert L.QKVParallelLinear(hidden, hd, nh).num_kv_heads == nh  # kv heads default to q heads


def test_indivisible_sizes_are_rejected(tp):
    tp(0, 4)
    with pytest.raises(AssertionError):
        L.ColumnParallelLinear(16, 30)
    with pytest.raises(AssertionError):
        L.RowParallelLinear(30, 16)


def test_unquantized_forward_and_sharded_sum(tp):
    torch.manual_seed(0)
    x = torch.randn(5, 32)
    W = torch.randn(24, 32)
    b = torch.randn(24)
    tp(0, 1)
    rep = L.ReplicatedLinear(32, 24, bias=True)
    rep.weight.weight_loader(rep.weight, W)
    rep.bias.weight_loader(rep.bias, b)
    ref = torch.nn.functional.linear(x, W, b)
    assert torch.allclose(rep(x), ref)
    # column-parallel outputs concatenate; row-parallel partials add up (bias only on rank 0)
    outs, partial = [], torch.zeros(5, 24)
    for rank in range(4):
        tp(rank, 4)
        col = L.ColumnParallelLinear(32, 24, bias=True)
        col.weight.weight_loader(col.weight, W)
        col.bias.weight_loader(col.bias, b)
        outs.append(col(x))
        row = L.RowParallelLinear(32, 24)
        row.tp_size = 1  # no process group in this test: add the partials by hand
        row.weight.weight_loader(row.weight, W)
        partial += row(x.chunk(4, dim=1)[rank])
    assert torch.allclose(torch.cat(outs, dim=1), ref, atol=1e-5)
    assert torch.allclose(partial + b, ref, atol=1e-4)


class _Recorder(QuantMethod):
    def __init__(self):
        self.seen = []

    def create_weights(self, layer, input_size, output_size):
        layer.qweight = nn.Parameter(torch.zeros(output_size, input_size, dtype=torch.int8), requires_grad=False)
        layer.scales = nn.Parameter(torch.ones(output_size), requires_grad=False)

    def quantize_activation(self, x):
        return None

    def apply(self, x, layer, bias=None):
        self.seen.append(bias)
        return torch.zeros(*x.shape[:-1], layer.qweight.shape[0])


def test_quantized_forward_dispatch_and_bias_argument(tp, monkeypatch):
    monkeypatch.setitem(L._QUANT_METHODS, "int8", _Recorder)
    tp(0, 2)
    col = L.ColumnParallelLinear(16, 8, bias=True, quantization="int8")
    col(torch.zeros(3, 16))
    assert col.quant_method.seen == [None]          # apply_linear never forwards a bias
    row0 = L.RowParallelLinear(16, 8, bias=True, quantization="int8")
    row0.tp_size = 1
    row0(torch.zeros(3, 8))
    assert row0.quant_method.seen[0] is row0.bias   # rank 0 passes its bias explicitly
    tp(1, 2)
    row1 = L.RowParallelLinear(16, 8, bias=True, quantization="int8")
    row1.tp_size = 1
    row1(torch.zeros(3, 8))
    assert row1.quant_method.seen == [None]         # other ranks pass None


def test_quant_methods_prefer_explicit_bias(monkeypatch):
    from tiny_vllm_b200.quantization import int8 as int8_mod, w8a8 as w8a8_mod
    calls = {}
    monkeypatch.setattr(int8_mod, "apply_int8_weight_only_linear",
                        lambda x, q, s, b: calls.setdefault("int8", b))
    monkeypatch.setattr(w8a8_mod, "quantize_activation_int8", lambda x: (x, x))
    monkeypatch.setattr(w8a8_mod, "apply_w8a8_linear",
                        lambda xq, a, q, s, bias, out_dtype, out_shape: calls.setdefault("w8a8", (bias, out_shape)))
    layer = nn.Module()
    layer.qweight = torch.zeros(8, 16, dtype=torch.int8)
    layer.scales = layer.w_scales = torch.ones(8)
    layer.bias = torch.full((8,), 2.0)
    explicit = torch.full((8,), 5.0)
    x = torch.zeros(2, 3, 16)
    Int8WeightOnlyQuantMethod().apply(x, layer, explicit)
    assert calls.pop("int8") is explicit
    Int8WeightOnlyQuantMethod().apply(x, layer)
    assert calls.pop("int8") is layer.bias
    W8A8QuantMethod().apply(x, layer, explicit)
    bias, shape = calls.pop("w8a8")
    assert bias is explicit and shape == (2, 3, 8)
    W8A8QuantMethod().apply(x, layer)
    assert calls.pop("w8a8")[0] is layer.bias

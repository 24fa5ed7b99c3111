"""The layer classes on the GPU: quantized forwards through the QuantMethod plug-ins,
CUDA-graph capture of decode-sized calls, bias selection."""
import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import device_status_ok
from tiny_vllm_b200.layers import linear as L

pytestmark = pytest.mark.gpu


def build(cls, quant, *args, **kw):
    with torch.device("cuda"):
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            return cls(*args, quantization=quant, **kw)
        finally:
            torch.set_default_dtype(prev)


@pytest.mark.parametrize("quant,scale", [("int8", "scales"), ("w8a8", "w_scales")])
def test_qwen3_layer_shapes_forward(quant, scale):
    hidden, inter = 1024, 3072
    layers = {
        "qkv": build(L.QKVParallelLinear, quant, hidden, 128, 16, 8),
        "o": build(L.RowParallelLinear, quant, 2048, hidden),
        "gate_up": build(L.MergedColumnParallelLinear, quant, hidden, [inter, inter]),
        "down": build(L.RowParallelLinear, quant, inter, hidden),
    }
    for name, layer in layers.items():
        N, K = layer.qweight.shape
        q, s = O.make_weight(N, K, seed=K + N)
        layer.qweight.weight_loader(layer.qweight, q)
        getattr(layer, scale).weight_loader(getattr(layer, scale), s)
        x = O.make_activation(48, K, seed=1)
        y = layer(x.cuda())
        assert y.shape == (48, N) and y.dtype == torch.bfloat16
        if quant == "int8":
            ref = O.w8a16_dequant_matmul(x, q, s)
        else:
            xq, a_s = O.quantize_per_row_dynamic(x)
            ref = O.w8a8_dequant_matmul(xq, a_s, q, s, None, torch.bfloat16)
        m = O.tensor_metrics(ref, y)
        assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, (name, m)
    assert device_status_ok()


@pytest.mark.parametrize("quant,scale", [("int8", "scales"), ("w8a8", "w_scales")])
def test_layer_bias_and_3d_input(quant, scale):
    layer = build(L.ColumnParallelLinear, quant, 256, 192, bias=True)
    q, s = O.make_weight(192, 256, seed=4)
    b = (torch.randn(192, generator=torch.Generator().manual_seed(2)) * 0.1).to(torch.bfloat16)
    layer.qweight.data.copy_(q)
    getattr(layer, scale).data.copy_(s)
    layer.bias.data.copy_(b)
    x = O.make_activation(12, 256, seed=2).view(3, 4, 256)
    y = layer(x.cuda())
    assert y.shape == (3, 4, 192)
    x2 = x.view(12, 256)
    if quant == "int8":
        ref = O.w8a16_dequant_matmul(x2, q, s, b)
    else:
        xq, a_s = O.quantize_per_row_dynamic(x2)
        ref = O.w8a8_dequant_matmul(xq, a_s, q, s, b, torch.bfloat16)
    m = O.tensor_metrics(ref, y.view(12, 192))
    assert m["relative_l2"] <= 1e-2 and m["cosine_similarity"] >= 0.9999, m


@pytest.mark.parametrize("quant,scale", [("int8", "scales"), ("w8a8", "w_scales")])
@pytest.mark.parametrize("bs", [1, 16, 256])
def test_cuda_graph_capture_of_decode_call(quant, scale, bs):
    layer = build(L.MergedColumnParallelLinear, quant, 1024, [3072, 3072])
    q, s = O.make_weight(6144, 1024, seed=8)
    layer.qweight.data.copy_(q)
    getattr(layer, scale).data.copy_(s)
    static_x = torch.zeros(512, 1024, dtype=torch.bfloat16, device="cuda")
    x1 = O.make_activation(bs, 1024, seed=bs).cuda()
    x2 = O.make_activation(bs, 1024, seed=bs + 1).cuda()
    static_x[:bs] = x1
    eager1 = layer(static_x[:bs]).clone()      # warm-up: sizes the workspace outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_y = layer(static_x[:bs])
    static_x[:bs] = x2
    graph.replay()
    torch.cuda.synchronize()
    eager2 = layer(x2)
    assert torch.equal(static_y, eager2)
    static_x[:bs] = x1
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_y, eager1)
    assert device_status_ok()


@pytest.mark.parametrize("quant,scale", [("int8", "scales"), ("w8a8", "w_scales")])
def test_cuda_graphs_for_the_runner_batch_list_share_one_pool(quant, scale):
    # The reference's runner captures one decode graph per batch size of
    # [1, 2, 4, 8] + range(16, max_bs + 1, 16), largest first, all in ONE memory pool, over views of
    # the same static buffers (nanovllm/engine/model_runner.py:298-335).  The same here over a
    # decoder layer's four projections (qkv -> o, gate_up -> down): every graph must replay to
    # what the eager call gives for that batch size, also after the other graphs were replayed.
    max_bs = 512
    sizes = [1, 2, 4, 8] + list(range(16, max_bs + 1, 16))
    hidden, inter = 1024, 3072
    layers = {
        "qkv": (build(L.QKVParallelLinear, quant, hidden, 128, 16, 8), 4096, hidden),
        "o": (build(L.RowParallelLinear, quant, 2048, hidden), hidden, 2048),
        "gate_up": (build(L.MergedColumnParallelLinear, quant, hidden, [inter, inter]), 2 * inter, hidden),
        "down": (build(L.RowParallelLinear, quant, inter, hidden), hidden, inter),
    }
    for i, (name, (layer, n, k)) in enumerate(layers.items()):
        q, s = O.make_weight(n, k, seed=20 + i)
        layer.qweight.data.copy_(q)
        getattr(layer, scale).data.copy_(s)

    def block(x):
        qkv = layers["qkv"][0](x)
        attn = layers["o"][0](qkv[:, :2048].contiguous())
        gu = layers["gate_up"][0](attn)
        return layers["down"][0]((gu[:, :inter] * torch.sigmoid(gu[:, inter:])).contiguous())

    static_x = torch.zeros(max_bs, hidden, dtype=torch.bfloat16, device="cuda")
    static_y = torch.zeros(max_bs, hidden, dtype=torch.bfloat16, device="cuda")
    probe = O.make_activation(max_bs, hidden, seed=77).cuda()
    graphs, pool = {}, None
    for bs in reversed(sizes):
        static_x[:bs] = probe[:bs]
        static_y[:bs] = block(static_x[:bs])          # warm-up, as the runner does
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool):
            static_y[:bs] = block(static_x[:bs])
        if pool is None:
            pool = g.pool()
        graphs[bs] = g
    torch.cuda.synchronize()
    other = O.make_activation(max_bs, hidden, seed=78).cuda()
    for bs in (1, 2, 8, 16, 48, 64, 80, 256, 496, 512, 4, 32):      # out of capture order on purpose
        static_x[:bs] = other[:bs]
        graphs[bs].replay()
        torch.cuda.synchronize()
        want = block(other[:bs])
        assert torch.equal(static_y[:bs], want), bs
    assert len(graphs) == 36
    assert device_status_ok()


def test_apply_quantized_writes_into_a_caller_buffer():
    # the row-parallel partial of a tensor-parallel exchange is produced straight into the
    # symmetric buffer: same bits as a fresh output, and the given tensor is the one returned
    layer = build(L.RowParallelLinear, "w8a8", 2048, 1024)
    q, s = O.make_weight(1024, 2048, seed=9)
    layer.qweight.weight_loader(layer.qweight, q)
    layer.w_scales.weight_loader(layer.w_scales, s)
    x = O.make_activation(64, 2048, seed=2).cuda()
    x_q, a_s = layer.quant_method.quantize_activation(x)
    fresh = layer.quant_method.apply_quantized(x_q, a_s, layer, torch.bfloat16)
    slab = torch.zeros(3, 64, 1024, dtype=torch.bfloat16, device="cuda")
    got = layer.quant_method.apply_quantized(x_q, a_s, layer, torch.bfloat16, out=slab[1])
    assert got.data_ptr() == slab[1].data_ptr()
    assert torch.equal(slab[1], fresh) and not slab[0].any() and not slab[2].any()
    with pytest.raises(RuntimeError):
        layer.quant_method.apply_quantized(x_q, a_s, layer, torch.bfloat16, out=slab[1].t())
    assert device_status_ok()

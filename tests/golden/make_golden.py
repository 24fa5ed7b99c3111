"""Generates tests/golden/quant_linear_golden.npz from the REFERENCE's own Python code.

Run where a checkout of the reference (daiyu1111/tiny-vllm) is available, passing its path
(or set NANOVLLM_REFERENCE):

    python tests/golden/make_golden.py /path/to/reference

It imports ``nanovllm.quantization.utils`` and ``nanovllm.quantization.cuda`` from
the reference, unmodified, runs them on CPU on seeded synthetic inputs and stores
inputs and outputs.  The fixture is what pins ``oracle/quant_linear_oracle.py``;
the tests only read the .npz, never the reference.

Three fixtures are written:

* ``quant_linear_golden.npz`` — five small cases of the four operator functions (below);
* ``fused_producers_golden.npz`` — the reference's ``RMSNorm`` (with and without the residual
  add, ``nanovllm/layers/layernorm.py:16-50``) and ``SiluAndMul``
  (``nanovllm/layers/activation.py:11-14``) modules.  Both are decorated with
  ``torch.compile``; Inductor's C++ backend does not build in the container this script runs
  in, so the modules run under ``torch.compiler.set_stance("force_eager")``: the same Python
  code, executed operation by operation (the activation then rounds silu(gate) to 16 bits
  before the product, which the compiled form does not);
* ``baseline_shapes_golden.npz`` — one case per benchmark shape family: the W8A16 linear
  256 x 1024 -> 6144 and a W8A8 decode shape 16 x 1024 -> 4096.  Inputs are regenerated from
  seeds by the tests; stored are SHA-256 digests of the reference's integer results and
  sampled rows / small outputs of its matmul paths.

Stored per case ``c<i>_``: x (16-bit pattern as uint16), w (fp32), bias (uint16),
and from the reference: q, s (quantize_int8_per_channel), xq, a_s
(quantize_int8_per_row_dynamic), y_w8a16 (int8_weight_only_linear_fallback),
y_w8a8 (w8a8_linear_fallback), acc_i32 (w8a8_linear_fallback with unit scales
evaluated in float64: exact integers, the int32 accumulators).
"""
import sys
from pathlib import Path

import numpy as np
import torch

CASES = [
    # (M, K, N, dtype, with_bias, outliers)
    (37, 256, 192, "bfloat16", True, True),
    (130, 512, 320, "bfloat16", False, True),
    (1, 128, 64, "bfloat16", False, False),
    (16, 256, 128, "float16", True, True),
    (64, 1024, 96, "bfloat16", False, True),
]


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    import os
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NANOVLLM_REFERENCE")
    if not where:
        raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
    ref = Path(where)
    sys.path.insert(0, str(ref))
    from nanovllm.quantization.cuda import int8_weight_only_linear_fallback, w8a8_linear_fallback
    from nanovllm.quantization.utils import quantize_int8_per_channel, quantize_int8_per_row_dynamic

    out = {"n_cases": np.array(len(CASES)), "torch_version": np.array(torch.__version__)}
    for i, (M, K, N, dt_name, with_bias, outliers) in enumerate(CASES):
        dt = getattr(torch, dt_name)
        g = torch.Generator().manual_seed(100 + i)
        w = torch.randn(N, K, generator=g) * 0.02
        x = torch.randn(M, K, generator=g)
        if outliers:
            idx = torch.randperm(K, generator=g)[: max(1, -(-K // 100))]
            x[:, idx] *= 20.0
        x = x.to(dt)
        bias = (torch.randn(N, generator=g) * 0.1).to(dt) if with_bias else None

        q, s = quantize_int8_per_channel(w)
        xq, a_s = quantize_int8_per_row_dynamic(x)
        y16 = int8_weight_only_linear_fallback(x, q, s, bias)
        y8 = w8a8_linear_fallback(xq, a_s, q, s, bias, dt)
        acc = w8a8_linear_fallback(xq, torch.ones(M), q, torch.ones(N), None, torch.float64)
        assert torch.equal(acc, acc.round()) and acc.abs().max() < 2 ** 31

        p = f"c{i}_"
        out[p + "shape"] = np.array([M, K, N])
        out[p + "dtype"] = np.array(dt_name)
        out[p + "x"] = bits16(x)
        # the float weight is kept for the small cases only (it does not compress)
        out[p + "w"] = w.numpy() if N * K <= 64 * 1024 else np.zeros((0, 0), np.float32)
        out[p + "bias"] = bits16(bias) if bias is not None else np.zeros(0, np.uint16)
        out[p + "q"] = q.numpy()
        out[p + "s"] = s.numpy()
        out[p + "xq"] = xq.numpy()
        out[p + "a_s"] = a_s.numpy()
        out[p + "y_w8a16"] = bits16(y16)
        out[p + "y_w8a8"] = bits16(y8)
        out[p + "acc_i32"] = acc.to(torch.int32).numpy()
    dst = Path(__file__).resolve().parent / "quant_linear_golden.npz"
    np.savez_compressed(dst, **out)
    print(dst, dst.stat().st_size, "bytes")
    fused_producers()
    baseline_shapes(quantize_int8_per_channel, quantize_int8_per_row_dynamic,
                    int8_weight_only_linear_fallback, w8a8_linear_fallback)


NORM_CASES = [  # (M, K, dtype, with_residual)
    (37, 256, "bfloat16", True), (16, 1024, "float16", False), (64, 1024, "bfloat16", True),
    (5, 272, "float16", True)]
SILU_CASES = [(37, 384, "bfloat16"), (16, 3072, "float16"), (8, 1024, "bfloat16")]  # (M, I, dtype)


def fused_producers():
    from nanovllm.layers.activation import SiluAndMul
    from nanovllm.layers.layernorm import RMSNorm

    out = {"n_norm": np.array(len(NORM_CASES)), "n_silu": np.array(len(SILU_CASES)),
           "eps": np.array(1e-6), "mode": np.array("force_eager")}
    with torch.compiler.set_stance("force_eager"), torch.no_grad():
        for i, (M, K, dt_name, with_res) in enumerate(NORM_CASES):
            dt = getattr(torch, dt_name)
            g = torch.Generator().manual_seed(300 + i)
            x = (torch.randn(M, K, generator=g) * 1.5).to(dt)
            res = (torch.randn(M, K, generator=g) * 2).to(dt) if with_res else None
            norm = RMSNorm(K, eps=1e-6).to(dt)
            norm.weight.copy_((1.0 + 0.2 * torch.randn(K, generator=g)).to(dt))
            if with_res:
                y, new_res = norm(x.clone(), res.clone())
            else:
                y, new_res = norm(x.clone()), None
            p = f"n{i}_"
            out[p + "shape"] = np.array([M, K])
            out[p + "dtype"] = np.array(dt_name)
            out[p + "x"] = bits16(x)
            out[p + "res"] = bits16(res) if with_res else np.zeros(0, np.uint16)
            out[p + "w"] = bits16(norm.weight.data)
            out[p + "y"] = bits16(y)
            out[p + "new_res"] = bits16(new_res) if with_res else np.zeros(0, np.uint16)
        act = SiluAndMul()
        for i, (M, inter, dt_name) in enumerate(SILU_CASES):
            dt = getattr(torch, dt_name)
            g = torch.Generator().manual_seed(400 + i)
            gate_up = (torch.randn(M, 2 * inter, generator=g) * 2).to(dt)
            p = f"s{i}_"
            out[p + "shape"] = np.array([M, inter])
            out[p + "dtype"] = np.array(dt_name)
            out[p + "gate_up"] = bits16(gate_up)
            out[p + "y"] = bits16(act(gate_up))
    dst = Path(__file__).resolve().parent / "fused_producers_golden.npz"
    np.savez_compressed(dst, **out)
    print(dst, dst.stat().st_size, "bytes")


def sha(t: torch.Tensor) -> np.ndarray:
    import hashlib
    return np.array(hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest())


def baseline_shapes(quantize_int8_per_channel, quantize_int8_per_row_dynamic,
                    int8_weight_only_linear_fallback, w8a8_linear_fallback):
    """Inputs come from the same seeded generators the oracle exposes (make_weight /
    make_activation): N(0, 0.02) weights, N(0, 1) activations with 1 % outlier channels x20."""
    def weight(N, K, seed):
        g = torch.Generator(device="cpu").manual_seed(seed)
        return torch.randn(N, K, generator=g, device="cpu") * 0.02

    def activation(M, K, seed, outliers):
        g = torch.Generator(device="cpu").manual_seed(seed + 1000003)
        x = torch.randn(M, K, generator=g, device="cpu")
        if outliers:
            idx = torch.randperm(K, generator=g, device="cpu")[:max(1, -(-K // 100))]
            x[:, idx] *= 20.0
        return x.to(torch.bfloat16)

    out = {}
    # configs[0]: single W8A16 linear, 256 x 1024 -> 6144, seed 0, no outliers
    M, K, N = 256, 1024, 6144
    q, s = quantize_int8_per_channel(weight(N, K, 0))
    x = activation(M, K, 0, False)
    y = int8_weight_only_linear_fallback(x, q, s, None)
    out["w8a16_shape"] = np.array([M, K, N])
    out["w8a16_q_sha"], out["w8a16_s_sha"] = sha(q), sha(s)
    out["w8a16_rows"] = np.arange(0, M, 16)
    out["w8a16_y_rows"] = bits16(y[::16])
    # configs[1] decode shape: W8A8, 16 tokens through qkv 1024 -> 4096, outlier channels
    M, K, N = 16, 1024, 4096
    q, s = quantize_int8_per_channel(weight(N, K, 1))
    x = activation(M, K, 1, True)
    xq, a_s = quantize_int8_per_row_dynamic(x)
    acc = w8a8_linear_fallback(xq, torch.ones(M), q, torch.ones(N), None, torch.float64)
    assert torch.equal(acc, acc.round())
    out["w8a8_shape"] = np.array([M, K, N])
    out["w8a8_q_sha"], out["w8a8_s_sha"] = sha(q), sha(s)
    out["w8a8_xq"] = xq.numpy()
    out["w8a8_a_s"] = a_s.numpy()
    out["w8a8_acc_i32"] = acc.to(torch.int32).numpy()
    out["w8a8_y"] = bits16(w8a8_linear_fallback(xq, a_s, q, s, None, torch.bfloat16))
    dst = Path(__file__).resolve().parent / "baseline_shapes_golden.npz"
    np.savez_compressed(dst, **out)
    print(dst, dst.stat().st_size, "bytes")


if __name__ == "__main__":
    main()

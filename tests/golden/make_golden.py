"""Generates tests/golden/quant_linear_golden.npz from the REFERENCE's own Python code.

Run where a checkout of the reference (daiyu1111/tiny-vllm) is available, passing its path
(or set NANOVLLM_REFERENCE):

    python tests/golden/make_golden.py /path/to/reference

It imports ``nanovllm.quantization.utils`` and ``nanovllm.quantization.cuda`` from
the reference, unmodified, runs them on CPU on seeded synthetic inputs and stores
inputs and outputs.  The fixture is what pins ``oracle/quant_linear_oracle.py``;
the tests only read the .npz, never the reference.

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


if __name__ == "__main__":
    main()

"""The CPU oracle against the golden vectors produced by the reference's own Python
functions (tests/golden/make_golden.py).  Integer results must be identical; the
16-bit matmul outputs are compared with a tolerance because the CPU BLAS behind
``F.linear`` may order its fp32 additions differently from one host to another."""
import numpy as np
import torch

from oracle import quant_linear_oracle as O


def test_per_channel_quant_matches_reference(golden_cases):
    checked = 0
    for c in golden_cases:
        if c["w"] is None:
            continue
        q, s = O.quantize_per_channel(c["w"])
        assert torch.equal(q, c["q"]) and torch.equal(s, c["s"])
        checked += 1
    assert checked >= 2


def test_per_row_dynamic_quant_matches_reference(golden_cases):
    for c in golden_cases:
        xq, a_s = O.quantize_per_row_dynamic(c["x"])
        assert torch.equal(xq, c["xq"]), c["id"]
        assert torch.equal(a_s, c["a_s"]), c["id"]


def test_int32_accumulators_match_reference(golden_cases, oracle_c_lib):
    for c in golden_cases:
        for use_c in (True, False):
            acc = O.w8a8_int32_accumulators(c["xq"], c["q"], use_c=use_c)
            assert acc.dtype == torch.int32
            assert torch.equal(acc, c["acc_i32"]), (c["id"], use_c)


def test_dequant_matmul_paths_match_reference(golden_cases):
    for c in golden_cases:
        y16 = O.w8a16_dequant_matmul(c["x"], c["q"], c["s"], c["bias"])
        m = O.tensor_metrics(c["y_w8a16"], y16)
        assert m["relative_l2"] < 2e-3 and m["cosine_similarity"] > 0.99999, (c["id"], m)
        y8 = O.w8a8_dequant_matmul(c["xq"], c["a_s"], c["q"], c["s"], c["bias"], c["dtype"])
        m = O.tensor_metrics(c["y_w8a8"], y8)
        assert m["relative_l2"] < 2e-3 and m["cosine_similarity"] > 0.99999, (c["id"], m)


def test_native_epilogue_is_within_the_parity_gate_of_the_reference_path(golden_cases):
    # The fused-kernel arithmetic (int32 accumulate, fp32 scale) and the reference's
    # Python path (dequantise both sides to 16 bit) must agree within rel-L2 1e-2.
    for c in golden_cases:
        y = O.w8a8_native_epilogue(c["acc_i32"], c["a_s"], c["s"], c["bias"], c["dtype"])
        m = O.tensor_metrics(c["y_w8a8"], y)
        assert m["relative_l2"] < 1e-2 and m["cosine_similarity"] >= 0.9999, (c["id"], m)
        y16 = O.w8a16_native_reference(c["x"], c["q"], c["s"], c["bias"])
        m = O.tensor_metrics(c["y_w8a16"], y16)
        assert m["relative_l2"] < 1e-2 and m["cosine_similarity"] >= 0.9999, (c["id"], m)


def test_edge_rows():
    # all-zero row -> scale clamps to 1e-8, codes 0; a single huge value -> +-127
    x = torch.zeros(3, 32, dtype=torch.bfloat16)
    x[1, 5] = -3.0
    x[2, 0] = 1e-30
    xq, a_s = O.quantize_per_row_dynamic(x)
    assert a_s[0].item() == np.float32(1e-8) and int(xq[0].abs().max()) == 0
    assert int(xq[1, 5]) == -127 and a_s[1].item() == np.float32(3.0) / np.float32(127.0)
    assert a_s[2].item() == np.float32(1e-8)


def test_metrics_definition():
    a = torch.tensor([1.0, 2.0, 3.0])
    m = O.tensor_metrics(a, a)
    assert m["relative_l2"] == 0.0 and abs(m["cosine_similarity"] - 1.0) < 1e-12

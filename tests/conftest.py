"""Shared pytest set-up: the ``gpu`` marker, import paths, golden-fixture access."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden" / "quant_linear_golden.npz"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def _from_bits16(arr: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(arr.view(np.int16).copy()).view(dtype)


def load_golden_cases():
    """List of dicts with torch tensors, one per case of the golden fixture."""
    z = np.load(GOLDEN)
    cases = []
    for i in range(int(z["n_cases"])):
        p = f"c{i}_"
        dt = getattr(torch, str(z[p + "dtype"]))
        M, K, N = (int(v) for v in z[p + "shape"])
        bias = z[p + "bias"]
        cases.append({
            "id": i, "M": M, "K": K, "N": N, "dtype": dt,
            "x": _from_bits16(z[p + "x"], dt),
            "w": torch.from_numpy(z[p + "w"]) if z[p + "w"].size else None,
            "bias": _from_bits16(bias, dt) if bias.size else None,
            "q": torch.from_numpy(z[p + "q"]), "s": torch.from_numpy(z[p + "s"]),
            "xq": torch.from_numpy(z[p + "xq"]), "a_s": torch.from_numpy(z[p + "a_s"]),
            "y_w8a16": _from_bits16(z[p + "y_w8a16"], dt),
            "y_w8a8": _from_bits16(z[p + "y_w8a8"], dt),
            "acc_i32": torch.from_numpy(z[p + "acc_i32"]),
        })
    return cases


@pytest.fixture(scope="session")
def golden_cases():
    return load_golden_cases()


def load_fused_producer_cases():
    """(norm cases, activation cases) of tests/golden/fused_producers_golden.npz: outputs of the
    reference's RMSNorm / SiluAndMul modules."""
    z = np.load(ROOT / "tests" / "golden" / "fused_producers_golden.npz")
    norm, silu = [], []
    for i in range(int(z["n_norm"])):
        p = f"n{i}_"
        dt = getattr(torch, str(z[p + "dtype"]))
        M, K = (int(v) for v in z[p + "shape"])
        res = z[p + "res"]
        norm.append({"id": i, "M": M, "K": K, "dtype": dt, "eps": float(z["eps"]),
                     "x": _from_bits16(z[p + "x"], dt).view(M, K),
                     "res": _from_bits16(res, dt).view(M, K) if res.size else None,
                     "w": _from_bits16(z[p + "w"], dt),
                     "y": _from_bits16(z[p + "y"], dt).view(M, K),
                     "new_res": _from_bits16(z[p + "new_res"], dt).view(M, K) if res.size else None})
    for i in range(int(z["n_silu"])):
        p = f"s{i}_"
        dt = getattr(torch, str(z[p + "dtype"]))
        M, inter = (int(v) for v in z[p + "shape"])
        silu.append({"id": i, "M": M, "I": inter, "dtype": dt,
                     "gate_up": _from_bits16(z[p + "gate_up"], dt).view(M, 2 * inter),
                     "y": _from_bits16(z[p + "y"], dt).view(M, inter)})
    return norm, silu


@pytest.fixture(scope="session")
def fused_producer_cases():
    return load_fused_producer_cases()


@pytest.fixture(scope="session")
def baseline_shape_golden():
    """Reference results at the benchmark's shape families (digests, sampled rows)."""
    z = np.load(ROOT / "tests" / "golden" / "baseline_shapes_golden.npz")
    return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def oracle_c_lib():
    """Builds the C part of the oracle (gcc) once per session."""
    from oracle import build_oracle
    return build_oracle.build()

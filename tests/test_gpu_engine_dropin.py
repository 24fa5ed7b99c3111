"""The reference's own engine over these layers, on the GPU.

``tests/engine_under_reference.py`` builds a random-initialised Qwen3-architecture model
directory and its quantized artifacts, then starts the reference's unmodified ``LLM`` (engine,
scheduler, ``ModelRunner`` with warm-up and CUDA-graph capture, attention) from the mirror in
``oracle/_ref`` with this package installed under the reference's module names, and generates
tokens.  Checked: the model's linears ARE this package's classes, the runner captured one graph
per decode batch size of its list, every sequence got its tokens, the library launched kernels
and its device status word stayed clean.  Skipped without the mirror or without flash-attn
(which the reference's attention layer imports).
"""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
HARNESS = ROOT / "tests" / "engine_under_reference.py"


def _engine_line(cmd):
    res = subprocess.run([sys.executable, str(HARNESS), *cmd], capture_output=True, text=True, timeout=900)
    lines = [l for l in res.stdout.splitlines() if l.startswith("ENGINE ")]
    assert res.returncode == 0 and lines, (res.stdout[-2000:], res.stderr[-3000:])
    return json.loads(lines[-1][len("ENGINE "):])


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    if not (ROOT / "oracle" / "_ref" / "nanovllm" / "engine" / "llm_engine.py").is_file():
        pytest.skip("oracle/_ref holds no mirror of the reference")
    if importlib.util.find_spec("flash_attn") is None:
        pytest.skip("the reference's attention layer needs flash-attn")
    root = tmp_path_factory.mktemp("engine")
    res = subprocess.run([sys.executable, str(HARNESS), "make", "--dir", str(root), "--layers", "2", "--vocab", "8192"],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    return root


@pytest.mark.parametrize("mode", ["w8a8", "int8"])
def test_reference_engine_generates_over_these_layers(model_dir, mode):
    line = _engine_line(["run", "--dir", str(model_dir), "--mode", mode, "--impl", "ours", "--seqs", "40",
                         "--out", "12", "--max-num-seqs", "64", "--max-model-len", "1024",
                         "--max-num-batched-tokens", "4096"])
    print(line)
    assert line["ok"] and line["linear_module"].startswith("tiny_vllm_b200")
    assert line["graph_batch_sizes"] == [1, 2, 4, 8, 16, 32, 48, 64] and line["graphs"] == 8
    assert line["b200q_launches"] > 0 and line["device_status"] == 0
    assert line["decode_tokens_per_second"] > 0 and line["prefill_tokens_per_second"] > 0

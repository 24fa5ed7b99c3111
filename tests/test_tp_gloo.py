"""Tensor-parallel host path with a real process group: two CPU ranks over gloo.
Covers rank discovery at construction, per-rank shard loading and the all-reduce after
a row-parallel layer (unquantized weights: the quantized kernels need a GPU)."""
import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import tiny_vllm_b200  # noqa: F401
    from tiny_vllm_b200.layers.linear import MergedColumnParallelLinear, RowParallelLinear
    try:
        g = torch.Generator().manual_seed(7)
        x = torch.randn(6, 32, generator=g)
        w_gu = torch.randn(64, 32, generator=g)
        w_down = torch.randn(32, 32, generator=g)
        b_down = torch.randn(32, generator=g)
        gate_up = MergedColumnParallelLinear(32, [32, 32])
        assert (gate_up.tp_rank, gate_up.tp_size) == (rank, world)
        gate_up.weight.weight_loader(gate_up.weight, w_gu[:32], 0)
        gate_up.weight.weight_loader(gate_up.weight, w_gu[32:], 1)
        down = RowParallelLinear(32, 32, bias=True)
        down.weight.weight_loader(down.weight, w_down)
        down.bias.data.copy_(b_down)
        h = gate_up(x)                              # [6, 64 / world]
        gate, up = h.chunk(2, dim=-1)
        y = down(gate * up)                          # all-reduce inside
        full = torch.nn.functional.linear(x, w_gu)
        ref = torch.nn.functional.linear(full[:, :32] * full[:, 32:], w_down, b_down)
        ok = bool(torch.allclose(y, ref, atol=1e-3, rtol=1e-4))

        # a communicator installed with set_tp_all_reduce takes over the exchange step
        from tiny_vllm_b200.layers import linear as LL

        class CountingComm:
            """Stands in for layers.tp_comm.PeerAllReduce: same ``reduce`` contract."""
            calls = 0

            def reduce(self, t):
                CountingComm.calls += 1
                dist.all_reduce(t)
                return t

        LL.set_tp_all_reduce(CountingComm())
        y2 = down(gate * up)
        LL.set_tp_all_reduce(None)
        y3 = down(gate * up)
        ok = ok and CountingComm.calls == 1 and torch.equal(y2, y) and torch.equal(y3, y)
        torch.save({"ok": ok, "y": y}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_row_parallel_all_reduce(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "r0.pt")
    r1 = torch.load(tmp_path / "r1.pt")
    assert r0["ok"] and r1["ok"]
    assert torch.equal(r0["y"], r1["y"])  # every rank holds the reduced result

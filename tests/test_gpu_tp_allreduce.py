"""Peer-memory all-reduce (b200q_tp_allreduce) on two or more GPUs: bit-identical to an fp32
sum in rank order, identical on every rank, repeated calls, both symmetric slots, and a
row-parallel W8A8 layer pair whose partial outputs it reduces.  Skipped on a one-GPU box."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_tensor(rank, n, seed, dtype):
    g = torch.Generator(device="cpu").manual_seed(seed * 100 + rank)
    return torch.randn(n, generator=g, device="cpu").to(dtype)


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import tiny_vllm_b200  # noqa: F401
    from tiny_vllm_b200 import _lib
    from tiny_vllm_b200.layers.tp_comm import PeerAllReduce
    ok, notes = True, []
    try:
        comm = PeerAllReduce(max_bytes=16 << 20)
        for call, (n, dtype) in enumerate([(8192 * 1024, torch.bfloat16), (4096, torch.bfloat16),
                                           (512 * 1024 + 8, torch.float16), (8, torch.bfloat16),
                                           (8192 * 1024, torch.bfloat16)]):
            parts = [_rank_tensor(r, n, call, dtype) for r in range(world)]
            expect = torch.zeros(n, dtype=torch.float32)
            for r in range(world):          # fp32, rank order: what the kernel does
                expect += parts[r].float()
            expect = expect.to(dtype)
            t = comm.buffer((n,), dtype)
            t.copy_(parts[rank])
            comm.all_reduce_(t)
            torch.cuda.synchronize()
            same = torch.equal(t.cpu().view(torch.int16), expect.view(torch.int16))
            ok = ok and same
            if not same:
                notes.append(f"call {call}: mismatch, max diff {(t.cpu().float() - expect.float()).abs().max()}")
        ok = ok and _lib.lib().b200q_device_status() == 0
        # timing against NCCL on the largest message
        t = comm.buffer((8192 * 1024,), torch.bfloat16)
        x = torch.zeros(8192 * 1024, dtype=torch.bfloat16, device="cuda")
        for fn, name in ((lambda: comm.all_reduce_(t), "peer"), (lambda: dist.all_reduce(x), "nccl")):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                fn()
            e1.record()
            torch.cuda.synchronize()
            notes.append(f"{name} 16 MiB all-reduce: {e0.elapsed_time(e1) / 20 * 1e3:.1f} us")
        ok = ok and _lib.lib().b200q_device_status() == 0
        # a quantized row-parallel layer: NCCL sum vs peer-memory sum vs the CPU oracle
        from oracle import quant_linear_oracle as O
        from tiny_vllm_b200.layers import linear as LL
        K, N, M = 512 * world, 384, 96
        q, s = O.make_weight(N, K, seed=11)
        x = O.make_activation(M, K, seed=12)
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        with torch.device("cuda"):
            layer = LL.RowParallelLinear(K, N, quantization="w8a8")
        torch.set_default_dtype(prev)
        layer.qweight.weight_loader(layer.qweight, q)
        layer.w_scales.weight_loader(layer.w_scales, s)
        x_local = x.chunk(world, dim=1)[rank].contiguous().cuda()
        y_nccl = layer(x_local).clone()
        LL.set_tp_all_reduce(comm)
        y_peer = layer(x_local).clone()
        LL.set_tp_all_reduce(None)
        ref = torch.zeros(M, N)
        for r in range(world):               # what each rank computes, summed in fp32
            xq, a_s = O.quantize_per_row_dynamic(x.chunk(world, dim=1)[r].contiguous())
            acc = O.w8a8_int32_accumulators(xq, q.chunk(world, dim=1)[r].contiguous(), use_c=False)
            ref += O.w8a8_native_epilogue(acc, a_s, s, None, torch.bfloat16).float()
        same = torch.equal(y_peer.cpu().view(torch.int16), ref.to(torch.bfloat16).view(torch.int16))
        m = O.tensor_metrics(y_nccl, y_peer)
        ok = ok and same and m["relative_l2"] < 1e-2
        if not same:
            notes.append(f"row-parallel layer: peer sum differs from rank-ordered fp32 sum, {m}")
    except Exception as exc:  # noqa: BLE001
        ok = False
        notes.append(repr(exc))
    torch.save({"ok": ok, "notes": notes}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_peer_all_reduce_matches_rank_ordered_fp32_sum(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"r{r}.pt")
        print(r, res["notes"])
        assert res["ok"], res["notes"]

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
        # pull variant: sum lands in a new local tensor, inputs alternate between the two slots
        for call, (n, dtype) in enumerate([(8192 * 1024, torch.bfloat16), (4096, torch.float16),
                                           (1024 * 1024 + 8, torch.bfloat16), (8, torch.bfloat16),
                                           (8192 * 1024, torch.bfloat16)]):
            parts = [_rank_tensor(r, n, 20 + call, dtype) for r in range(world)]
            expect = torch.zeros(n, dtype=torch.float32)
            for r in range(world):
                expect += parts[r].float()
            expect = expect.to(dtype)
            t = comm.buffer((n,), dtype)
            t.copy_(parts[rank])
            out = comm.all_reduce_pull(t)
            torch.cuda.synchronize()
            if not torch.equal(out.cpu().view(torch.int16), expect.view(torch.int16)):
                ok = False
                notes.append(f"pull call {call} (n={n}): mismatch")
            if not torch.equal(t.cpu().view(torch.int16), parts[rank].view(torch.int16)):
                ok = False
                notes.append(f"pull call {call}: the input buffer was modified")
        ok = ok and _lib.lib().b200q_device_status() == 0
        # in-switch reduction (when the fabric offers a multicast mapping): identical bits on
        # all ranks, within one unit in the last place of the rank-ordered sum
        if comm._mc_ptr != 0:
            for call, (n, dtype) in enumerate([(8192 * 1024, torch.bfloat16), (4096, torch.float16),
                                               (8, torch.bfloat16), (1024 * 1024 + 8, torch.bfloat16)]):
                parts = [_rank_tensor(r, n, 70 + call, dtype) for r in range(world)]
                expect = torch.zeros(n, dtype=torch.float32)
                for r in range(world):
                    expect += parts[r].float()
                expect = expect.to(dtype)
                t = comm.buffer((n,), dtype)
                t.copy_(parts[rank])
                comm.all_reduce_multimem_(t)
                torch.cuda.synchronize()
                got = t.cpu()
                ulp = (got.view(torch.int16).int() - expect.view(torch.int16).int()).abs()
                if int(ulp.max()) > 1:
                    ok = False
                    notes.append(f"multimem call {call} (n={n}): off by {int(ulp.max())} units in the last place")
                gathered = [torch.empty_like(t) for _ in range(world)]
                dist.all_gather(gathered, t)
                if not all(torch.equal(g.view(torch.int16), t.view(torch.int16)) for g in gathered):
                    ok = False
                    notes.append(f"multimem call {call}: ranks disagree")
            notes.append("multicast mapping available")
        else:
            notes.append("no multicast mapping: in-switch reduction not tested")
        ok = ok and _lib.lib().b200q_device_status() == 0
        # one-trip kernel for small tensors: any local tensor, in place, same bits
        for call, (n, dtype) in enumerate([(8, torch.bfloat16), (4096, torch.float16),
                                           (16 * 1024, torch.bfloat16), (96 * 1024, torch.bfloat16),
                                           (512 * 1024, torch.bfloat16), (8, torch.float16)]):
            parts = [_rank_tensor(r, n, 50 + call, dtype) for r in range(world)]
            expect = torch.zeros(n, dtype=torch.float32)
            for r in range(world):
                expect += parts[r].float()
            expect = expect.to(dtype)
            t = parts[rank].cuda()
            if world * n * 4 > comm.fused_bytes // 2:
                continue
            comm.all_reduce_small_(t)
            torch.cuda.synchronize()
            if not torch.equal(t.cpu().view(torch.int16), expect.view(torch.int16)):
                ok = False
                notes.append(f"one-trip call {call} (n={n}): mismatch")
        ok = ok and _lib.lib().b200q_device_status() == 0
        # latency by size: one-trip vs two-shot vs NCCL (CUDA-graph replays)
        for n in (16 * 1024, 128 * 1024, 512 * 1024, 1024 * 1024):
            if world * n * 4 > comm.fused_bytes // 2:
                continue
            loc = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
            sym = comm.buffer((n,), torch.bfloat16)
            sym.zero_()
            row = [f"{n * 2 // 1024} KiB:"]
            for fn, name in ((lambda: comm.all_reduce_small_(loc), "one-trip"),
                             (lambda: comm.all_reduce_(sym), "two-shot"),
                             (lambda: dist.all_reduce(loc), "nccl")):
                row.append(f"{name} {_graph_time_us(fn):.1f} us")
            notes.append(" ".join(row))
        ok = ok and _lib.lib().b200q_device_status() == 0
        # timing against NCCL on the largest message
        t = comm.buffer((8192 * 1024,), torch.bfloat16)
        x = torch.zeros(8192 * 1024, dtype=torch.bfloat16, device="cuda")
        t2 = comm.buffer((8192 * 1024,), torch.bfloat16)
        turn = [0]

        def pull_alternating():
            turn[0] ^= 1
            comm.all_reduce_pull(t if turn[0] else t2)

        routes = [(lambda: comm.all_reduce_(t), "peer"), (pull_alternating, "peer pull"),
                  (lambda: dist.all_reduce(x), "nccl")]
        if comm._mc_ptr != 0:
            routes.insert(2, (lambda: comm.all_reduce_multimem_(t), "peer multimem"))
        for fn, name in routes:
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


def _graph_time_us(fn, reps=20):
    """Microseconds per call of ``fn`` replayed from a CUDA graph (launch overhead excluded)."""
    import torch.distributed as dist
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def _fused_worker(rank, world, port, out_dir):
    """Decode-sized row-parallel layers: GEMM + sum over ranks in one kernel, against the
    two-kernel route (same GEMM kernel, then b200q_tp_allreduce) and the CPU oracle."""
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import tiny_vllm_b200  # noqa: F401
    from oracle import quant_linear_oracle as O
    from tiny_vllm_b200 import _lib
    from tiny_vllm_b200.layers import linear as LL
    from tiny_vllm_b200.layers.tp_comm import PeerAllReduce
    ok, notes = True, []
    try:
        comm = PeerAllReduce(max_bytes=4 << 20)
        LL.set_tp_all_reduce(comm)
        launches = _lib.lib().b200q_launch_count
        for scheme, dtype, N, K_local, with_bias in (("w8a8", torch.bfloat16, 1024, 1024, False),
                                                     ("w8a8", torch.float16, 256, 1536, True),
                                                     ("int8", torch.bfloat16, 1024, 512, False),
                                                     ("int8", torch.float16, 384, 768, True)):
            K = K_local * world
            q, s = O.make_weight(N, K, seed=21)
            prev = torch.get_default_dtype()
            torch.set_default_dtype(dtype)
            with torch.device("cuda"):
                layer = LL.RowParallelLinear(K, N, bias=with_bias, quantization=scheme)
            torch.set_default_dtype(prev)
            layer.qweight.weight_loader(layer.qweight, q)
            scale_param = layer.w_scales if scheme == "w8a8" else layer.scales
            scale_param.weight_loader(scale_param, s)
            if with_bias:
                g = torch.Generator(device="cpu").manual_seed(5)
                layer.bias.data.copy_(torch.randn(N, generator=g).to(dtype))
            for M in (1, 16, 33, 64, 7, 64):      # repeated calls alternate the receive halves
                x = O.make_activation(M, K, seed=30 + M).to(dtype)
                x_local = x.chunk(world, dim=1)[rank].contiguous().cuda()
                before = launches()
                y_fused = layer(x_local)
                n_fused = launches() - before
                # two-kernel route: the same GEMM kernel, then the peer all-reduce
                part = layer.quant_method.apply(x_local, layer, layer.bias if rank == 0 else None)
                buf = comm.buffer(part.shape, part.dtype)
                buf.copy_(part)
                y_two = comm.all_reduce_(buf)
                torch.cuda.synchronize()
                # (the unfused route runs the same decode kernel for these shapes, so W8A16 sums
                # K in the same order too)
                same = torch.equal(y_fused.view(torch.int16), y_two.view(torch.int16))
                expect_launches = 2 if scheme == "w8a8" else 1   # act-quant + GEMM / GEMM
                if not same or n_fused != expect_launches:
                    ok = False
                    notes.append(f"{scheme} {dtype} M={M}: fused != two-kernel route "
                                 f"(launches {n_fused}), "
                                 f"{O.tensor_metrics(y_two.float().cpu(), y_fused.float().cpu())}")
                # every rank holds the same bits
                gathered = [torch.empty_like(y_fused) for _ in range(world)]
                dist.all_gather(gathered, y_fused.contiguous())
                if not all(torch.equal(g.view(torch.int16), y_fused.view(torch.int16)) for g in gathered):
                    ok = False
                    notes.append(f"{scheme} M={M}: ranks disagree")
                bias_cpu = layer.bias.data.cpu() if with_bias else None
                if scheme == "w8a8":
                    # per-rank oracle partials (bias on every rank, as the reference's quantized
                    # row-parallel layers do), summed in fp32 in rank order: bit-exact
                    ref = torch.zeros(M, N)
                    for r in range(world):
                        xq_r, as_r = O.quantize_per_row_dynamic(x.chunk(world, dim=1)[r].contiguous())
                        acc = O.w8a8_int32_accumulators(xq_r, q.chunk(world, dim=1)[r].contiguous())
                        ref += O.w8a8_native_epilogue(acc, as_r, s, bias_cpu, dtype).float()
                    if not torch.equal(ref.to(dtype).view(torch.int16), y_fused.cpu().view(torch.int16)):
                        ok = False
                        notes.append(f"w8a8 {dtype} M={M}: differs from the oracle's rank-ordered sum")
                else:
                    ref = O.w8a16_dequant_matmul(x, q, s, None).float()
                    if with_bias:
                        ref = ref + world * bias_cpu.float()
                    m = O.tensor_metrics(ref, y_fused)
                    if m["relative_l2"] > 1e-2 or m["cosine_similarity"] < 0.9999:
                        ok = False
                        notes.append(f"int8 {dtype} M={M}: far from the oracle {m}")
        ok = ok and _lib.lib().b200q_device_status() == 0
        # shapes the fused kernels do not take fall back to the two-kernel route
        x_big = O.make_activation(96, K, seed=3).to(dtype).chunk(world, dim=1)[rank].contiguous().cuda()
        y_big = layer(x_big)
        ok = ok and tuple(y_big.shape) == (96, N)
        # timing, decode step of a 1024-wide model: fused vs GEMM + peer all-reduce vs GEMM + NCCL
        K = 1024 * world
        q, s = O.make_weight(1024, K, seed=22)
        torch.set_default_dtype(torch.bfloat16)
        with torch.device("cuda"):
            layer = LL.RowParallelLinear(K, 1024, quantization="w8a8")
        torch.set_default_dtype(prev)
        layer.qweight.weight_loader(layer.qweight, q)
        layer.w_scales.weight_loader(layer.w_scales, s)
        x_local = O.make_activation(16, K, seed=1).chunk(world, dim=1)[rank].contiguous().cuda()
        x_q, a_s = layer.quant_method.quantize_activation(x_local)

        def fused():
            return comm.fused_w8a8(x_q, a_s, layer.qweight, layer.w_scales, None, torch.bfloat16)

        from tiny_vllm_b200.quantization.cuda import apply_w8a8_linear
        buf = comm.buffer((16, 1024), torch.bfloat16)

        def two_kernel():
            buf.copy_(apply_w8a8_linear(x_q, a_s, layer.qweight, layer.w_scales, None, torch.bfloat16))
            return comm.all_reduce_(buf)

        def nccl():
            y = apply_w8a8_linear(x_q, a_s, layer.qweight, layer.w_scales, None, torch.bfloat16)
            dist.all_reduce(y)
            return y

        for fn, name in ((fused, "fused"), (two_kernel, "gemm + peer all-reduce"), (nccl, "gemm + nccl")):
            notes.append(f"decode M=16 N=1024 K/rank=1024 {name}: {_graph_time_us(fn):.1f} us")
        ok = ok and _lib.lib().b200q_device_status() == 0
        LL.set_tp_all_reduce(None)
    except Exception as exc:  # noqa: BLE001
        import traceback
        ok = False
        notes.append(traceback.format_exc())
    torch.save({"ok": ok, "notes": notes}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _tiled_worker(rank, world, port, out_dir):
    """Prefill-sized row-parallel W8A8 layers: GEMM with the reduce-scatter in its epilogue +
    sum-and-gather kernel, against GEMM + two-shot all-reduce and the CPU oracle."""
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import tiny_vllm_b200  # noqa: F401
    from oracle import quant_linear_oracle as O
    from tiny_vllm_b200 import _lib
    from tiny_vllm_b200.layers import linear as LL
    from tiny_vllm_b200.layers.tp_comm import PeerAllReduce
    from tiny_vllm_b200.quantization.cuda import apply_w8a8_linear
    ok, notes = True, []
    try:
        comm = PeerAllReduce(max_bytes=16 << 20, slots=2, tiled_prefill=True)
        LL.set_tp_all_reduce(comm)
        for dtype, M, N, K_local, with_bias in ((torch.bfloat16, 1024, 1024, 512, False),
                                                (torch.float16, 2048, 384, 256, True),
                                                (torch.bfloat16, 4096, 1000, 1024, False),
                                                (torch.bfloat16, 1024, 1024, 512, False)):
            K = K_local * world
            M = -(-M // (world * 256)) * (world * 256)   # the route takes whole 256-row tiles per rank
            q, s = O.make_weight(N, K, seed=41)
            prev = torch.get_default_dtype()
            torch.set_default_dtype(dtype)
            with torch.device("cuda"):
                layer = LL.RowParallelLinear(K, N, bias=with_bias, quantization="w8a8")
            torch.set_default_dtype(prev)
            layer.qweight.weight_loader(layer.qweight, q)
            layer.w_scales.weight_loader(layer.w_scales, s)
            if with_bias:
                g = torch.Generator(device="cpu").manual_seed(5)
                layer.bias.data.copy_(torch.randn(N, generator=g).to(dtype))
            x = O.make_activation(M, K, seed=60 + N).to(dtype)
            x_local = x.chunk(world, dim=1)[rank].contiguous().cuda()
            assert comm.tiled_fits(M, N)
            for rep in range(2):
                y_fused = layer(x_local).clone()
                x_q, a_s = layer.quant_method.quantize_activation(x_local)
                part = apply_w8a8_linear(x_q, a_s, layer.qweight, layer.w_scales,
                                         layer.bias, out_dtype=dtype)
                buf = comm.buffer(part.shape, part.dtype)
                buf.copy_(part)
                y_two = comm.all_reduce_(buf).clone()
                torch.cuda.synchronize()
                if not torch.equal(y_fused.view(torch.int16), y_two.view(torch.int16)):
                    ok = False
                    bad = (y_fused.view(torch.int16) != y_two.view(torch.int16))
                    rows = bad.any(dim=1).nonzero().flatten()
                    notes.append(f"{dtype} M={M} N={N} rep {rep}: fused != two-kernel route, "
                                 f"{int(bad.sum())} values in rows {rows[:4].tolist()}..{rows[-1:].tolist()}")
            gathered = [torch.empty_like(y_fused) for _ in range(world)]
            dist.all_gather(gathered, y_fused.contiguous())
            if not all(torch.equal(g.view(torch.int16), y_fused.view(torch.int16)) for g in gathered):
                ok = False
                notes.append(f"M={M} N={N}: ranks disagree")
            if M <= 2048:
                bias_cpu = layer.bias.data.cpu() if with_bias else None
                ref = torch.zeros(M, N)
                for r in range(world):
                    xq_r, as_r = O.quantize_per_row_dynamic(x.chunk(world, dim=1)[r].contiguous())
                    acc = O.w8a8_int32_accumulators(xq_r, q.chunk(world, dim=1)[r].contiguous())
                    ref += O.w8a8_native_epilogue(acc, as_r, s, bias_cpu, dtype).float()
                if not torch.equal(ref.to(dtype).view(torch.int16), y_fused.cpu().view(torch.int16)):
                    ok = False
                    notes.append(f"{dtype} M={M} N={N}: differs from the oracle's rank-ordered sum")
        ok = ok and _lib.lib().b200q_device_status() == 0
        # timing at the bench shape: o_proj of Qwen3-0.6B, 8192 tokens
        M, N, K = 8192, 1024, 2048
        q, s = O.make_weight(N, K, seed=42)
        torch.set_default_dtype(torch.bfloat16)
        with torch.device("cuda"):
            layer = LL.RowParallelLinear(K, N, quantization="w8a8")
        torch.set_default_dtype(prev)
        layer.qweight.weight_loader(layer.qweight, q)
        layer.w_scales.weight_loader(layer.w_scales, s)
        x_local = O.make_activation(M, K, seed=2).chunk(world, dim=1)[rank].contiguous().cuda()
        x_q, a_s = layer.quant_method.quantize_activation(x_local)
        buf = comm.buffer((M, N), torch.bfloat16)
        y_plain = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")

        def fused():
            return comm.fused_w8a8_tiled(x_q, a_s, layer.qweight, layer.w_scales, None, torch.bfloat16)

        def gemm_only():
            return apply_w8a8_linear(x_q, a_s, layer.qweight, layer.w_scales, None, torch.bfloat16)

        def two_shot():
            comm.all_reduce_(buf)

        def nccl():
            dist.all_reduce(y_plain)

        for fn, name in ((fused, "fused GEMM + reduce-scatter + gather"), (gemm_only, "GEMM alone"),
                         (two_shot, "two-shot all-reduce alone"), (nccl, "NCCL all-reduce alone")):
            notes.append(f"o_proj M=8192 tp={world} {name}: {_graph_time_us(fn, reps=10):.1f} us")
        ok = ok and _lib.lib().b200q_device_status() == 0
        LL.set_tp_all_reduce(None)
    except Exception:  # noqa: BLE001
        import traceback
        ok = False
        notes.append(traceback.format_exc())
    torch.save({"ok": ok, "notes": notes}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _exchange_worker(rank, world, port, out_dir):
    """Fused exchange (reduce + residual add + RMSNorm + quantise + gather of codes) against the
    two-kernel route all-reduce -> b200q_add_rmsnorm_quant_i8, then the chain a layer runs:
    row-parallel W8A8 GEMM -> exchange -> column-parallel W8A8 GEMM on the gathered codes."""
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
    from tiny_vllm_b200.quantization.cuda import add_rmsnorm_quantize_int8
    ok, notes = True, []
    try:
        comm = PeerAllReduce(max_bytes=16 << 20)
        for call, (M, K, dtype, with_res) in enumerate([(8192, 1024, torch.bfloat16, True),
                                                        (64, 1024, torch.bfloat16, True),
                                                        (8 * world, 2048, torch.float16, False),
                                                        (8192, 1024, torch.bfloat16, True)]):
            g = torch.Generator().manual_seed(900 + call)
            parts = [(torch.randn(M, K, generator=g) * 1.5).to(dtype) for _ in range(world)]
            residual = (torch.randn(M, K, generator=g) * 2).to(dtype) if with_res else None
            weight = (1.0 + 0.2 * torch.randn(K, generator=g)).to(dtype).cuda()
            rows = M // world
            # two-kernel route
            t = comm.buffer((M, K), dtype)
            t.copy_(parts[rank])
            comm.all_reduce_(t)
            want_q, want_s, want_res, _ = add_rmsnorm_quantize_int8(
                t, weight, 1e-6, None if residual is None else residual.cuda())
            want_q, want_s = want_q.clone(), want_s.clone()
            # fused route
            t2 = comm.buffer((M, K), dtype)
            t2.copy_(parts[rank])
            res_shard = None if residual is None else residual[rank * rows:(rank + 1) * rows].contiguous().cuda()
            xq, a_s, new_res, _ = comm.reduce_rmsnorm_quant(t2, weight, 1e-6, res_shard)
            torch.cuda.synchronize()
            same = torch.equal(xq, want_q) and torch.equal(a_s, want_s)
            if with_res:
                same = same and torch.equal(new_res.view(torch.int16),
                                            want_res[rank * rows:(rank + 1) * rows].view(torch.int16))
            ok = ok and same
            if not same:
                notes.append(f"exchange call {call} (M={M} K={K}): differs from all-reduce + norm + quant")
        ok = ok and _lib.lib().b200q_device_status() == 0
        # timing at the benchmark's size: fused exchange vs all-reduce + add-RMSNorm + quant
        M, K = 8192, 1024
        bufs = [comm.buffer((M, K), torch.bfloat16) for _ in range(2)]
        for b in bufs:
            b.normal_()
        w = torch.ones(K, dtype=torch.bfloat16, device="cuda")
        res = torch.zeros(M // world, K, dtype=torch.bfloat16, device="cuda")
        res_full = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")
        turn = [0]

        def fused():
            turn[0] ^= 1
            comm.reduce_rmsnorm_quant(bufs[turn[0]], w, 1e-6, res)

        def two_kernels():
            turn[0] ^= 1
            y = comm.large_(bufs[turn[0]])
            add_rmsnorm_quantize_int8(y, w, 1e-6, res_full)

        for fn, name in ((fused, "fused exchange"), (two_kernels, "all-reduce + add-RMSNorm + quant")):
            notes.append(f"8192 x 1024 tp={world} {name}: {_graph_time_us(fn, reps=10):.1f} us")
        ok = ok and _lib.lib().b200q_device_status() == 0
    except Exception:  # noqa: BLE001
        import traceback
        ok = False
        notes.append(traceback.format_exc())
    torch.save({"ok": ok, "notes": notes}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _report(tmp_path, world, name):
    """Asserts every rank's verdict; the ranks' notes (timings, routes taken) are appended to a
    log in the directory B200Q_TEST_LOG_DIR names, when it is set."""
    lines = []
    for r in range(world):
        res = torch.load(tmp_path / f"r{r}.pt")
        print(r, res["notes"])
        lines.append(f"{name} world={world} rank={r} ok={res['ok']}: " + " | ".join(str(n) for n in res["notes"]))
    out = os.environ.get("B200Q_TEST_LOG_DIR")
    if out and Path(out).is_dir():
        with open(Path(out) / f"tp_tests_world{world}.log", "a") as f:
            f.write("\n".join(lines) + "\n")
    for r in range(world):
        res = torch.load(tmp_path / f"r{r}.pt")
        assert res["ok"], res["notes"]


def test_fused_exchange_matches_allreduce_then_norm_quant(tmp_path):
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mp.spawn(_exchange_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    _report(tmp_path, world, "exchange")


def test_fused_row_parallel_prefill_matches_two_kernel_route(tmp_path):
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mp.spawn(_tiled_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    _report(tmp_path, world, "tiled")


def test_fused_row_parallel_decode_matches_two_kernel_route(tmp_path):
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mp.spawn(_fused_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    _report(tmp_path, world, "fused_decode")


def test_peer_all_reduce_matches_rank_ordered_fp32_sum(tmp_path):
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    _report(tmp_path, world, "allreduce")

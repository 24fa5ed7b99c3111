"""Benchmark of the quantized-linear hot path on B200.

Workload (N = 1): the W8A8 prefill sweep — M = 8192 tokens through the four
Qwen3-0.6B projections (qkv 1024->4096, o 2048->1024, gate_up 1024->6144,
down 3072->1024).  One step = for each projection: per-token activation
quantisation (bf16 -> int8 + scale) followed by the int8 GEMM with the fused scale
epilogue (bf16 out).  Inputs are seeded synthetic tensors (N(0,1) activations with
1 % outlier channels x20, N(0,0.02) weights quantised per channel).

With --gpus N > 1 (launched by torchrun, one rank per GPU) the same 8192 tokens run
tensor-parallel: qkv / gate_up split their output channels, o / down split their input
features and are followed by an NCCL all-reduce of the bf16 result ("strong" scaling).

Prints ONE JSON line (rank 0).  ``value`` is device-timed with inputs resident in HBM;
``e2e`` goes through the layer API with host buffers (H2D of activations, D2H of
outputs inside the timed region); ``roofline`` is for the GEMM kernel, from CUDA-event
durations of its launches inside the timed region; ``cpu_baseline`` times the CPU
oracle's dequantize-then-matmul path on the host cores.

``--impl reference`` times the reference's CPU algorithm (the oracle port of its
dequantize-then-matmul path) on the host cores for the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

TOKENS = 8192
# name, K (in features), N (out features), tensor-parallel split: "col" splits N, "row" splits K
PROJECTIONS = [("qkv", 1024, 4096, "col"), ("o", 2048, 1024, "row"),
               ("gate_up", 1024, 6144, "col"), ("down", 3072, 1024, "row")]
METRIC = "quant GEMM TOPS (W8A8 prefill sweep: act-quant + int8 GEMM, M=8192, Qwen3-0.6B qkv/o/gate_up/down)"


def total_ops(tokens: int = TOKENS) -> float:
    return float(sum(2 * tokens * k * n for _, k, n, _ in PROJECTIONS))


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"],
                "bf16_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------- CPU arm
def cpu_problems(tokens: int):
    """Seeded inputs of the four projections for ``tokens`` tokens (made outside any timing)."""
    from oracle import quant_linear_oracle as O
    problems = []
    for i, (_, K, N, _) in enumerate(PROJECTIONS):
        q, s = O.make_weight(N, K, seed=i)
        x = O.make_activation(tokens, K, seed=i)
        problems.append((x, q, s))
    return problems


def cpu_sweep_once(problems) -> float:
    """Wall time of one pass of the CPU oracle's W8A8 path (per-token quantise, then dequantise
    both operands and matmul) over the four projections."""
    from oracle import quant_linear_oracle as O
    t0 = time.perf_counter()
    for x, q, s in problems:
        xf = x.float()
        a_s = (xf.abs().amax(dim=1) / 127.0).clamp_min(1e-8)
        xq = torch.round(xf / a_s[:, None]).clamp(-127, 127).to(torch.int8)
        O.w8a8_dequant_matmul(xq, a_s, q, s, None, torch.bfloat16)
    return time.perf_counter() - t0


def cpu_sweep_seconds(tokens: int, repeats: int):
    """Best-of-``repeats`` wall time of one pass for ``tokens`` tokens."""
    problems = cpu_problems(tokens)
    return min(cpu_sweep_once(problems) for _ in range(repeats))


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs are meant to use every host core."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_baseline(budget_s: float = 20.0):
    threads = use_all_host_threads()
    probe_tokens = 256
    t_probe = cpu_sweep_seconds(probe_tokens, 1)
    per_token = t_probe / probe_tokens
    tokens = int(min(TOKENS, max(256, (budget_s / 3.0) / per_token)))
    tokens = max(256, tokens // 256 * 256)
    t = cpu_sweep_seconds(tokens, 3)
    return {"value": total_ops(tokens) / t / 1e12, "unit": "TOPS", "cores": threads, "kind": "port",
            "sample": f"{tokens} of {TOKENS} tokens through all four projections, best of 3 passes, "
                      f"torch CPU bf16 dequantize-then-matmul (oracle port), {threads} threads of "
                      f"{os.cpu_count()} logical CPUs",
            "seconds": t}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = use_all_host_threads()
    t_probe = cpu_sweep_seconds(256, 1)
    tokens = int(min(TOKENS, max(256, 1.5 / (t_probe / 256))))  # about 1.5 s per step at most
    tokens = max(256, tokens // 256 * 256)
    problems = cpu_problems(tokens)          # inputs are made once, outside the timed steps
    for _ in range(max(0, min(args.warmup, 3))):
        cpu_sweep_once(problems)
    steps = max(1, min(args.steps, 20))
    dt = sum(cpu_sweep_once(problems) for _ in range(steps)) / steps
    value = total_ops(tokens) / dt / 1e12
    sample = (f"{tokens} of {TOKENS} tokens per step, {steps} timed steps, torch CPU bf16 "
              f"dequantize-then-matmul (oracle port of the reference's Python path)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "configs[1] W8A8 prefill sweep, CPU sample", "tokens": tokens,
                   "parallelism": "cpu"},
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------- GPU arm
class GraphEventTimer:
    """CUDA events that can be recorded inside a captured graph and read from outside
    (cudaEventRecordWithFlags + cudaEventRecordExternal): torch's own events become plain
    dependency edges when recorded during capture and carry no time stamp."""

    def __init__(self):
        import ctypes
        self._c = ctypes
        self._rt = ctypes.CDLL("libcudart.so.12")
        self._rt.cudaEventCreate.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        self._rt.cudaEventRecordWithFlags.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint]
        self._rt.cudaEventElapsedTime.argtypes = [ctypes.POINTER(ctypes.c_float), ctypes.c_void_p,
                                                  ctypes.c_void_p]

    def record(self, stream: int):
        ev = self._c.c_void_p()
        rc = self._rt.cudaEventCreate(self._c.byref(ev))
        if rc == 0:
            rc = self._rt.cudaEventRecordWithFlags(ev, self._c.c_void_p(stream), 1)  # external
        if rc != 0:
            raise RuntimeError(f"cudaEventRecordWithFlags failed with CUDA error {rc}")
        return ev

    def elapsed_ms(self, start, stop) -> float:
        out = self._c.c_float()
        rc = self._rt.cudaEventElapsedTime(self._c.byref(out), start, stop)
        if rc != 0:
            raise RuntimeError(f"cudaEventElapsedTime failed with CUDA error {rc}")
        return float(out.value)


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": max(mx),
                "power_w": statistics.median(pw) if pw else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def run_gpu_arm(args):
    import torch.distributed as dist

    import tiny_vllm_b200  # noqa: F401
    from oracle import quant_linear_oracle as O
    from tiny_vllm_b200 import _lib
    from tiny_vllm_b200.layers import linear as LL

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback of the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tp = world
    comm = None
    if tp > 1 and not args.nccl_allreduce:
        # partial outputs of the row-parallel layers live in symmetric memory and are summed
        # in place over NVLink by b200q_tp_allreduce (one slot per row-parallel layer)
        from tiny_vllm_b200.layers.tp_comm import PeerAllReduce
        try:
            comm = PeerAllReduce(max_bytes=TOKENS * 1024 * 2, slots=2)
            made = 1
        except Exception as exc:  # symmetric memory not available on this box
            print(f"[bench] rank {rank}: peer all-reduce unavailable ({exc!r}); using NCCL", file=sys.stderr)
            comm, made = None, 0
        agree = torch.tensor([made], device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)     # all ranks take the same route
        if int(agree.item()) == 0:
            comm = None
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream

    # ---- layers (public API) and raw buffers (kernel-only loop), per-rank shapes
    prev_dtype = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    layers, work = [], []
    for i, (name, K, N, split) in enumerate(PROJECTIONS):
        q_full, s_full = O.make_weight(N, K, seed=i)
        x_full = O.make_activation(TOKENS, K, seed=i)
        with torch.device(dev):
            if name == "qkv":
                layer = LL.QKVParallelLinear(K, 128, 16, 8, quantization="w8a8")
            elif name == "gate_up":
                layer = LL.MergedColumnParallelLinear(K, [N // 2, N // 2], quantization="w8a8")
            else:
                layer = LL.RowParallelLinear(K, N, quantization="w8a8")
        layer.qweight.weight_loader(layer.qweight, q_full)
        layer.w_scales.weight_loader(layer.w_scales, s_full)
        x_local = x_full if split == "col" else x_full.chunk(tp, dim=1)[rank].contiguous()
        layers.append(layer)
        n_loc, k_loc = layer.qweight.shape
        work.append({
            "name": name, "split": split, "K": k_loc, "N": n_loc,
            "x_host": x_local.pin_memory(), "x": x_local.to(dev),
            "xq": torch.empty(TOKENS, k_loc, dtype=torch.int8, device=dev),
            "a_s": torch.empty(TOKENS, dtype=torch.float32, device=dev),
            "y": (comm.buffer((TOKENS, n_loc), torch.bfloat16) if (comm is not None and split == "row")
                  else torch.empty(TOKENS, n_loc, dtype=torch.bfloat16, device=dev)),
            "y_host": torch.empty(TOKENS, n_loc, dtype=torch.bfloat16, device="cpu").pin_memory(),
            "layer": layer, "ops": 2.0 * TOKENS * k_loc * n_loc,
        })
    torch.set_default_dtype(prev_dtype)
    ws_bytes = max([L.b200q_workspace_bytes(_lib.OP_W8A8, TOKENS, w["N"], w["K"]) for w in work] + [16])
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)

    def kernel_step(events=None):
        """One pass of the hot path.  ``events``: optional list that receives torch events
        around every GEMM (eager launches only)."""
        stream = torch.cuda.current_stream().cuda_stream     # the capture stream while capturing
        for w in work:
            rc = L.b200q_act_quant_i8(w["x"].data_ptr(), w["K"], _lib.DTYPE_BF16, w["xq"].data_ptr(),
                                      w["a_s"].data_ptr(), TOKENS, w["K"], stream)
            _lib.check(rc, "b200q_act_quant_i8")
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record()
            rc = L.b200q_w8a8_gemm(w["xq"].data_ptr(), w["a_s"].data_ptr(), w["layer"].qweight.data_ptr(),
                                   w["layer"].w_scales.data_ptr(), None, w["y"].data_ptr(), TOKENS,
                                   w["N"], w["K"], _lib.DTYPE_BF16, ws.data_ptr(), ws.numel(), stream)
            _lib.check(rc, "b200q_w8a8_gemm")
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                events.append((w["name"], e0, e1))
            if w["split"] == "row" and tp > 1:
                if comm is not None:
                    comm.large_(w["y"])     # pull kernel for two ranks, two-shot beyond
                else:
                    dist.all_reduce(w["y"])

    # End-to-end step: pinned host activations -> device -> layer API -> pinned host outputs.
    # Uploads, compute and downloads run on three streams so that the two copy engines and
    # the SMs work at the same time.  Steps are pipelined like batches of a server: step i may
    # start uploading while step i - 1 is still downloading; at most two steps are in flight
    # (two pinned output buffers per projection), and the run ends when the last output is
    # back on the host.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    s_main = torch.cuda.current_stream(dev)
    for w in work:
        w["y_hosts"] = [w["y_host"], torch.empty_like(w["y_host"]).pin_memory()]
    in_flight = []

    def e2e_step(i):
        if len(in_flight) >= 2:
            in_flight.pop(0).synchronize()       # step i - 2 is back on the host: its buffers are free
        for w in work:
            with torch.cuda.stream(s_in):
                x = w["x_host"].to(dev, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            s_main.wait_event(ready)
            x.record_stream(s_main)
            y = w["layer"](x)                       # act-quant + GEMM (+ all-reduce) via the layer API
            done = torch.cuda.Event()
            done.record(s_main)
            s_out.wait_event(done)
            y.record_stream(s_out)
            with torch.cuda.stream(s_out):
                w["y_hosts"][i % 2].copy_(y, non_blocking=True)
        finished = torch.cuda.Event()
        finished.record(s_out)
        in_flight.append(finished)

    def sync_all():
        torch.cuda.synchronize()
        if tp > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- warm-up
    for _ in range(max(3, args.warmup)):
        kernel_step()
    sync_all()
    if L.b200q_device_status() != 0:
        raise SystemExit("device status word set during warm-up: a bounded wait gave up")

    # ---- capture: one CUDA graph per step, so that the timed region holds no host launch
    # overhead and no event records (an event record between two kernels costs about 4 us of
    # idle GPU per boundary here, 35 us per step)
    step_graph, per_graph = None, 0
    # (NCCL collectives stay out of graph capture: with the NCCL route the step is launched
    # from the host, kernel by kernel)
    if not args.no_graph and (tp == 1 or comm is not None):
        step_graph = torch.cuda.CUDAGraph()
        before = L.b200q_launch_count()
        with torch.cuda.graph(step_graph):
            kernel_step()
        per_graph = L.b200q_launch_count() - before
        for _ in range(3):
            step_graph.replay()
        sync_all()

    # ---- timed region (device time, inputs resident in HBM)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = L.b200q_launch_count()
    events = []
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    t_start.record()
    if step_graph is not None:
        for _ in range(args.steps):
            step_graph.replay()
    else:
        for _ in range(args.steps):
            kernel_step()
    t_end.record()
    sync_all()
    elapsed_ms = t_start.elapsed_time(t_end)
    launches = per_graph * args.steps if step_graph is not None else L.b200q_launch_count() - launches0
    clocks = sampler.stop() if sampler is not None else None
    if tp > 1:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    full_ops = total_ops()
    value = full_ops / (ms_per_step * 1e-3) / 1e12

    # ---- per-kernel durations, right after the timed region: every kernel of the step is
    # replayed as a graph of REPS back-to-back launches bracketed by two event nodes, so that
    # the cost of the event records is spread over REPS launches
    REPS, ROUNDS = 8, 6
    rt = GraphEventTimer()

    def batch_us(launch_one):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            cs = torch.cuda.current_stream().cuda_stream
            m0 = rt.record(cs)
            for _ in range(REPS):
                launch_one(cs)
            m1 = rt.record(cs)
        g.replay()
        torch.cuda.synchronize()
        samples = []
        for _ in range(ROUNDS):
            g.replay()
            torch.cuda.synchronize()
            samples.append(rt.elapsed_ms(m0, m1) * 1e3 / REPS)
        return sum(samples) / len(samples)

    per_shape, aq_us = {}, {}
    for w in work:
        def one_gemm(cs, w=w):
            _lib.check(L.b200q_w8a8_gemm(
                w["xq"].data_ptr(), w["a_s"].data_ptr(), w["layer"].qweight.data_ptr(),
                w["layer"].w_scales.data_ptr(), None, w["y"].data_ptr(), TOKENS, w["N"], w["K"],
                _lib.DTYPE_BF16, ws.data_ptr(), ws.numel(), cs), "b200q_w8a8_gemm")

        # the quantiser reads its input from HBM inside a step (nothing of x survives a step's
        # 450 MB in L2), so its launches here rotate over REPS distinct copies of x
        x_copies = [w["x"]] + [w["x"].clone() for _ in range(REPS - 1)]
        turn = [0]

        def one_quant(cs, w=w, x_copies=x_copies, turn=turn):
            x = x_copies[turn[0] % REPS]
            turn[0] += 1
            _lib.check(L.b200q_act_quant_i8(x.data_ptr(), w["K"], _lib.DTYPE_BF16,
                                            w["xq"].data_ptr(), w["a_s"].data_ptr(), TOKENS, w["K"], cs),
                       "b200q_act_quant_i8")

        per_shape[w["name"]] = [batch_us(one_gemm) * 1e-3]
        aq_us[w["name"]] = batch_us(one_quant)
        del x_copies
    sync_all()
    gemm_ms_total, gemm_ops_total = 0.0, 0.0
    ops_of = {w["name"]: w["ops"] for w in work}
    bytes_of = {w["name"]: TOKENS * w["K"] + w["N"] * w["K"] + 4 * TOKENS + 4 * w["N"] + 2 * TOKENS * w["N"]
                for w in work}
    detail = {}
    for name, ms in per_shape.items():
        avg = sum(ms) / len(ms)
        gemm_ms_total += sum(ms)
        gemm_ops_total += ops_of[name] * len(ms)
        detail[name] = {"gemm_us": avg * 1e3, "gemm_tops": ops_of[name] / (avg * 1e-3) / 1e12,
                        "gemm_algorithmic_gbs": bytes_of[name] / (avg * 1e-3) / 1e9}
    peaks = load_peaks()
    int8_peak = 2.0 * peaks["bf16_sustained"]
    achieved = gemm_ops_total / (gemm_ms_total * 1e-3) / 1e12
    # DRAM bytes per launch from the ncu capture summarised in
    # profiles/w8a8_umma_pair_kernel_prefill_sweep_m8192.md (mean of the four shapes, TP=1 only)
    traffic = 127.1e6 / 4 if world == 1 else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                "frac": achieved / int8_peak, "traffic": traffic,
                "traffic_note": "dram__bytes_read+write per launch, mean over the 4 shapes; algorithmic "
                                "mean is 66.6 MB, the difference is output still dirty in L2 at kernel end",
                "timing": f"CUDA event nodes around graphs of {REPS} back-to-back launches of each GEMM, "
                          f"{ROUNDS} replays, taken right after the timed region (event records between "
                          "the kernels of a step would add about 4 us of idle GPU per boundary); "
                          "achieved = ops of the four GEMMs / sum of their durations",
                "kernel": "w8a8_umma_pair_kernel (tcgen05 cta_group::2 kind::i8)" if world == 1 else "w8a8_umma kernels (tcgen05 kind::i8)",
                "peak_note": f"2 x {peaks['source']} sustained bf16 dense TFLOP/s ({peaks['bf16_sustained']}); "
                             "int8 is the double-rate kind; nominal 4500"}

    # ---- end-to-end through the layer API with host buffers
    e2e_steps = max(3, min(args.steps, 20))
    for i in range(2):
        e2e_step(i)
    sync_all()
    in_flight.clear()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    sync_all()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    if tp > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    h2d = sum(w["x_host"].numel() * 2 for w in work)
    d2h = sum(w["y_host"].numel() * 2 for w in work)
    e2e = {"value": full_ops / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
           "pipelining": "at most two steps in flight (upload of step i overlaps download of step i - 1); "
                         "wall clock from the first upload to the last byte back on the host"}

    status = L.b200q_device_status()
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "configs[1]: W8A8 prefill GEMM sweep, M=8192, Qwen3-0.6B projections "
                                   "(qkv 1024->4096, o 2048->1024, gate_up 1024->6144, down 3072->1024)",
                       "tokens": TOKENS, "parallelism": f"tp{world}",
                       "allreduce": ("none" if world == 1 else
                                     ("b200q_tp_allreduce_pull (peer memory)" if world == 2 else "b200q_tp_allreduce (peer memory)") if comm is not None else "nccl"),
                       "launch": ("one CUDA graph replay per step (act-quant + GEMM x 4, plus the "
                                  "all-reduces at tp > 1)" if step_graph is not None
                                  else "eager launches through the C ABI"),
                       "l2": "no flush: one step touches about 450 MB (activations, int8 copies, outputs), "
                             "more than the 126 MB L2"},
            "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "device_status": status, "detail": detail,
            "step_breakdown_us": {"step": ms_per_step * 1e3,
                                  "gemm_sum": sum(v["gemm_us"] for v in detail.values()),
                                  "act_quant_sum": sum(aq_us.values()), "act_quant": aq_us},
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line))
    if tp > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_shape_sweep(args):
    """Secondary tables (not the headline line): per-shape kernel times for the decode shapes
    M in {1, 16, 128, 512} and the prefill shape M = 8192 of both GEMM kinds and for the
    activation quantiser.  Launches are replayed from a CUDA graph (no host overhead in the
    numbers) over rotating buffers larger than L2.  Prints one JSON line."""
    import tiny_vllm_b200  # noqa: F401
    from tiny_vllm_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200)")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    L = _lib.lib()
    ws = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    peaks = load_peaks()

    def time_op(op, M, N, K, iters):
        nbuf = max(2, min(16, int(300e6 // max(1, N * K + 2 * M * N)) + 1))
        xq = [torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev) for _ in range(nbuf)]
        xb = [torch.randn(M, K, dtype=torch.bfloat16, device=dev) for _ in range(nbuf)]
        wq = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(nbuf)]
        a_s = torch.rand(M, device=dev)
        w_s = torch.rand(N, device=dev)
        y = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(nbuf)]
        res = [torch.randn(M, K, dtype=torch.bfloat16, device=dev) for _ in range(nbuf)] \
            if op == "add_rmsnorm_quant" else None
        gu = [torch.randn(M, 2 * K, dtype=torch.bfloat16, device=dev) for _ in range(nbuf)] \
            if op == "silu_mul_quant" else None
        norm_w = torch.ones(K, dtype=torch.bfloat16, device=dev)
        side = torch.cuda.Stream(device=dev)

        def call(i, st):
            j = i % nbuf
            if op == "w8a8":
                rc = L.b200q_w8a8_gemm(xq[j].data_ptr(), a_s.data_ptr(), wq[j].data_ptr(), w_s.data_ptr(),
                                       None, y[j].data_ptr(), M, N, K, _lib.DTYPE_BF16, ws.data_ptr(),
                                       ws.numel(), st)
            elif op == "w8a16":
                rc = L.b200q_w8a16_gemm(xb[j].data_ptr(), wq[j].data_ptr(), w_s.data_ptr(), None,
                                        y[j].data_ptr(), M, N, K, _lib.DTYPE_BF16, ws.data_ptr(),
                                        ws.numel(), st)
            elif op == "act_quant":
                rc = L.b200q_act_quant_i8(xb[j].data_ptr(), K, _lib.DTYPE_BF16, xq[j].data_ptr(),
                                          a_s.data_ptr(), M, K, st)
            elif op == "add_rmsnorm_quant":   # x + residual -> new residual (in place), codes
                rc = L.b200q_add_rmsnorm_quant_i8(xb[j].data_ptr(), res[j].data_ptr(), norm_w.data_ptr(),
                                                  1e-6, res[j].data_ptr(), None, xq[j].data_ptr(),
                                                  a_s.data_ptr(), M, K, _lib.DTYPE_BF16, st)
            else:                             # silu_mul_quant: [M, 2 K] -> codes [M, K]
                rc = L.b200q_silu_mul_quant_i8(gu[j].data_ptr(), 2 * K, None, xq[j].data_ptr(),
                                               a_s.data_ptr(), M, K, _lib.DTYPE_BF16, st)
            _lib.check(rc, op)

        for i in range(3):
            call(i, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(iters):
                    call(i, side.cuda_stream)
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / iters

    results = []
    shapes = [(name, n, k) for name, k, n, _ in PROJECTIONS]
    want_ops = args.sweep_op.split(",") if args.sweep_op else ["w8a8", "w8a16", "act_quant", "fused_quant"]
    want_m = [int(m) for m in args.sweep_m.split(",")] if args.sweep_m else [1, 16, 128, 512, TOKENS]
    for op in ("w8a8", "w8a16"):
        if op not in want_ops:
            continue
        for M in want_m:
            for name, N, K in shapes:
                us = time_op(op, M, N, K, 20 if M == TOKENS else 100)
                in_bytes = M * K * (1 if op == "w8a8" else 2)
                alg_bytes = in_bytes + N * K + 4 * N + 2 * M * N + (4 * M if op == "w8a8" else 0)
                ops = 2.0 * M * N * K
                results.append({"op": op, "proj": name, "M": M, "N": N, "K": K, "us": round(us, 2),
                                "tops": round(ops / us / 1e6, 1),
                                "algorithmic_gbs": round(alg_bytes / us / 1e3, 1),
                                "hbm_frac": round(alg_bytes / us / 1e3 / peaks["hbm_gbs"], 3),
                                "path": L.b200q_select_path(_lib.OP_W8A8 if op == "w8a8" else _lib.OP_W8A16,
                                                            M, N, K).decode()})
    for name, N, K in shapes:
        if "act_quant" not in want_ops:
            break
        us = time_op("act_quant", TOKENS, N, K, 50)
        b = 3 * TOKENS * K + 4 * TOKENS
        results.append({"op": "act_quant", "proj": name, "M": TOKENS, "K": K, "us": round(us, 2),
                        "algorithmic_gbs": round(b / us / 1e3, 1),
                        "hbm_frac": round(b / us / 1e3 / peaks["hbm_gbs"], 3)})
    if "fused_quant" in want_ops:
        # quantisation fused into its producers: hidden-size rows (norm) and intermediate-size
        # rows (activation) of Qwen3-0.6B at the prefill token count
        for op, K, per_row in (("add_rmsnorm_quant", 1024, 7 * 1024 + 4), ("silu_mul_quant", 3072, 5 * 3072 + 4)):
            us = time_op(op, TOKENS, 8, K, 50)
            b = per_row * TOKENS
            results.append({"op": op, "M": TOKENS, "K": K, "us": round(us, 2),
                            "algorithmic_gbs": round(b / us / 1e3, 1),
                            "hbm_frac": round(b / us / 1e3 / peaks["hbm_gbs"], 3)})
    print(json.dumps({"mode": "shape_sweep", "peaks": peaks, "device_status": L.b200q_device_status(),
                      "results": results}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel from the host inside the timed region instead of "
                         "replaying one CUDA graph per step")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="sum row-parallel outputs with NCCL instead of the peer-memory kernel")
    ap.add_argument("--sweep-op", default="", help="shape_sweep: comma list of w8a8,w8a16,act_quant,fused_quant")
    ap.add_argument("--sweep-m", default="", help="shape_sweep: comma list of token counts")
    ap.add_argument("--mode", default="headline", choices=["headline", "shape_sweep"],
                    help="shape_sweep prints per-shape kernel times (decode and prefill shapes)")
    args = ap.parse_args()
    if args.mode == "shape_sweep":
        run_shape_sweep(args)
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()

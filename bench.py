"""Benchmark of the quantized-linear hot path on B200.

Workload (N = 1): the W8A8 prefill sweep — M = 8192 tokens through the four
Qwen3-0.6B projections (qkv 1024->4096, o 2048->1024, gate_up 1024->6144,
down 3072->1024).  One step = for each projection: per-token activation
quantisation (bf16 -> int8 + scale) followed by the int8 GEMM with the fused scale
epilogue (bf16 out).  Inputs are seeded synthetic tensors (N(0,1) activations with
1 % outlier channels x20, N(0,0.02) weights quantised per channel).

With --gpus N > 1 (launched by torchrun, one rank per GPU) the same 8192 tokens run
tensor-parallel ("strong" scaling): qkv / gate_up split their output channels, o / down split
their input features, and what follows a row-parallel layer in the model — sum over ranks,
residual add, RMSNorm, quantisation for the next projection — is one fused exchange kernel
over peer memory whose int8 codes feed the next GEMM (``--tp-step allreduce``: plain
all-reduce and a stand-alone quantiser in front of every GEMM instead).  Every N > 1 run checks
the exchange bit for bit against all-gather + rank-ordered sum (``exchange_check``).

Prints ONE JSON line (rank 0).  ``value`` is device-timed with inputs resident in HBM;
``e2e`` goes through the layer API with host buffers (H2D of activations, D2H of
outputs inside the timed region); ``roofline`` is for the GEMM kernel, from CUDA-event
durations of graphs of back-to-back launches taken right after the timed region;
``cpu_baseline`` times the reference's CPU path (or the oracle's port of it) on the host cores;
``detail`` holds the other kernels of the path on the same shapes (W8A16, the library bf16
GEMM, decode batches, the Qwen3-8B shapes, the reference's own CUDA kernels).

``--impl reference`` times the reference's own CPU implementation of the path — its
``quantize_int8_per_row_dynamic`` and ``w8a8_linear_fallback`` from the mirror that
``oracle/build_ref.py`` keeps in ``oracle/_ref`` (kind "reference"), or the oracle's port of
them when no mirror was built (kind "port") — on all host cores, same workload, same steps.
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
WORKLOAD = ("configs[1]: W8A8 prefill GEMM sweep, M=8192, Qwen3-0.6B projections "
            "(qkv 1024->4096, o 2048->1024, gate_up 1024->6144, down 3072->1024)")


def cpu_problems(tokens: int):
    """Seeded inputs of the four projections for ``tokens`` tokens (made outside any timing)."""
    from oracle import quant_linear_oracle as O
    problems = []
    for i, (_, K, N, _) in enumerate(PROJECTIONS):
        q, s = O.make_weight(N, K, seed=i)
        x = O.make_activation(tokens, K, seed=i)
        problems.append((x, q, s))
    return problems


def cpu_path():
    """(quantiser, linear, kind): the reference's own Python functions when oracle/_ref holds
    its mirror, else the oracle's restatement of them."""
    from oracle import build_ref
    ref = build_ref.load_reference()
    if ref is not None:
        return ref.utils.quantize_int8_per_row_dynamic, ref.cuda.w8a8_linear_fallback, "reference"
    from oracle import quant_linear_oracle as O

    def quantise(x):
        xf = x.float()
        a_s = (xf.abs().amax(dim=1) / 127.0).clamp_min(1e-8)
        return torch.round(xf / a_s[:, None]).clamp(-127, 127).to(torch.int8), a_s
    return quantise, O.w8a8_dequant_matmul, "port"


def cpu_sweep_once(problems, quantise, linear) -> float:
    """Wall time of one pass of the reference's CPU W8A8 path (per-token quantise, then
    dequantise both operands and matmul) over the four projections."""
    t0 = time.perf_counter()
    for x, q, s in problems:
        xq, a_s = quantise(x)
        linear(xq, a_s, q, s, None, torch.bfloat16)
    return time.perf_counter() - t0


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs are meant to use every host core."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_description(kind: str, threads: int) -> str:
    what = ("the reference's quantize_int8_per_row_dynamic + w8a8_linear_fallback (oracle/_ref mirror)"
            if kind == "reference" else "oracle port of the reference's dequantize-then-matmul path")
    return f"torch CPU bf16, {what}, {threads} threads of {os.cpu_count()} logical CPUs"


def cpu_baseline():
    """The same workload, all 8192 tokens, on the host cores: best of 3 passes (about 0.1 s each)."""
    threads = use_all_host_threads()
    quantise, linear, kind = cpu_path()
    problems = cpu_problems(TOKENS)
    cpu_sweep_once(problems, quantise, linear)
    t = min(cpu_sweep_once(problems, quantise, linear) for _ in range(3))
    return {"value": total_ops(TOKENS) / t / 1e12, "unit": "TOPS", "cores": threads, "kind": kind,
            "sample": f"{TOKENS} of {TOKENS} tokens through all four projections, best of 3 passes, "
                      + cpu_description(kind, threads),
            "seconds": t}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = use_all_host_threads()
    quantise, linear, kind = cpu_path()
    problems = cpu_problems(TOKENS)          # inputs are made once, outside the timed steps
    for _ in range(max(0, args.warmup)):
        cpu_sweep_once(problems, quantise, linear)
    steps = max(1, args.steps)
    dt = sum(cpu_sweep_once(problems, quantise, linear) for _ in range(steps)) / steps
    value = total_ops(TOKENS) / dt / 1e12
    sample = (f"{TOKENS} of {TOKENS} tokens per step, {steps} timed steps after {max(0, args.warmup)} "
              f"warm-up steps, " + cpu_description(kind, threads))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": steps, "warmup": max(0, args.warmup), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens": TOKENS, "parallelism": f"tp{args.gpus}"},
        "note": "runs on the host cores of rank 0: the reference's CPU path does not use the GPUs, "
                "so the figure is the same at every --gpus",
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": threads, "kind": kind, "sample": sample},
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


def load_traffic(world: int):
    """DRAM bytes per launch of the GEMM kernel (mean of the four shapes) from the figures file
    of the ncu capture kept under profiles/; None when the file is absent or at TP > 1."""
    path = ROOT / "profiles" / "w8a8_umma_pair_kernel_prefill_m8192.traffic.json"
    if world != 1 or not path.exists():
        return None, "no ncu capture on file for this configuration"
    d = json.loads(path.read_text())
    per = [v["dram_bytes_read"] + v["dram_bytes_write"] for v in d["per_shape"].values()]
    return sum(per) / len(per), d["note"]


EIGHT_B = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 24576), ("down", 12288, 4096)]


def extras(detail, work, ws, dev, batch_us, peaks):
    """Per-shape times of the kernels that are not in the timed step.  Same timing method as the
    GEMM figures: event nodes around graphs of back-to-back launches."""
    import tiny_vllm_b200  # noqa: F401
    from tiny_vllm_b200 import _lib
    L = _lib.lib()

    def w8a8(xq, a_s, q, s, y, M, N, K, wsp):
        return lambda cs: _lib.check(L.b200q_w8a8_gemm(
            xq.data_ptr(), a_s.data_ptr(), q.data_ptr(), s.data_ptr(), None, y.data_ptr(), M, N, K,
            _lib.DTYPE_BF16, wsp.data_ptr(), wsp.numel(), cs), "b200q_w8a8_gemm")

    def w8a16(x, q, s, y, M, N, K, wsp):
        return lambda cs: _lib.check(L.b200q_w8a16_gemm(
            x.data_ptr(), q.data_ptr(), s.data_ptr(), None, y.data_ptr(), M, N, K,
            _lib.DTYPE_BF16, wsp.data_ptr(), wsp.numel(), cs), "b200q_w8a16_gemm")

    def library_bf16(x, wt, y):
        # torch.matmul -> the vendor GEMM library, on the capture stream
        return lambda cs: torch.matmul(x, wt, out=y)

    for w in work:
        name, K, N = w["name"], w["K"], w["N"]
        q, s = w["layer"].qweight, w["layer"].w_scales
        ops = 2.0 * TOKENS * N * K
        d = detail[name]
        us = batch_us(w8a16(w["x"], q, s, w["y"], TOKENS, N, K, ws))
        d["w8a16_us"], d["w8a16_tflops"] = us, ops / us / 1e6
        d["w8a16_frac_of_burst_bf16"] = ops / us / 1e6 / peaks["bf16_burst"]
        d["w8a16_path"] = L.b200q_select_path(_lib.OP_W8A16, TOKENS, N, K).decode()
        wt = torch.randn(K, N, dtype=torch.bfloat16, device=dev).t().contiguous().t()   # [K, N] view of an [N, K] matrix
        torch.matmul(w["x"], wt, out=w["y"])
        us = batch_us(library_bf16(w["x"], wt, w["y"]))
        d["library_bf16_us"], d["library_bf16_tflops"] = us, ops / us / 1e6
        d["w8a8_speedup_over_library_bf16"] = us / d["gemm_us"]
        d["w8a16_speedup_over_library_bf16"] = us / d["w8a16_us"]
        del wt
        dec = {}
        for M in (16, 128):
            dec[f"w8a8_m{M}_us"] = batch_us(w8a8(w["xq"], w["a_s"], q, s, w["y"], M, N, K, ws))
            dec[f"w8a16_m{M}_us"] = batch_us(w8a16(w["x"], q, s, w["y"], M, N, K, ws))
        d["decode"] = dec
    detail["summary"] = {
        "w8a8_gemm_sum_us": sum(detail[w["name"]]["gemm_us"] for w in work),
        "w8a16_gemm_sum_us": sum(detail[w["name"]]["w8a16_us"] for w in work),
        "library_bf16_gemm_sum_us": sum(detail[w["name"]]["library_bf16_us"] for w in work),
        "note": "the four projections at 8192 tokens; library_bf16 = torch.matmul on bf16 operands of "
                "the same shapes (the unquantized path the quantized layers replace)"}

    # the larger model's projections at the same token count: long K loops, where the epilogue
    # and the per-launch costs are amortised
    big = {}
    for name, K, N in EIGHT_B:
        ops = 2.0 * TOKENS * N * K
        xq = torch.randint(-127, 128, (TOKENS, K), dtype=torch.int8, device=dev)
        xb = torch.randn(TOKENS, K, dtype=torch.bfloat16, device=dev)
        q = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
        a_s = torch.rand(TOKENS, device=dev)
        s = torch.rand(N, device=dev)
        y = torch.empty(TOKENS, N, dtype=torch.bfloat16, device=dev)
        wsp = torch.zeros(max(16, L.b200q_workspace_bytes(_lib.OP_W8A16, TOKENS, N, K),
                              L.b200q_workspace_bytes(_lib.OP_W8A8, TOKENS, N, K)), dtype=torch.uint8, device=dev)
        t8 = batch_us(w8a8(xq, a_s, q, s, y, TOKENS, N, K, wsp))
        t16 = batch_us(w8a16(xb, q, s, y, TOKENS, N, K, wsp))
        wt = torch.randn(N, K, dtype=torch.bfloat16, device=dev).t()
        torch.matmul(xb, wt, out=y)
        tl = batch_us(library_bf16(xb, wt, y))
        big[name] = {"K": K, "N": N, "w8a8_us": t8, "w8a8_tops": ops / t8 / 1e6,
                     "w8a8_frac_of_2x_burst_bf16": ops / t8 / 1e6 / (2 * peaks["bf16_burst"]),
                     "w8a16_us": t16, "w8a16_tflops": ops / t16 / 1e6,
                     "w8a16_frac_of_burst_bf16": ops / t16 / 1e6 / peaks["bf16_burst"],
                     "library_bf16_us": tl, "library_bf16_tflops": ops / tl / 1e6}
        del xq, xb, q, y, wsp, wt
    detail["qwen3_8b_prefill_m8192"] = big

    # the reference's own CUDA kernels (compiled from its sources into oracle/_ref) on this GPU
    from oracle import build_ref
    ref = build_ref.load_reference(with_cuda_extensions=True)
    if ref is None or not ref.native_w8a8:
        detail["reference_gpu"] = {"unavailable": "oracle/_ref (the reference's package and CUDA "
                                                  "extensions) was not built"}
        return
    rg = {}

    def eager_us(fn, iters=5):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / iters

    step_us = 0.0
    for w in work:
        q, s = w["layer"].qweight, w["layer"].w_scales
        xq, a_s = ref.utils.quantize_int8_per_row_dynamic(w["x"])
        t_q = eager_us(lambda: ref.utils.quantize_int8_per_row_dynamic(w["x"]))
        t_g = eager_us(lambda: ref.cuda.native_w8a8_linear(xq, a_s, q, s, None, torch.bfloat16))
        t_16 = eager_us(lambda: ref.cuda.native_int8_weight_only_linear(w["x"], q, s, None))
        rg[w["name"]] = {"quantize_us": t_q, "w8a8_gemm_us": t_g, "w8a16_gemm_us": t_16,
                         "w8a8_gemm_tops": w["ops"] / t_g / 1e6}
        # the same kernels on a decode batch of 16 tokens (this library: detail.<shape>.decode)
        x16 = w["x"][:16].contiguous()
        xq16, as16 = ref.utils.quantize_int8_per_row_dynamic(x16)
        rg[w["name"]]["decode_m16"] = {
            "w8a8_gemm_us": eager_us(lambda: ref.cuda.native_w8a8_linear(xq16, as16, q, s, None, torch.bfloat16), 20),
            "w8a16_gemm_us": eager_us(lambda: ref.cuda.native_int8_weight_only_linear(x16, q, s, None), 20)}
        step_us += t_q + t_g
    rg["step_us"] = step_us
    rg["step_tops"] = sum(w["ops"] for w in work) / step_us / 1e6
    rg["how"] = ("the reference's quantize_int8_per_row_dynamic (eager torch ops) + native_w8a8_linear "
                 "(its WMMA kernel) per projection, 8192 tokens, host-launched, CUDA events around 5 "
                 "calls; compiled from the reference's sources for sm_100a by oracle/build_ref.py")
    detail["reference_gpu"] = rg


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
    ws_bytes = max([L.b200q_workspace_bytes(op, TOKENS, w["N"], w["K"])
                    for w in work for op in (_lib.OP_W8A8, _lib.OP_W8A16)] + [16])
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)

    # At TP > 1 the default step is the chain a layer runs: the partial output of a row-parallel
    # projection is reduced, residual-added, RMS-normed and quantised by the rank that owns the
    # token rows, and the int8 codes are gathered as the input of the NEXT column-parallel
    # projection (o -> gate_up, down -> qkv of the following step): b200q_tp_reduce_rmsnorm_quant.
    # --tp-step allreduce runs the plain route instead: all-reduce after o / down, and a
    # stand-alone activation quantiser in front of every projection, as at TP = 1.
    fused_tp = tp > 1 and comm is not None and args.tp_step == "fused"
    norm_w = torch.ones(1024, dtype=torch.bfloat16, device=dev)
    res_shard = (torch.randn(TOKENS // tp, 1024, device=dev) * 0.5).to(torch.bfloat16) if tp > 1 else None
    by_name = {w["name"]: w for w in work}
    chained = {}      # projection name -> (codes, scales) produced by the exchange in front of it

    def gemm(w, xq, a_s, stream):
        rc = L.b200q_w8a8_gemm(xq.data_ptr(), a_s.data_ptr(), w["layer"].qweight.data_ptr(),
                               w["layer"].w_scales.data_ptr(), None, w["y"].data_ptr(), TOKENS,
                               w["N"], w["K"], _lib.DTYPE_BF16, ws.data_ptr(), ws.numel(), stream)
        _lib.check(rc, "b200q_w8a8_gemm")

    def quantise(w, stream):
        rc = L.b200q_act_quant_i8(w["x"].data_ptr(), w["K"], _lib.DTYPE_BF16, w["xq"].data_ptr(),
                                  w["a_s"].data_ptr(), TOKENS, w["K"], stream)
        _lib.check(rc, "b200q_act_quant_i8")

    def kernel_step():
        """One pass of the hot path."""
        stream = torch.cuda.current_stream().cuda_stream     # the capture stream while capturing
        for w in work:
            if fused_tp and w["name"] in chained:
                gemm(w, *chained[w["name"]], stream)
            else:
                quantise(w, stream)
                gemm(w, w["xq"], w["a_s"], stream)
            if w["split"] == "row" and tp > 1:
                if fused_tp:
                    feeds = "gate_up" if w["name"] == "o" else "qkv"
                    xq, a_s, _, _ = comm.reduce_rmsnorm_quant(w["y"], norm_w, 1e-6, res_shard)
                    chained[feeds] = (xq, a_s)
                elif comm is not None:
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

    # ---- TP > 1: one exchanged tensor checked against a sum built from an NCCL all-gather
    exchange_check = None
    if tp > 1:
        from tiny_vllm_b200.quantization.cuda import add_rmsnorm_quantize_int8
        w = by_name["o"]
        quantise(w, stream)
        part = torch.empty(TOKENS, w["N"], dtype=torch.bfloat16, device=dev)   # this rank's partial
        keep, w["y"] = w["y"], part
        gemm(w, w["xq"], w["a_s"], stream)
        w["y"] = keep
        gathered = [torch.empty_like(part) for _ in range(tp)]
        dist.all_gather(gathered, part)
        total = torch.zeros(TOKENS, w["N"], dtype=torch.float32, device=dev)
        for g in gathered:                       # fp32, rank order, one rounding
            total += g.float()
        reduced = total.to(torch.bfloat16)
        if fused_tp:
            res_full = [torch.empty_like(res_shard) for _ in range(tp)]
            dist.all_gather(res_full, res_shard)
            want_q, want_s, _, _ = add_rmsnorm_quantize_int8(reduced, norm_w, 1e-6, torch.cat(res_full))
            w["y"].copy_(part)
            got_q, got_s, _, _ = comm.reduce_rmsnorm_quant(w["y"], norm_w, 1e-6, res_shard)
            comm.reduce_rmsnorm_quant(w["y"], norm_w, 1e-6, res_shard)       # keeps the two code buffers' turn
            torch.cuda.synchronize()
            same = torch.equal(got_q, want_q) and torch.equal(got_s, want_s)
            what = "codes and scales of the fused exchange vs all-gather + fp32 rank-ordered sum + add-RMSNorm + quantise"
        else:
            w["y"].copy_(part)
            out = comm.large_(w["y"]) if comm is not None else dist.all_reduce(w["y"]) or w["y"]
            if comm is not None and tp == 2:
                comm.large_(w["y"])          # the pull route alternates its slots: keep their turn
            torch.cuda.synchronize()
            same = torch.equal(out.view(torch.int16), reduced.view(torch.int16)) if comm is not None else \
                bool(((out.float() - reduced.float()).abs() <= 0.02 * reduced.float().abs() + 1e-2).all())
            what = "all-reduced o_proj output vs all-gather + fp32 rank-ordered sum"
        flag = torch.tensor([1 if same else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        exchange_check = {"result": "bit-exact" if int(flag.item()) == 1 else "MISMATCH", "what": what}
        if comm is not None and int(flag.item()) != 1:
            raise SystemExit(f"tensor-parallel exchange check failed: {what}")
        sync_all()

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
    tp_us = {}
    if tp > 1 and comm is not None:
        # the exchange kernels alone, same method (every rank replays the same graphs in step)
        w_o, w_d = by_name["o"], by_name["down"]
        turn = [0]

        def one_exchange(cs):
            turn[0] ^= 1
            comm.reduce_rmsnorm_quant((w_o if turn[0] else w_d)["y"], norm_w, 1e-6, res_shard)

        def one_allreduce(cs):
            turn[0] ^= 1
            comm.large_((w_o if turn[0] else w_d)["y"])

        dist.barrier()
        tp_us["fused_exchange_us"] = batch_us(one_exchange)
        dist.barrier()
        tp_us["allreduce_us"] = batch_us(one_allreduce)
        tp_us["note"] = ("per call on the [8192, 1024] bf16 output of o / down; fused_exchange = reduce + "
                         "residual add + RMSNorm + quantise + gather of int8 codes; allreduce = the plain sum")
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
    # the GEMM kernel is timed alone (graphs of a few launches), so the burst figure applies;
    # int8 is the double-rate MMA kind, and no int8 peak is measured on this pool
    int8_peak = 2.0 * peaks["bf16_burst"]
    achieved = gemm_ops_total / (gemm_ms_total * 1e-3) / 1e12
    traffic, traffic_note = load_traffic(world)
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                "frac": achieved / int8_peak, "traffic": traffic, "traffic_note": traffic_note,
                "frac_of_2x_sustained_bf16": achieved / (2.0 * peaks["bf16_sustained"]),
                "frac_of_nominal_4500": achieved / 4500.0,
                "timing": f"CUDA event nodes around graphs of {REPS} back-to-back launches of each GEMM, "
                          f"{ROUNDS} replays, taken right after the timed region (event records between "
                          "the kernels of a step would add about 4 us of idle GPU per boundary); "
                          "achieved = ops of the four GEMMs / sum of their durations",
                "kernel": "umma_pair_kernel<int8> (tcgen05 cta_group::2 kind::i8, TMA-store epilogue)"
                          if world == 1 else "W8A8 tcgen05 kernels on the per-rank shapes",
                "peak_note": f"2 x {peaks['source']} burst bf16 dense TFLOP/s ({peaks['bf16_burst']}): the "
                             "kernel is timed in isolation; nominal int8 peak 4500"}

    # ---- the other kernels of the path on the same shapes (not part of the timed step):
    # W8A16 prefill, the library bf16 GEMM both are meant to beat, decode batches, the larger
    # model's projections, and the reference's own CUDA kernels when oracle/_ref holds them
    if world == 1 and not args.no_extras:
        extras(detail, work, ws, dev, batch_us, peaks)

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
            "config": {"workload": WORKLOAD, "tokens": TOKENS, "parallelism": f"tp{world}",
                       "exchange": ("none" if world == 1 else
                                    "b200q_tp_reduce_rmsnorm_quant after o / down: reduce + residual add + "
                                    "RMSNorm + int8 quantise on the owning rank, codes gathered as the next "
                                    "column-parallel projection's input (peer memory)" if fused_tp else
                                    ("b200q_tp_allreduce_pull (peer memory)" if world == 2 else
                                     "b200q_tp_allreduce (peer memory)") if comm is not None else "nccl all-reduce"),
                       "launch": ("one CUDA graph replay per step (act-quant + GEMM x 4; at tp > 1 the "
                                  "exchanges too)" if step_graph is not None
                                  else "eager launches through the C ABI"),
                       "l2": "no flush: one step touches about 450 MB (activations, int8 copies, outputs), "
                             "more than the 126 MB L2"},
            "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "device_status": status, "detail": detail,
            "step_breakdown_us": {"step": ms_per_step * 1e3,
                                  "gemm_sum": sum(detail[w["name"]]["gemm_us"] for w in work),
                                  "act_quant_sum": sum(aq_us.values()), "act_quant": aq_us,
                                  **tp_us},
        }
        if exchange_check is not None:
            line["exchange_check"] = exchange_check
        rg = detail.get("reference_gpu", {})
        if "step_tops" in rg:
            # the reference's own CUDA kernels on this GPU, same step (vs_baseline stays null:
            # the reference publishes no number for this metric)
            line["vs_reference_gpu"] = {"ratio": value / rg["step_tops"], "reference_step_tops": rg["step_tops"],
                                        "what": "this step's TOPS / the same step through the reference's "
                                                "quantiser + WMMA kernel on the same B200 (detail.reference_gpu)"}
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
    for item in filter(None, args.sweep_knob.split(",")):
        name, value = item.split("=")
        _lib.check(L.b200q_debug_set(getattr(_lib, "KNOB_" + name), int(value)), "debug_set")
    if args.sweep_force:
        L.b200q_debug_force_path({"simt": _lib.PATH_SIMT_STREAM, "umma": _lib.PATH_UMMA,
                                  "umma_swap": _lib.PATH_UMMA_SWAP, "mma": _lib.PATH_MMA_STREAM}[args.sweep_force])

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
    if args.sweep_model == "8b":
        # Qwen3-8B projections, whole and as the shards of 8 tensor-parallel ranks
        shapes = [(name, n, k) for name, k, n in EIGHT_B] + \
                 [("qkv_tp8", 768, 4096), ("o_tp8", 4096, 512), ("gate_up_tp8", 3072, 4096), ("down_tp8", 4096, 1536)]
    want_ops = args.sweep_op.split(",") if args.sweep_op else ["w8a8", "w8a16", "act_quant", "fused_quant"]
    want_m = [int(m) for m in args.sweep_m.split(",")] if args.sweep_m else [1, 16, 128, 512, TOKENS]
    for op in ("w8a8", "w8a16"):
        if op not in want_ops:
            continue
        for M in want_m:
            for name, N, K in shapes:
                us = time_op(op, M, N, K, args.sweep_iters or (20 if M >= 2048 or N * K > (32 << 20) else 100))
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
        us = time_op("act_quant", TOKENS, N, K, args.sweep_iters or 50)
        b = 3 * TOKENS * K + 4 * TOKENS
        results.append({"op": "act_quant", "proj": name, "M": TOKENS, "K": K, "us": round(us, 2),
                        "algorithmic_gbs": round(b / us / 1e3, 1),
                        "hbm_frac": round(b / us / 1e3 / peaks["hbm_gbs"], 3)})
    if "fused_quant" in want_ops:
        # quantisation fused into its producers: hidden-size rows (norm) and intermediate-size
        # rows (activation) of Qwen3-0.6B at the prefill token count
        for op, K, per_row in (("add_rmsnorm_quant", 1024, 7 * 1024 + 4), ("silu_mul_quant", 3072, 5 * 3072 + 4)):
            us = time_op(op, TOKENS, 8, K, args.sweep_iters or 50)
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
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the per-shape figures of the kernels that are not in the timed step")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel from the host inside the timed region instead of "
                         "replaying one CUDA graph per step")
    ap.add_argument("--tp-step", default="fused", choices=["fused", "allreduce"],
                    help="TP > 1: 'fused' chains the projections through the fused reduce + RMSNorm + "
                         "quantise + gather exchange, 'allreduce' sums o / down outputs with an "
                         "all-reduce and quantises every input separately")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="sum row-parallel outputs with NCCL instead of the peer-memory kernel")
    ap.add_argument("--sweep-op", default="", help="shape_sweep: comma list of w8a8,w8a16,act_quant,fused_quant")
    ap.add_argument("--sweep-m", default="", help="shape_sweep: comma list of token counts")
    ap.add_argument("--sweep-model", default="0.6b", choices=["0.6b", "8b"],
                    help="shape_sweep: projections of Qwen3-0.6B or of Qwen3-8B (and its TP=8 shards)")
    ap.add_argument("--sweep-iters", type=int, default=0,
                    help="shape_sweep: launches per graph (default 20 or 100 by size); 1 keeps a profiler capture short")
    ap.add_argument("--sweep-force", default="", choices=["", "simt", "umma", "umma_swap", "mma"],
                    help="shape_sweep: force one kernel family (a debugging aid; default: the library's choice)")
    ap.add_argument("--sweep-knob", default="", help="shape_sweep: comma list of debug knobs NAME=VALUE")
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

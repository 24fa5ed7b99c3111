"""Tensor-parallel exchange step after a row-parallel linear.

The reference sums the per-rank partial outputs with ``dist.all_reduce(y)`` (NCCL,
``nanovllm/layers/linear.py:274-275``).  This module keeps that as the default and adds
an in-place all-reduce over peer memory (``b200q_tp_allreduce``: NVLink loads/stores
between the ranks' buffers, bounded flag waits) for tensors that live in a symmetric
allocation — memory of the same size on every rank, mapped into every process with
``torch.distributed._symmetric_memory``.

Usage (every rank, same order of calls)::

    comm = PeerAllReduce(max_bytes=64 << 20)          # once, after init_process_group
    y = comm.buffer((tokens, hidden), torch.bfloat16)  # write the partial result here
    ...                                                # e.g. the GEMM's output pointer
    comm.all_reduce_(y)                                # y now holds the sum on every rank

For decode-sized batches (at most 64 tokens) the sum can be fused into the GEMM kernel
itself (``b200q_w8a8_gemm_allreduce`` / ``b200q_w8a16_gemm_allreduce``): every CTA pushes
its partial tile to all ranks and adds up the peers' tiles, so a row-parallel layer is one
kernel.  ``fused_w8a8`` / ``fused_w8a16`` return ``None`` when the library refuses the shape
and the caller then uses the two-kernel route.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _lib

_DTYPE_IDS = {torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16}
_PAD_BYTES = 4096
_FUSED_MAX_M = 64
_FUSED_FLAG_BYTES = 256


class PeerAllReduce:
    """Owns one symmetric data buffer and one symmetric flag pad for a process group."""

    def __init__(self, max_bytes: int, group=None, slots: int = 2, fused_bytes: int = 16 << 20,
                 tiled_prefill: bool = False, code_bytes: int | None = None,
                 small_max_bytes: int | None = None, multimem: bool = False):
        """``max_bytes``: largest tensor a data slot holds.  ``slots``: number of rotating data
        slots, AT LEAST 2: the pull all-reduce (two ranks) leaves its input slot readable by
        the peer until the next collective, so the next partial result must go to another
        slot.  ``code_bytes``: size of each of the two int8 code buffers that
        :meth:`reduce_rmsnorm_quant` gathers into (default: ``max_bytes // 2``, i.e. the same
        number of elements as a 16-bit data slot).  ``small_max_bytes``: largest tensor the
        one-trip all-reduce takes (default by group size, see below).  ``multimem``: use the
        in-switch reduction for large tensors where the fabric offers a multicast mapping and
        the group has at least 4 ranks (off by default: it measured slower).  Nothing is read
        from the environment."""
        import torch.distributed._symmetric_memory as symm_mem

        if not dist.is_initialized():
            raise RuntimeError("PeerAllReduce needs an initialised process group")
        if slots < 2:
            raise ValueError("PeerAllReduce needs at least 2 data slots: with one, a rank would "
                             "overwrite a partial result its peer may still be reading")
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > 8:
            raise RuntimeError("PeerAllReduce supports up to 8 ranks (one node)")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.slot_bytes = (max_bytes + 255) // 256 * 256
        self.slots = slots
        self._next = 0
        name = self.group.group_name
        self._data = symm_mem.empty(self.slot_bytes * slots, dtype=torch.uint8, device=dev)
        self._data_hdl = symm_mem.rendezvous(self._data, name)
        self._pad = symm_mem.empty(_PAD_BYTES, dtype=torch.uint8, device=dev)
        self._pad.zero_()
        self._pad_hdl = symm_mem.rendezvous(self._pad, name)
        # receive area and flags of the fused decode kernels
        self.fused_bytes = (fused_bytes + 511) // 512 * 512
        # largest tensor the one-trip all-reduce takes: every rank sends (world - 1) copies at
        # twice the size, so the cross-over with the two-shot kernel falls as the group grows
        # (measured: 2 ranks about 2 MiB, 4 ranks about 400 KiB)
        default_small = (1 << 20) if self.world <= 2 else (256 << 10) if self.world <= 4 else (128 << 10)
        self.small_max_bytes = int(small_max_bytes) if small_max_bytes is not None else default_small
        self._recv = symm_mem.empty(self.fused_bytes, dtype=torch.uint8, device=dev)
        self._recv.zero_()
        self._recv_hdl = symm_mem.rendezvous(self._recv, name)
        self._fflags = symm_mem.empty(_FUSED_FLAG_BYTES, dtype=torch.uint8, device=dev)
        self._fflags.zero_()
        self._fflags_hdl = symm_mem.rendezvous(self._fflags, name)
        # staging area of the fused prefill route (GEMM + reduce-scatter); the route is opt-in:
        # at TP=2 it measured 54 us against 56 us for GEMM + two-shot all-reduce (o_proj of
        # Qwen3-0.6B, 8192 tokens) — SM-issued stores over NVLink, not the GEMM, set its pace
        self.tiled_prefill = bool(tiled_prefill)
        self._stage = self._stage_hdl = None
        if self.tiled_prefill:
            self._stage = symm_mem.empty(self.slot_bytes, dtype=torch.uint8, device=dev)
            self._stage_hdl = symm_mem.rendezvous(self._stage, name)
        # int8 codes + fp32 scales of the fused reduce + RMSNorm + quantise exchange: two
        # rotating buffers, each [codes | scales]
        self.code_bytes = ((code_bytes if code_bytes is not None else max_bytes // 2) + 255) // 256 * 256
        self._scale_bytes = (self.code_bytes // 16 * 4 + 255) // 256 * 256     # rows are >= 16 wide
        self._codes = symm_mem.empty(2 * (self.code_bytes + self._scale_bytes), dtype=torch.uint8, device=dev)
        self._codes_hdl = symm_mem.rendezvous(self._codes, name)
        self._code_next = 0
        torch.cuda.synchronize()
        dist.barrier(self.group)           # every pad is zero before anyone signals
        self._code_ptrs = [int(p) for p in self._codes_hdl.buffer_ptrs]
        self._data_ptrs = [int(p) for p in self._data_hdl.buffer_ptrs]
        # multicast mapping of the data buffer (0 when the fabric offers none): in-switch sums
        self._mc_ptr = int(getattr(self._data_hdl, "multicast_ptr", 0) or 0)
        self.use_multimem = bool(multimem) and self._mc_ptr != 0 and self.world >= 4
        pads = [int(p) for p in self._pad_hdl.buffer_ptrs]
        self._pad_arr = (ctypes.c_void_p * self.world)(*pads)
        self._recv_arr = (ctypes.c_void_p * self.world)(*[int(p) for p in self._recv_hdl.buffer_ptrs])
        self._fflags_arr = (ctypes.c_void_p * self.world)(
            *[int(p) for p in self._fflags_hdl.buffer_ptrs])
        self._stage_arr = None
        if self._stage_hdl is not None:
            self._stage_arr = (ctypes.c_void_p * self.world)(
                *[int(p) for p in self._stage_hdl.buffer_ptrs])

    def buffer(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """A tensor inside the symmetric allocation (slots are handed out round-robin, so a
        tensor stays valid until ``slots`` further buffers have been requested)."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if nbytes > self.slot_bytes:
            raise RuntimeError(f"tensor of {nbytes} bytes exceeds the symmetric slot ({self.slot_bytes})")
        off = self._next * self.slot_bytes
        self._next = (self._next + 1) % self.slots
        return self._data[off:off + nbytes].view(dtype).view(*shape)

    def owns(self, t: torch.Tensor) -> bool:
        base = self._data.data_ptr()
        return t.is_contiguous() and base <= t.data_ptr() < base + self._data.numel()

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        """Sums ``t`` (a tensor from :meth:`buffer`, same slot on every rank) over the group,
        in place, on the current stream."""
        if not self.owns(t):
            raise RuntimeError("all_reduce_ needs a contiguous tensor obtained from buffer()")
        if t.dtype not in _DTYPE_IDS or t.numel() % 8 != 0:
            raise RuntimeError("all_reduce_ supports fp16/bf16 tensors with a multiple of 8 elements")
        off = t.data_ptr() - self._data.data_ptr()
        bufs = (ctypes.c_void_p * self.world)(*[p + off for p in self._data_ptrs])
        rc = _lib.lib().b200q_tp_allreduce(bufs, self._pad_arr, self.rank, self.world, t.numel(),
                                           _DTYPE_IDS[t.dtype],
                                           torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "b200q_tp_allreduce", f"n={t.numel()} world={self.world}")
        return t

    def all_reduce_pull(self, t: torch.Tensor) -> torch.Tensor:
        """Sums ``t`` (a tensor from :meth:`buffer`) over the group into a NEW local tensor:
        every rank reads the peers' buffers, nothing is written remotely and no closing
        barrier is needed.  ``t`` must not be rewritten before the next collective of this
        communicator on a symmetric slot has run (the rotating slots of :meth:`buffer` and a
        sequence of row-parallel layers guarantee that)."""
        if not self.owns(t):
            raise RuntimeError("all_reduce_pull needs a contiguous tensor obtained from buffer()")
        if t.dtype not in _DTYPE_IDS or t.numel() % 8 != 0:
            raise RuntimeError("all_reduce_pull supports fp16/bf16 tensors with a multiple of 8 elements")
        out = torch.empty_like(t)
        off = t.data_ptr() - self._data.data_ptr()
        bufs = (ctypes.c_void_p * self.world)(*[p + off for p in self._data_ptrs])
        rc = _lib.lib().b200q_tp_allreduce_pull(bufs, self._pad_arr, out.data_ptr(), self.rank,
                                                self.world, t.numel(), _DTYPE_IDS[t.dtype],
                                                torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "b200q_tp_allreduce_pull", f"n={t.numel()} world={self.world}")
        return out

    def all_reduce_multimem_(self, t: torch.Tensor) -> torch.Tensor:
        """In-place sum of a tensor from :meth:`buffer` through the NVSwitch's reduction engine
        (needs a multicast mapping).  Same bits on every rank; the addition order is the
        switch's, so the last bit can differ from :meth:`all_reduce_`."""
        if self._mc_ptr == 0:
            raise RuntimeError("no multicast mapping for the symmetric buffer on this system")
        if not self.owns(t):
            raise RuntimeError("all_reduce_multimem_ needs a contiguous tensor obtained from buffer()")
        if t.dtype not in _DTYPE_IDS or t.numel() % 8 != 0:
            raise RuntimeError("all_reduce_multimem_ supports fp16/bf16 tensors with a multiple of 8 elements")
        off = t.data_ptr() - self._data.data_ptr()
        rc = _lib.lib().b200q_tp_allreduce_multimem(self._mc_ptr + off, self._pad_arr, self.rank,
                                                    self.world, t.numel(), _DTYPE_IDS[t.dtype],
                                                    torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "b200q_tp_allreduce_multimem", f"n={t.numel()} world={self.world}")
        return t

    def reduce_rmsnorm_quant(self, partial: torch.Tensor, weight: torch.Tensor, eps: float,
                             residual: torch.Tensor | None = None, return_normed: bool = False):
        """The exchange after a row-parallel layer fused with the residual add, RMSNorm and int8
        quantisation that follow it (``b200q_tp_reduce_rmsnorm_quant``).

        ``partial``: this rank's partial output ``[M, K]`` from :meth:`buffer` (same slot on
        every rank), ``M`` a multiple of the group size.  ``residual``: THIS RANK'S ROWS of the
        residual stream, ``[M / world, K]`` (rank ``r`` owns rows ``r * M / world`` onward), or
        ``None``.  Returns ``(x_q [M, K] int8, a_scales [M] fp32, new_residual [M / world, K] or
        None, normed [M / world, K] or None)``: codes and scales of ALL rows (gathered from every
        rank; they live in a symmetric buffer that is reused two calls later), the new residual
        and, on request, the normalised values of the own rows only."""
        if not self.owns(partial) or partial.dim() != 2 or partial.dtype not in _DTYPE_IDS:
            raise RuntimeError("reduce_rmsnorm_quant needs a 2-D fp16/bf16 tensor obtained from buffer()")
        M, K = partial.shape
        if M % self.world != 0 or K % 16 != 0:
            raise RuntimeError("reduce_rmsnorm_quant needs M % world == 0 and K % 16 == 0")
        if M * K > self.code_bytes or M * 4 > self._scale_bytes:
            raise RuntimeError(f"[{M}, {K}] codes exceed the symmetric code buffer ({self.code_bytes} bytes)")
        rows = M // self.world
        if residual is not None and (tuple(residual.shape) != (rows, K) or residual.dtype != partial.dtype
                                     or not residual.is_contiguous()):
            raise RuntimeError(f"residual must be this rank's contiguous [{rows}, {K}] rows in the partial's dtype")
        if weight.dtype != partial.dtype or weight.numel() != K:
            raise RuntimeError("weight must have K elements of the partial's dtype")
        base = self._code_next * (self.code_bytes + self._scale_bytes)
        self._code_next ^= 1
        xq = self._codes[base:base + M * K].view(torch.int8).view(M, K)
        a_s = self._codes[base + self.code_bytes:base + self.code_bytes + 4 * M].view(torch.float32)
        new_res = torch.empty_like(residual) if residual is not None else None
        normed = torch.empty((rows, K), dtype=partial.dtype, device=partial.device) if return_normed else None
        off = partial.data_ptr() - self._data.data_ptr()
        parts = (ctypes.c_void_p * self.world)(*[p + off for p in self._data_ptrs])
        xqs = (ctypes.c_void_p * self.world)(*[p + base for p in self._code_ptrs])
        scs = (ctypes.c_void_p * self.world)(*[p + base + self.code_bytes for p in self._code_ptrs])
        rc = _lib.lib().b200q_tp_reduce_rmsnorm_quant(
            parts, self._pad_arr, None if residual is None else residual.data_ptr(),
            None if new_res is None else new_res.data_ptr(), weight.contiguous().data_ptr(), float(eps),
            xqs, scs, None if normed is None else normed.data_ptr(), M, K, self.rank, self.world,
            _DTYPE_IDS[partial.dtype], torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "b200q_tp_reduce_rmsnorm_quant", f"M={M} K={K} world={self.world}")
        return xq, a_s, new_res, normed

    def large_(self, t: torch.Tensor) -> torch.Tensor:
        """All-reduce of a tensor that lives in a symmetric slot by the fastest large-tensor
        kernel: pull for two ranks, in-switch reduction from four ranks up where a multicast
        mapping exists, two-shot otherwise."""
        if self.world == 2:
            return self.all_reduce_pull(t)
        if self.use_multimem:
            return self.all_reduce_multimem_(t)
        return self.all_reduce_(t)

    def small_fits(self, t: torch.Tensor) -> bool:
        """True when ``t`` qualifies for the one-trip kernel: 16-bit, contiguous, a multiple of
        8 elements, at most ``small_max_bytes`` and within the receive area."""
        return (t.is_cuda and t.dtype in _DTYPE_IDS and t.is_contiguous() and t.numel() > 0
                and t.numel() % 8 == 0 and t.data_ptr() % 16 == 0
                and t.numel() * 2 <= self.small_max_bytes
                and self.world * t.numel() * 4 <= self.fused_bytes // 2)

    def all_reduce_small_(self, t: torch.Tensor) -> torch.Tensor:
        """Sums any local 16-bit tensor over the group in place with the one-trip kernel."""
        rc = _lib.lib().b200q_tp_allreduce_small(
            t.data_ptr(), t.data_ptr(), t.numel(), _DTYPE_IDS[t.dtype], self._recv_arr,
            self._fflags_arr, self.fused_bytes, self.rank, self.world,
            torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "b200q_tp_allreduce_small", f"n={t.numel()} world={self.world}")
        return t

    def reduce(self, y: torch.Tensor) -> torch.Tensor:
        """Sum of ``y`` over the group by the cheapest route that takes it: the one-trip
        kernel for small tensors, the two-shot kernel through a symmetric slot for large ones,
        NCCL for everything else.  Returns the reduced tensor (``y`` itself or a slot)."""
        if self.small_fits(y):
            return self.all_reduce_small_(y)
        if y.is_cuda and y.dtype in _DTYPE_IDS and y.numel() % 8 == 0 \
                and y.numel() * y.element_size() <= self.slot_bytes:
            if self.owns(y):
                return self.large_(y)
            shared = self.buffer(y.shape, y.dtype)
            shared.copy_(y)
            return self.large_(shared)
        dist.all_reduce(y, group=self.group)
        return y

    # ------------------------------------------------------------------ fused decode route
    def fused_fits(self, tokens: int, n_out: int) -> bool:
        return (0 < tokens <= _FUSED_MAX_M and n_out % 8 == 0
                and self.world * tokens * n_out * 4 <= self.fused_bytes // 2)

    def _finish_fused(self, rc: int, name: str, detail: str, y: torch.Tensor):
        if rc == _lib.ERR_UNSUPPORTED_SHAPE:
            return None
        _lib.check(rc, name, detail)
        return y

    def fused_w8a8(self, x_q, a_scales, qweight, w_scales, bias, out_dtype):
        """Row-parallel W8A8 linear plus the sum over ranks in one kernel.  ``x_q`` int8
        ``[M, K_local]``, ``qweight`` int8 ``[N, K_local]``; returns ``[M, N]`` or ``None``."""
        M, K = x_q.shape
        N = qweight.shape[0]
        if not self.fused_fits(M, N):
            return None
        y = torch.empty((M, N), dtype=out_dtype, device=x_q.device)
        rc = _lib.lib().b200q_w8a8_gemm_allreduce(
            x_q.data_ptr(), a_scales.data_ptr(), qweight.data_ptr(), w_scales.data_ptr(),
            None if bias is None else bias.data_ptr(), y.data_ptr(), M, N, K,
            _DTYPE_IDS[out_dtype], self._recv_arr, self._fflags_arr, self.fused_bytes,
            self.rank, self.world, torch.cuda.current_stream().cuda_stream)
        return self._finish_fused(rc, "b200q_w8a8_gemm_allreduce", f"M={M} N={N} K={K}", y)

    def fused_w8a16(self, x_2d, qweight, scales, bias):
        """Row-parallel W8A16 linear plus the sum over ranks in one kernel."""
        M, K = x_2d.shape
        N = qweight.shape[0]
        if not self.fused_fits(M, N):
            return None
        y = torch.empty((M, N), dtype=x_2d.dtype, device=x_2d.device)
        rc = _lib.lib().b200q_w8a16_gemm_allreduce(
            x_2d.data_ptr(), qweight.data_ptr(), scales.data_ptr(),
            None if bias is None else bias.data_ptr(), y.data_ptr(), M, N, K,
            _DTYPE_IDS[x_2d.dtype], self._recv_arr, self._fflags_arr, self.fused_bytes,
            self.rank, self.world, torch.cuda.current_stream().cuda_stream)
        return self._finish_fused(rc, "b200q_w8a16_gemm_allreduce", f"M={M} N={N} K={K}", y)

    # ------------------------------------------------------------------ fused prefill route
    def tiled_fits(self, tokens: int, n_out: int) -> bool:
        """Shapes the fused GEMM + reduce-scatter + all-gather route takes."""
        return (self.tiled_prefill and tokens >= 512 and tokens % (self.world * 256) == 0
                and n_out % 8 == 0 and tokens * n_out * 2 <= self.slot_bytes)

    def fused_w8a8_tiled(self, x_q, a_scales, qweight, w_scales, bias, out_dtype):
        """Row-parallel W8A8 linear at prefill size: the GEMM's epilogue sends every partial
        tile to the rank that owns its token rows, a second kernel sums and gathers.  Returns
        the reduced ``[M, N]`` tensor (in a symmetric slot) or ``None``."""
        M, K = x_q.shape
        N = qweight.shape[0]
        if not self.tiled_fits(M, N):
            return None
        y = self.buffer((M, N), out_dtype)
        off = y.data_ptr() - self._data.data_ptr()
        ys = (ctypes.c_void_p * self.world)(*[p + off for p in self._data_ptrs])
        rc = _lib.lib().b200q_w8a8_gemm_allreduce_tiled(
            x_q.data_ptr(), a_scales.data_ptr(), qweight.data_ptr(), w_scales.data_ptr(),
            None if bias is None else bias.data_ptr(), ys, M, N, K, _DTYPE_IDS[out_dtype],
            self._stage_arr, self.slot_bytes, self._fflags_arr, self.rank, self.world,
            torch.cuda.current_stream().cuda_stream)
        return self._finish_fused(rc, "b200q_w8a8_gemm_allreduce_tiled", f"M={M} N={N} K={K}", y)

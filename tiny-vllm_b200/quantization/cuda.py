"""Python entry points of the quantized-linear kernels.

Counterpart of ``nanovllm/quantization/cuda.py`` in the reference: the same
public functions (``apply_int8_weight_only_linear`` — reference lines 303-366,
``apply_w8a8_linear`` — lines 468-504) with the same argument meaning and the
same input checks (reference lines 21-33, 225-258, 369-432).  Differences, all
deliberate:

* one backend — the sm_100a library behind ``include/b200q.h``; the backend
  environment switches of the reference are gone;
* no Python/CPU fallback: an input the kernels cannot take raises
  ``RuntimeError`` where the reference would silently run dequantize + matmul;
* kernels run on ``torch.cuda.current_stream()`` so CUDA-graph capture records
  them (the reference launches on the legacy default stream).
"""
from __future__ import annotations

import threading

import torch

from .. import _lib

_DTYPE_IDS = {torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16}
_DEFAULT_WORKSPACE_BYTES = 64 << 20

_ws_lock = threading.Lock()
_workspaces: dict[int, torch.Tensor] = {}
_workspace_floor = [_DEFAULT_WORKSPACE_BYTES]


def reserve_workspace(nbytes: int, device: torch.device | None = None) -> None:
    """Makes the per-device scratch buffer at least ``nbytes`` large (call before CUDA-graph
    capture when a model's shapes need more than the default 64 MiB; ``b200q_workspace_bytes``
    of the C ABI gives the need of a shape).  With a ``device`` the buffer is allocated now."""
    _workspace_floor[0] = max(_workspace_floor[0], int(nbytes))
    if device is not None:
        _workspace(torch.device(device), int(nbytes))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(device: torch.device) -> int:
    """Handle of the current stream of ``device`` (what ``torch.cuda.current_stream(device)
    .cuda_stream`` returns, without building the stream object: this is on the path of every
    linear of an eagerly executed step)."""
    if _raw_stream is not None:
        idx = device.index
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _on_device(device: torch.device):
    """Device guard for a launch: nothing when ``device`` is the current device already (the
    usual case; entering ``torch.cuda.device`` costs several microseconds per call)."""
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor | None:
    """Zero-filled scratch buffer shared by every call on ``device``.

    The split-K kernels keep their tile counters in it and leave them at zero,
    so a single buffer serves all layers as long as calls are stream-ordered
    (they are: one stream per model runner).  It is allocated once, large enough
    for the shapes of a decode step, so that nothing is allocated while a CUDA
    graph is being captured.
    """
    if nbytes == 0:
        return None
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is not None and ws.numel() >= nbytes:
        return ws
    with _ws_lock:
        ws = _workspaces.get(idx)
        if ws is None or ws.numel() < nbytes:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(
                    f"b200q workspace of {nbytes} bytes requested during CUDA graph capture; "
                    "run the shape once eagerly first or call reserve_workspace() before capture")
            want = max(nbytes, _workspace_floor[0])
            ws = torch.zeros(want, dtype=torch.uint8, device=torch.device("cuda", idx))
            _workspaces[idx] = ws
    return ws


def _require_cuda(*tensors: torch.Tensor) -> None:
    if not all(t.is_cuda for t in tensors):
        raise RuntimeError(
            "b200q kernels need CUDA tensors on a B200; there is no CPU implementation of this path")


def select_path(op: int, M: int, N: int, K: int) -> str:
    """Kernel family the library picks for a problem (reference: ``select_path`` of the
    pybind modules, ``csrc/w8a8_gemm.cpp:51-54``)."""
    return _lib.lib().b200q_select_path(op, M, N, K).decode()


def quantize_activation_int8(x_2d: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token dynamic int8 quantisation on the GPU (one kernel).

    ``x_2d`` is ``[M, K]`` fp16/bf16 with unit inner stride.  Returns ``(x_q int8
    [M, K], a_scales fp32 [M])``, bit-identical to the reference's
    ``quantize_int8_per_row_dynamic`` (``nanovllm/quantization/utils.py:28-32``).
    """
    _require_cuda(x_2d)
    if x_2d.dim() != 2 or x_2d.dtype not in _DTYPE_IDS:
        raise RuntimeError("activation quantisation expects a 2-D float16/bfloat16 tensor")
    if x_2d.stride(1) != 1 or x_2d.stride(0) < x_2d.shape[1] or x_2d.stride(0) % 8 != 0 \
            or x_2d.data_ptr() % 16 != 0:
        x_2d = x_2d.contiguous()
    M, K = x_2d.shape
    if M == 0:
        return (torch.empty((0, K), dtype=torch.int8, device=x_2d.device),
                torch.empty((0,), dtype=torch.float32, device=x_2d.device))
    x_q = torch.empty((M, K), dtype=torch.int8, device=x_2d.device)
    a_scales = torch.empty((M,), dtype=torch.float32, device=x_2d.device)
    with _on_device(x_2d.device):
        rc = _lib.lib().b200q_act_quant_i8(x_2d.data_ptr(), x_2d.stride(0), _DTYPE_IDS[x_2d.dtype],
                                           x_q.data_ptr(), a_scales.data_ptr(), M, K,
                                           _stream_ptr(x_2d.device))
    if rc:
        _lib.check(rc, "b200q_act_quant_i8", f"M={M} K={K}")
    return x_q, a_scales


def add_rmsnorm_quantize_int8(x: torch.Tensor, weight: torch.Tensor, eps: float,
                              residual: torch.Tensor | None = None, return_normed: bool = False):
    """RMSNorm (optionally with the residual add in front) and the per-token int8 quantisation
    of its output in one kernel: what ``RMSNorm.forward`` (``nanovllm/layers/layernorm.py:16-50``)
    followed by ``quantize_int8_per_row_dynamic`` computes, without the 16-bit round trip.
    The new residual is bit-identical to the module's; the normalised value is within two units
    in the last place of it in at most 2 % of the elements (the mean of squares is summed in a
    different order); codes and scales are bit-identical to quantising the value formed here.

    ``x``: ``[..., K]`` fp16/bf16; ``weight``: ``[K]`` same dtype; ``residual``: like ``x`` or
    ``None``.  Returns ``(x_q [M, K] int8, a_scales [M] fp32, new_residual or None, normed or
    None)`` with ``M`` the flattened token count; ``new_residual`` has ``x``'s shape."""
    _require_cuda(x, weight)
    if x.dtype not in _DTYPE_IDS or weight.dtype != x.dtype or weight.dim() != 1 \
            or weight.numel() != x.shape[-1]:
        raise RuntimeError("add_rmsnorm_quantize_int8 expects fp16/bf16 x and a weight of its width and dtype")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype or not residual.is_cuda):
        raise RuntimeError("residual must match x in shape, dtype and device")
    K = x.shape[-1]
    x2 = x.contiguous().view(-1, K)
    M = x2.shape[0]
    r2 = None if residual is None else residual.contiguous().view(-1, K)
    x_q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    a_s = torch.empty((M,), dtype=torch.float32, device=x.device)
    new_res = torch.empty_like(x2) if residual is not None else None
    normed = torch.empty_like(x2) if return_normed else None
    with _on_device(x.device):
        rc = _lib.lib().b200q_add_rmsnorm_quant_i8(
            x2.data_ptr(), None if r2 is None else r2.data_ptr(), weight.contiguous().data_ptr(),
            float(eps), None if new_res is None else new_res.data_ptr(),
            None if normed is None else normed.data_ptr(), x_q.data_ptr(), a_s.data_ptr(), M, K,
            _DTYPE_IDS[x.dtype], _stream_ptr(x.device))
    if rc:
        _lib.check(rc, "b200q_add_rmsnorm_quant_i8", f"M={M} K={K}")
    return (x_q, a_s, None if new_res is None else new_res.view(x.shape),
            None if normed is None else normed.view(x.shape))


def silu_mul_quantize_int8(gate_up: torch.Tensor, return_act: bool = False):
    """``SiluAndMul.forward`` (``nanovllm/layers/activation.py:11-14``) and the per-token int8
    quantisation of its output in one kernel.  ``gate_up``: ``[..., 2 I]`` fp16/bf16.  Returns
    ``(x_q [M, I] int8, a_scales [M] fp32, act [..., I] or None)``.

    Rounding: the activation is formed as ``T(silu(float(gate)) * float(up))`` — ONE rounding of
    the fp32 product, which is what the module's ``torch.compile`` decorator produces on a GPU.
    Run operation by operation (no compiler), the module rounds ``silu(gate)`` to 16 bits before
    the product; against that form the activation is never more than one unit in the last place
    off, in 26-27 % of the elements (measured on the reference module's outputs), and codes and
    scales can differ accordingly.  Against the single-rounding form fewer than 2 % of the
    elements differ by one unit (hardware ``exp``).  The int8 codes and scales are always
    bit-identical to quantising the activation this kernel formed."""
    _require_cuda(gate_up)
    if gate_up.dtype not in _DTYPE_IDS or gate_up.shape[-1] % 2 != 0:
        raise RuntimeError("silu_mul_quantize_int8 expects an fp16/bf16 tensor with an even last dimension")
    two_i = gate_up.shape[-1]
    g2 = gate_up.contiguous().view(-1, two_i)
    M, inter = g2.shape[0], two_i // 2
    x_q = torch.empty((M, inter), dtype=torch.int8, device=gate_up.device)
    a_s = torch.empty((M,), dtype=torch.float32, device=gate_up.device)
    act = torch.empty((M, inter), dtype=gate_up.dtype, device=gate_up.device) if return_act else None
    with _on_device(gate_up.device):
        rc = _lib.lib().b200q_silu_mul_quant_i8(g2.data_ptr(), two_i, None if act is None else act.data_ptr(),
                                                x_q.data_ptr(), a_s.data_ptr(), M, inter,
                                                _DTYPE_IDS[gate_up.dtype], _stream_ptr(gate_up.device))
    if rc:
        _lib.check(rc, "b200q_silu_mul_quant_i8", f"M={M} I={inter}")
    return x_q, a_s, None if act is None else act.view(*gate_up.shape[:-1], inter)


def _check_w8a16(x, qweight, scales, bias) -> None:
    _require_cuda(x, qweight, scales)
    if x.dtype not in _DTYPE_IDS or qweight.dtype != torch.int8 or scales.dtype != torch.float32:
        raise RuntimeError("CUDA INT8 weight-only backend does not support the provided tensors")
    if x.numel() == 0 or qweight.numel() == 0 or scales.numel() == 0:
        raise RuntimeError("CUDA INT8 weight-only backend does not support the provided tensors")
    if qweight.dim() != 2 or x.shape[-1] != qweight.shape[-1]:
        raise RuntimeError(f"Incompatible shapes: x[-1]={x.shape[-1]} vs qweight[-1]={qweight.shape[-1]}")
    if scales.dim() != 1 or scales.numel() != qweight.shape[0]:
        raise RuntimeError("scales must be 1D with one value per output channel")
    if bias is not None:
        if bias.dim() != 1 or bias.numel() != qweight.shape[0]:
            raise RuntimeError("bias must be 1D with one value per output channel")
        if bias.dtype != x.dtype or not bias.is_cuda:
            raise RuntimeError("bias must be a CUDA tensor of the activation dtype")


def apply_int8_weight_only_linear(
    x: torch.Tensor,
    qweight: torch.Tensor,
    scales: torch.Tensor,
    bias: torch.Tensor | None = None,
) -> torch.Tensor:
    """W8A16 linear ``y = x @ dequant(qweight, scales).T + bias``.

    ``x``: ``[..., K]`` fp16/bf16; ``qweight``: int8 ``[N, K]``; ``scales``: fp32
    ``[N]``; returns ``[..., N]`` in ``x.dtype``.
    """
    _check_w8a16(x, qweight, scales, bias)
    K = x.shape[-1]
    N = qweight.shape[0]
    x_2d = x.contiguous().view(-1, K)
    qweight = qweight.contiguous()
    scales = scales.contiguous()
    bias = None if bias is None else bias.contiguous()
    M = x_2d.shape[0]
    y = torch.empty((M, N), dtype=x.dtype, device=x.device)
    L = _lib.lib()
    with _on_device(x.device):
        ws_bytes = L.b200q_workspace_bytes(_lib.OP_W8A16, M, N, K)
        ws = _workspace(x.device, ws_bytes)
        rc = L.b200q_w8a16_gemm(x_2d.data_ptr(), qweight.data_ptr(), scales.data_ptr(),
                                None if bias is None else bias.data_ptr(), y.data_ptr(), M, N, K,
                                _DTYPE_IDS[x.dtype], None if ws is None else ws.data_ptr(),
                                0 if ws is None else ws.numel(), _stream_ptr(x.device))
    if rc:
        _lib.check(rc, "b200q_w8a16_gemm", f"M={M} N={N} K={K}")
    return y.view(*x.shape[:-1], N)


def _check_w8a8(x_q, a_scales, qweight, w_scales, bias, out_dtype) -> None:
    _require_cuda(x_q, a_scales, qweight, w_scales)
    ok = (x_q.dtype == torch.int8 and qweight.dtype == torch.int8
          and a_scales.dtype == torch.float32 and w_scales.dtype == torch.float32
          and out_dtype in _DTYPE_IDS and x_q.dim() == 2 and qweight.dim() == 2
          and x_q.numel() > 0 and qweight.numel() > 0)
    if not ok:
        raise RuntimeError("CUDA W8A8 backend does not support the provided tensors")
    if x_q.shape[-1] != qweight.shape[-1]:
        raise RuntimeError(f"Incompatible shapes: x_q[-1]={x_q.shape[-1]} vs qweight[-1]={qweight.shape[-1]}")
    if a_scales.dim() != 1 or a_scales.numel() != x_q.shape[0]:
        raise RuntimeError("a_scales must be 1D with one value per input row")
    if w_scales.dim() != 1 or w_scales.numel() != qweight.shape[0]:
        raise RuntimeError("w_scales must be 1D with one value per output channel")
    if bias is not None:
        if bias.dim() != 1 or bias.numel() != qweight.shape[0]:
            raise RuntimeError("bias must be 1D with one value per output channel")
        if bias.dtype != out_dtype or not bias.is_cuda:
            raise RuntimeError("bias must be a CUDA tensor of the output dtype")


def apply_w8a8_linear(
    x_q: torch.Tensor,
    a_scales: torch.Tensor,
    qweight: torch.Tensor,
    w_scales: torch.Tensor,
    bias: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.float16,
    out_shape: tuple[int, ...] | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """W8A8 linear: exact int32 ``x_q @ qweight.T``, then
    ``(acc * a_scales[:, None]) * w_scales[None, :] + bias`` cast to ``out_dtype``.
    ``out``: a contiguous ``[M, N]`` tensor of ``out_dtype`` to write into instead of a new one
    (e.g. a slot of the symmetric buffer that a tensor-parallel exchange reads)."""
    _check_w8a8(x_q, a_scales, qweight, w_scales, bias, out_dtype)
    x_q = x_q.contiguous()
    a_scales = a_scales.contiguous()
    qweight = qweight.contiguous()
    w_scales = w_scales.contiguous()
    bias = None if bias is None else bias.contiguous()
    M, K = x_q.shape
    N = qweight.shape[0]
    if out is None:
        y = torch.empty((M, N), dtype=out_dtype, device=x_q.device)
    else:
        if tuple(out.shape) != (M, N) or out.dtype != out_dtype or not out.is_contiguous() \
                or out.device != x_q.device:
            raise RuntimeError(f"out must be a contiguous [{M}, {N}] {out_dtype} tensor on {x_q.device}")
        y = out
    L = _lib.lib()
    with _on_device(x_q.device):
        ws_bytes = L.b200q_workspace_bytes(_lib.OP_W8A8, M, N, K)
        ws = _workspace(x_q.device, ws_bytes)
        rc = L.b200q_w8a8_gemm(x_q.data_ptr(), a_scales.data_ptr(), qweight.data_ptr(),
                               w_scales.data_ptr(), None if bias is None else bias.data_ptr(),
                               y.data_ptr(), M, N, K, _DTYPE_IDS[out_dtype],
                               None if ws is None else ws.data_ptr(),
                               0 if ws is None else ws.numel(), _stream_ptr(x_q.device))
    if rc:
        _lib.check(rc, "b200q_w8a8_gemm", f"M={M} N={N} K={K}")
    return y if out_shape is None else y.view(out_shape)


def w8a8_int32_accumulators(x_q: torch.Tensor, qweight: torch.Tensor) -> torch.Tensor:
    """Raw int32 ``x_q @ qweight.T`` from the same kernels (parity/debug entry)."""
    _require_cuda(x_q, qweight)
    if x_q.dtype != torch.int8 or qweight.dtype != torch.int8 or x_q.dim() != 2 or qweight.dim() != 2:
        raise RuntimeError("w8a8_int32_accumulators expects 2-D int8 tensors")
    if x_q.shape[1] != qweight.shape[1]:
        raise RuntimeError("x_q and qweight shapes do not align")
    x_q = x_q.contiguous()
    qweight = qweight.contiguous()
    M, K = x_q.shape
    N = qweight.shape[0]
    acc = torch.empty((M, N), dtype=torch.int32, device=x_q.device)
    L = _lib.lib()
    with _on_device(x_q.device):
        ws_bytes = L.b200q_workspace_bytes(_lib.OP_W8A8, M, N, K)
        ws = _workspace(x_q.device, ws_bytes)
        rc = L.b200q_w8a8_gemm_i32(x_q.data_ptr(), qweight.data_ptr(), acc.data_ptr(), M, N, K,
                                   None if ws is None else ws.data_ptr(),
                                   0 if ws is None else ws.numel(), _stream_ptr(x_q.device))
    if rc:
        _lib.check(rc, "b200q_w8a8_gemm_i32", f"M={M} N={N} K={K}")
    return acc

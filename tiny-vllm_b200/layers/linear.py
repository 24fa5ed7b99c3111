"""Tensor-parallel linear layers with the reference's constructors and loaders.

Drop-in counterpart of ``nanovllm/layers/linear.py``: the same class names,
constructor signatures, attributes (``tp_dim``, ``tp_rank``, ``tp_size``,
``quant_method``, ``output_sizes``, ``num_heads``, ``num_kv_heads``, ``head_size``)
and per-parameter ``weight_loader`` hooks, so the reference's model code
(``nanovllm/models/qwen3.py:43-56,103-114``) and loader
(``nanovllm/utils/loader.py:44-68``) work unchanged.  Quantized forwards go to the
sm_100a kernels through the ``QuantMethod`` plug-ins.

Sharding rules (reference lines in parentheses):

* column-parallel (101-113): output channels are split; rank ``r`` owns rows
  ``[r*N/t, (r+1)*N/t)`` of the weight and the same slice of scales and bias;
* merged / QKV (139-171, 209-244): the stored matrix packs several sub-matrices
  along the output dimension; each sub-matrix is split separately and the local
  pieces are packed in the same order;
* row-parallel (259-276): input features are split; each rank produces a partial
  ``[tokens, N]`` result and the results are summed with an all-reduce; per-channel
  scales are replicated.

Every layout is described once as a list of ``(dst_offset, dst_size, src_offset,
src_size)`` segments and copied by one helper.

Besides the reference's ``weight_loader`` hooks (which take the whole stored tensor and keep
this rank's part), every parameter carries a ``shard_plan(stored_shape, *shard_id)`` hook that
returns the same copy as a list of ``(dst_index, src_index)`` slice tuples.  A loader that can
read parts of a stored tensor (safetensors ``get_slice``) uses it to read only this rank's
share from disk: 1 / tp of the bytes instead of all of them on every rank
(``nanovllm/utils/loader.py:50-64`` reads every full tensor on every rank).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from ..quantization import Int8WeightOnlyQuantMethod, W8A8QuantMethod

_QUANT_METHODS = {"int8": Int8WeightOnlyQuantMethod, "w8a8": W8A8QuantMethod}
# scale parameter name per scheme (artifact suffixes ".scales" / ".w_scales")
_SCALE_NAMES = ("scales", "w_scales")


# Optional replacement for the NCCL all-reduce after row-parallel layers: an object with
# ``reduce(tensor) -> tensor`` and, optionally, the fused decode hooks ``fused_fits`` /
# ``fused_w8a8`` / ``fused_w8a16`` (layers.tp_comm.PeerAllReduce).
_peer_all_reduce = None


def set_tp_all_reduce(comm) -> None:
    """Routes the sum after every RowParallelLinear through ``comm`` (peer-memory kernel)
    instead of ``dist.all_reduce``; ``None`` restores NCCL.  With a communicator a large
    result lives in one of its rotating symmetric slots: it stays valid until that many
    further large row-parallel calls have been made.  Decode-sized quantized calls run the
    GEMM and the sum as one kernel, small tensors take the one-trip all-reduce."""
    global _peer_all_reduce
    _peer_all_reduce = comm


def divide(numerator: int, denominator: int) -> int:
    quotient, rest = divmod(numerator, denominator)
    assert rest == 0, f"{numerator} is not divisible by {denominator}"
    return quotient


def _tp_coordinates() -> tuple[int, int]:
    """(rank, world size) of the tensor-parallel group; (0, 1) without a process group."""
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _segment_plan(dim: int, ndim: int, segments, rank: int, size: int):
    """The copies of :func:`_copy_segments` as ``(dst_index, src_index)`` slice tuples."""
    plan = []
    for dst_off, dst_size, src_off, src_size in segments:
        part = src_size // size
        lo = src_off + rank * part
        dst = [slice(None)] * ndim
        src = [slice(None)] * ndim
        dst[dim] = slice(dst_off, dst_off + dst_size)
        src[dim] = slice(lo, lo + part)
        plan.append((tuple(dst), tuple(src)))
    return plan


def _copy_segments(dst: torch.Tensor, src: torch.Tensor, dim: int, segments, rank: int, size: int):
    """For every segment: split ``src[src_off : src_off+src_size]`` into ``size`` equal
    parts along ``dim`` and copy part ``rank`` to ``dst[dst_off : dst_off+dst_size]``."""
    for dst_off, dst_size, src_off, src_size in segments:
        piece = src.narrow(dim, src_off, src_size).chunk(size, dim)[rank]
        dst.narrow(dim, dst_off, dst_size).copy_(piece)


class LinearBase(nn.Module):
    """Owns the parameters (plain ``weight`` or quantized ``qweight`` + scales) and
    their loader hooks; subclasses define the sharding and the forward."""

    def __init__(
        self,
        input_size: int,
        output_size: int,
        bias: bool = False,
        tp_dim: int | None = None,
        quantization: str | None = None,
    ):
        super().__init__()
        if quantization is not None and quantization not in _QUANT_METHODS:
            raise NotImplementedError(f"Unsupported linear quantization: {quantization}")
        self.tp_dim = tp_dim
        self.tp_rank, self.tp_size = _tp_coordinates()
        self.quantization = quantization
        self.quant_method = _QUANT_METHODS[quantization]() if quantization else None
        if self.quant_method is None:
            self.weight = nn.Parameter(torch.empty(output_size, input_size))
            self.weight.weight_loader = self.weight_loader
            self.weight.shard_plan = self._plan_for("weight")
        else:
            self.quant_method.create_weights(self, input_size, output_size)
            self.qweight.weight_loader = self.qweight_loader
            self.qweight.shard_plan = self._plan_for("qweight")
            for name in _SCALE_NAMES:
                if hasattr(self, name):
                    getattr(self, name).weight_loader = self.scales_loader
                    getattr(self, name).shard_plan = self._plan_for("scales")
        if bias:
            self.bias = nn.Parameter(torch.empty(output_size))
            self.bias.weight_loader = self.bias_loader
            self.bias.shard_plan = self._plan_for("bias")
        else:
            self.register_parameter("bias", None)

    def _plan_for(self, kind: str):
        return lambda stored_shape, *shard_id: self.shard_plan(kind, tuple(stored_shape), *shard_id)

    def shard_plan(self, kind: str, stored_shape: tuple, *shard_id):
        """What this rank copies out of a stored tensor of ``stored_shape`` into the parameter of
        ``kind`` ("weight" | "qweight" | "scales" | "bias"): ``[(dst_index, src_index), ...]``.
        Default: the whole tensor (replicated parameters)."""
        whole = tuple(slice(None) for _ in stored_shape)
        return [(whole, whole)]

    # -- loader hooks; the defaults copy the stored tensor as is -------------
    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        param.data.copy_(loaded_weight)

    def bias_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        self.weight_loader(param, loaded_weight)

    def qweight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        self.weight_loader(param, loaded_weight)

    def scales_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        self.weight_loader(param, loaded_weight)

    def apply_linear(self, x: torch.Tensor) -> torch.Tensor:
        if self.quant_method is None:
            return F.linear(x, self.weight, self.bias)
        return self.quant_method.apply(x, self)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class ReplicatedLinear(LinearBase):
    """Every rank holds the full matrix."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False,
                 quantization: str | None = None):
        super().__init__(input_size, output_size, bias, quantization=quantization)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.apply_linear(x)


class ColumnParallelLinear(LinearBase):
    """Output channels split over ranks; no communication in forward."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False,
                 quantization: str | None = None):
        _, world = _tp_coordinates()
        super().__init__(input_size, divide(output_size, world), bias, 0, quantization)

    def _load_rank_slice(self, param: nn.Parameter, stored: torch.Tensor, dim: int):
        local = param.data.size(dim)
        param.data.copy_(stored.narrow(dim, self.tp_rank * local, local))

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        self._load_rank_slice(param, loaded_weight, self.tp_dim)

    def scales_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        self._load_rank_slice(param, loaded_weight, 0)

    def shard_plan(self, kind: str, stored_shape: tuple, *shard_id):
        rows = stored_shape[0]
        return _segment_plan(0, len(stored_shape), [(0, rows // self.tp_size, 0, rows)],
                             self.tp_rank, self.tp_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.apply_linear(x)


class _PackedColumnParallel(ColumnParallelLinear):
    """Shared logic of layers whose matrix packs several sub-matrices along dim 0."""

    def _segments(self):
        """(dst_offset, dst_size, src_offset, src_size) per packed sub-matrix."""
        raise NotImplementedError

    def _segment_of(self, shard_id):
        """The segment that one unpacked HF tensor (shard id) fills."""
        raise NotImplementedError

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id):
        dst_off, dst_size, _, _ = self._segment_of(loaded_shard_id)
        _copy_segments(param.data, loaded_weight, self.tp_dim,
                       [(dst_off, dst_size, 0, loaded_weight.size(self.tp_dim))],
                       self.tp_rank, self.tp_size)

    def packed_weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        _copy_segments(param.data, loaded_weight, self.tp_dim, self._segments(),
                       self.tp_rank, self.tp_size)

    def packed_scales_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        _copy_segments(param.data, loaded_weight, 0, self._segments(), self.tp_rank, self.tp_size)

    def bias_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id=None):
        if loaded_shard_id is None:
            self.packed_scales_loader(param, loaded_weight)
        else:
            self.weight_loader(param, loaded_weight, loaded_shard_id)

    def qweight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        self.packed_weight_loader(param, loaded_weight)

    def scales_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        self.packed_scales_loader(param, loaded_weight)

    def shard_plan(self, kind: str, stored_shape: tuple, *shard_id):
        if shard_id and shard_id[0] is not None:    # one unpacked sub-matrix (HF checkpoint)
            dst_off, dst_size, _, _ = self._segment_of(shard_id[0])
            segments = [(dst_off, dst_size, 0, stored_shape[0])]
        else:                                       # the packed tensor of a quantized artifact
            segments = self._segments()
        return _segment_plan(0, len(stored_shape), segments, self.tp_rank, self.tp_size)


class MergedColumnParallelLinear(_PackedColumnParallel):
    """Several column-parallel matrices sharing one input, stored back to back
    (gate_proj and up_proj -> ``gate_up_proj``).  Shard ids are list indices."""

    def __init__(self, input_size: int, output_sizes: list[int], bias: bool = False,
                 quantization: str | None = None):
        self.output_sizes = output_sizes
        super().__init__(input_size, sum(output_sizes), bias, quantization)

    def _segments(self):
        segments, src_off = [], 0
        for size in self.output_sizes:
            segments.append((src_off // self.tp_size, size // self.tp_size, src_off, size))
            src_off += size
        return segments

    def _segment_of(self, shard_id: int):
        return self._segments()[shard_id]


class QKVParallelLinear(_PackedColumnParallel):
    """Fused q/k/v projection; heads are split over ranks.  Shard ids ``"q" | "k" | "v"``."""

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int,
                 total_num_kv_heads: int | None = None, bias: bool = False,
                 quantization: str | None = None):
        _, world = _tp_coordinates()
        total_num_kv_heads = total_num_kv_heads or total_num_heads
        self.head_size = head_size
        self.num_heads = divide(total_num_heads, world)
        self.num_kv_heads = divide(total_num_kv_heads, world)
        out = (total_num_heads + 2 * total_num_kv_heads) * head_size
        super().__init__(hidden_size, out, bias, quantization)

    def qkv_shards(self):
        q = self.num_heads * self.head_size
        kv = self.num_kv_heads * self.head_size
        t = self.tp_size
        return ((0, q, 0, q * t),
                (q, kv, q * t, kv * t),
                (q + kv, kv, (q + kv) * t, kv * t))

    def _segments(self):
        return self.qkv_shards()

    def _segment_of(self, shard_id: str):
        assert shard_id in ("q", "k", "v")
        return self.qkv_shards()["qkv".index(shard_id)]


class RowParallelLinear(LinearBase):
    """Input features split over ranks; partial results are summed by all-reduce."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False,
                 quantization: str | None = None):
        _, world = _tp_coordinates()
        super().__init__(divide(input_size, world), output_size, bias, 1, quantization)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        local = param.data.size(self.tp_dim)
        param.data.copy_(loaded_weight.narrow(self.tp_dim, self.tp_rank * local, local))

    def scales_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        param.data.copy_(loaded_weight)  # one scale per output channel: replicated

    def shard_plan(self, kind: str, stored_shape: tuple, *shard_id):
        if kind in ("weight", "qweight"):
            cols = stored_shape[1]
            return _segment_plan(1, 2, [(0, cols // self.tp_size, 0, cols)], self.tp_rank, self.tp_size)
        return super().shard_plan(kind, stored_shape)    # scales and bias are replicated

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bias = self.bias if self.tp_rank == 0 else None
        comm = _peer_all_reduce if self.tp_size > 1 else None
        if self.quant_method is None:
            y = F.linear(x, self.weight, bias)
        else:
            if comm is not None and x.is_cuda and hasattr(comm, "fused_fits"):
                # decode-sized batch: GEMM and the sum over ranks in one kernel
                fused = self.quant_method.apply_row_parallel(x, self, bias, comm)
                if fused is not None:
                    return fused
            # As in the reference (linear.py:270-271 with int8.py:29 / w8a8.py:37): a
            # ``None`` bias lets the quant method pick ``self.bias`` on every rank.
            y = self.quant_method.apply(x, self, bias)
        if self.tp_size > 1:
            if comm is not None:
                return comm.reduce(y)
            dist.all_reduce(y)
        return y

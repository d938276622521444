"""Tensor-parallel linear layers (bf16/fp32 weights; torch GEMMs, and for decode-sized inputs of at
most 8 rows the library's weight-streaming kernel `fdms_linear_decode`, `FDMS_DECODE_LINEAR=0` turns
it off).

Same class names, parameter layout and `weight_loader` protocol as the reference's
`fastdms/layers/linear.py` (:946-1048), so checkpoints load the same way: QKV and gate/up are
packed column-parallel weights, o_proj/down_proj are row-parallel and all-reduce their output over
the tensor-parallel group: at decode sizes in one launch with the projection (`fdms_linear_decode_allreduce`,
see `layers/peer_allreduce.py`), otherwise with NCCL.  Other decode-size forms: the gate_up projection with its
activation (`gated_linear`), weight-only FP8 (`LinearBase.quantize_fp8`, `Config.fp8_weights`).  The reference's
activation-quantised FP8 and its int4 weight paths are not part of the compact-DMS decode path and are not
provided.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from fastdms_b200 import _lib

_DECODE_LINEAR = os.environ.get("FDMS_DECODE_LINEAR", "1") != "0"


# Opt-in: the fused norm + linear launch measured SLOWER in the 1B decode step (0.91 against 0.78 ms per
# graph replay): every CTA of the projection recomputes the row statistics and the normalised input
# after the dependency wait, which costs more than the chained RMSNorm launch it removes.
_FUSE_NORM = os.environ.get("FDMS_FUSE_NORM_LINEAR", "0") == "1"
_GATED_LINEAR = os.environ.get("FDMS_GATED_LINEAR", "1") != "0"      # gate_up + SiLU * up in one launch


def _decode_linear_ok(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> bool:
    return (_DECODE_LINEAR and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype
            and x.dim() == 2 and 0 < x.shape[0] <= 8 and x.stride(1) == 1 and weight.is_contiguous()
            and weight.shape[0] % 16 == 0 and weight.shape[0] < 65536 and weight.shape[1] % 2048 == 0
            and x.shape[1] == weight.shape[1] and (bias is None or bias.dtype == x.dtype)
            and x.data_ptr() % 16 == 0 and (x.stride(0) * 2) % 16 == 0 and weight.data_ptr() % 16 == 0
            and not torch.is_grad_enabled())


def norm_linear(x: torch.Tensor, residual: torch.Tensor | None, norm, lin) -> tuple[torch.Tensor, torch.Tensor]:
    """`h, r = norm(x, residual); return lin(h), r` of a decoder block (`norm` an RMSNorm, `lin` a
    column-parallel linear layer; with `residual=None` the new residual is `x`, as in the reference's
    `models/llama.py` decoder layer).  With `FDMS_FUSE_NORM_LINEAR=1` decode-sized 16-bit
    inputs take ONE launch of `fdms_linear_decode_norm`; otherwise the two modules run."""
    w, b = lin.weight, lin.bias
    if (_FUSE_NORM and _decode_linear_ok(x, w, b) and norm.weight.dtype == x.dtype and norm.weight.is_contiguous()
            and norm.weight.data_ptr() % 16 == 0
            and (residual is None or (residual.dtype == x.dtype and residual.shape == x.shape and residual.stride(1) == 1
                                      and residual.data_ptr() % 16 == 0 and (residual.stride(0) * 2) % 16 == 0))):
        rows, n = x.shape[0], w.shape[0]
        y = torch.empty((rows, n), dtype=x.dtype, device=x.device)
        res_out = torch.empty_like(x) if residual is not None else None
        with torch.cuda.device(x.device):
            rc = _lib.lib().fdms_linear_decode_norm(
                x.data_ptr(), x.stride(0), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
                norm.weight.data_ptr(), float(norm.eps), _lib.ptr(res_out), res_out.stride(0) if res_out is not None else 0,
                w.data_ptr(), w.stride(0), b.data_ptr() if b is not None else None, y.data_ptr(), y.stride(0),
                _lib.dtype_code(x.dtype), rows, n, w.shape[1], _lib.stream_ptr(x.device))
        _lib.check(rc)
        return y, (res_out if residual is not None else x)
    if residual is None:
        h, r = norm(x), x
    else:
        h, r = norm(x, residual)
    return lin(h), r


def quantize_weight_fp8(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-output-column FP8 quantisation of a [out, in] weight: returns (e4m3 bytes, float32 scale per
    row, the dequantised weight in the original dtype).  scale = absmax / 448, stored = w / scale."""
    w = weight.detach().float()
    scale = (w.abs().amax(dim=1) / 448.0).clamp_min(1e-12).contiguous()
    w8 = (w / scale[:, None]).to(torch.float8_e4m3fn).contiguous()
    return w8, scale, (w8.float() * scale[:, None]).to(weight.dtype)


def linear_fp8(x: torch.Tensor, weight_fp8: torch.Tensor, scale: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """One launch of `fdms_linear_decode_fp8` (decode-sized 16-bit input, FP8 weights)."""
    rows, n = x.shape[0], weight_fp8.shape[0]
    y = torch.empty((rows, n), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().fdms_linear_decode_fp8(
            x.data_ptr(), x.stride(0), weight_fp8.data_ptr(), weight_fp8.stride(0), scale.data_ptr(), _lib.ptr(bias),
            y.data_ptr(), y.stride(0), _lib.dtype_code(x.dtype), rows, n, weight_fp8.shape[1], _lib.stream_ptr(x.device))
    _lib.check(rc)
    return y


def _fp8_linear_ok(x: torch.Tensor, w8: torch.Tensor, bias: torch.Tensor | None) -> bool:
    return (_DECODE_LINEAR and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.dim() == 2
            and 0 < x.shape[0] <= 8 and x.stride(1) == 1 and w8.shape[0] % 16 == 0 and w8.shape[1] % 2048 == 0
            and x.shape[1] == w8.shape[1] and (bias is None or bias.dtype == x.dtype)
            and x.data_ptr() % 16 == 0 and (x.stride(0) * 2) % 16 == 0 and not torch.is_grad_enabled())


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """`F.linear`, except that 16-bit CUDA inputs of at most 8 rows go through one launch of
    `fdms_linear_decode` (weights streamed once, f32 accumulation) when the shapes allow it; very wide
    outputs (the LM head) stay on the library GEMM, which streams them faster."""
    if _decode_linear_ok(x, weight, bias):
        rows, n = x.shape[0], weight.shape[0]
        y = torch.empty((rows, n), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            rc = _lib.lib().fdms_linear_decode(
                x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0),
                bias.data_ptr() if bias is not None else None, y.data_ptr(), y.stride(0),
                _lib.dtype_code(x.dtype), rows, n, weight.shape[1], _lib.stream_ptr(x.device))
        _lib.check(rc)
        return y
    return F.linear(x, weight, bias)


def gated_linear(x: torch.Tensor, lin) -> torch.Tensor | None:
    """`SiluAndMul(lin(x))` for a merged gate_up projection (gate rows first, then up rows) in ONE launch of
    `fdms_linear_decode_gated` when the decode linear kernel applies (same bits as the two launches), else None."""
    w, b = lin.weight, lin.bias
    if (not _GATED_LINEAR or getattr(lin, "weight_fp8", None) is not None or not _decode_linear_ok(x, w, b)
            or w.shape[0] % 32 != 0):
        return None
    # The gated launch has one CTA per 16 gate + 16 up columns.  Between one and two waves of such CTAs the plain
    # projection (twice as many CTAs of half the work) plus the activation launch is faster: measured on the 8B
    # shape, 384 CTAs (TP = 2) 2.46 against 2.41 ms per step, 192 CTAs (TP = 4) 2.10 against 2.19, 768 (one GPU)
    # 3.84 against 3.88, 512 (1B shape) 0.81 against 0.84.
    if 256 <= w.shape[0] // 32 < 512:
        return None
    rows, n = x.shape[0], w.shape[0]
    y = torch.empty((rows, n // 2), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().fdms_linear_decode_gated(
            x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), b.data_ptr() if b is not None else None,
            y.data_ptr(), y.stride(0), _lib.dtype_code(x.dtype), rows, n, w.shape[1], _lib.stream_ptr(x.device))
    _lib.check(rc)
    return y


def norm_gated_linear(x: torch.Tensor, residual: torch.Tensor | None, norm, lin, act_fn) -> tuple[torch.Tensor, torch.Tensor]:
    """`h, r = norm(x, residual); return act_fn(lin(h)), r` of a decoder block's MLP entry, with the projection and
    the activation in one launch at decode sizes."""
    if _FUSE_NORM:
        gate_up, r = norm_linear(x, residual, norm, lin)
        return act_fn(gate_up), r
    if residual is None:
        h, r = norm(x), x
    else:
        h, r = norm(x, residual)
    y = gated_linear(h, lin)
    return (y if y is not None else act_fn(lin(h))), r


_REPLICA_MODE = False


def set_replica_mode(enabled: bool) -> None:
    """Replica mode: every rank of the job holds the whole model (sequence sharding); the process
    group is then only used to exchange results, never by the layers."""
    global _REPLICA_MODE
    _REPLICA_MODE = bool(enabled)


def tp_world() -> tuple[int, int]:
    """(tensor-parallel size, rank) seen by the layers: the process group, or (1, 0) without one or
    in replica mode."""
    if not _REPLICA_MODE and dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def divide(a: int, b: int) -> int:
    assert a % b == 0, f"{a} is not divisible by {b}"
    return a // b


class LinearBase(nn.Module):
    def __init__(self, input_size: int, output_size: int, bias: bool = False, tp_dim: int | None = None):
        super().__init__()
        self.tp_dim = tp_dim
        self.tp_size, self.tp_rank = tp_world()
        self.weight = nn.Parameter(torch.empty(output_size, input_size))
        self.weight.weight_loader = self.weight_loader
        if bias:
            self.bias = nn.Parameter(torch.empty(output_size))
            self.bias.weight_loader = self.weight_loader
        else:
            self.register_parameter("bias", None)

        self.weight_fp8 = None          # set by quantize_fp8(): e4m3 copy of the weight and its per-row scale
        self.weight_scale = None

    def quantize_fp8(self) -> None:
        """Keeps an FP8 copy of the weight for decode-sized inputs and replaces the 16-bit weight by its
        dequantised value, so that prefill (library GEMM) and decode (FP8 stream) use the same numbers."""
        w8, scale, deq = quantize_weight_fp8(self.weight.data)
        self.weight_fp8, self.weight_scale = w8, scale
        self.weight.data.copy_(deq)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.weight_fp8 is not None and _fp8_linear_ok(x, self.weight_fp8, self.bias):
            return linear_fp8(x, self.weight_fp8, self.weight_scale, self.bias)
        return linear(x, self.weight, self.bias)


class ReplicatedLinear(LinearBase):
    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        param.data.copy_(loaded_weight)


class ColumnParallelLinear(LinearBase):
    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        tp_size, _ = tp_world()
        super().__init__(input_size, divide(output_size, tp_size), bias, 0)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        shard = param.data.size(0)
        param.data.copy_(loaded_weight.narrow(0, self.tp_rank * shard, shard))


class MergedColumnParallelLinear(ColumnParallelLinear):
    def __init__(self, input_size: int, output_sizes: list[int], bias: bool = False):
        self.output_sizes = output_sizes
        super().__init__(input_size, sum(output_sizes), bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: int):
        offset = sum(self.output_sizes[:loaded_shard_id]) // self.tp_size
        size = self.output_sizes[loaded_shard_id] // self.tp_size
        param.data.narrow(0, offset, size).copy_(loaded_weight.chunk(self.tp_size, 0)[self.tp_rank])


class QKVParallelLinear(ColumnParallelLinear):
    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int,
                 total_num_kv_heads: int | None = None, bias: bool = False):
        tp_size, _ = tp_world()
        total_num_kv_heads = total_num_kv_heads or total_num_heads
        self.head_size = head_size
        self.num_heads = divide(total_num_heads, tp_size)
        self.num_kv_heads = divide(total_num_kv_heads, tp_size)
        super().__init__(hidden_size, (total_num_heads + 2 * total_num_kv_heads) * head_size, bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: str):
        assert loaded_shard_id in ("q", "k", "v")
        qs, ks = self.num_heads * self.head_size, self.num_kv_heads * self.head_size
        offset, size = {"q": (0, qs), "k": (qs, ks), "v": (qs + ks, ks)}[loaded_shard_id]
        param.data.narrow(0, offset, size).copy_(loaded_weight.chunk(self.tp_size, 0)[self.tp_rank])


class RowParallelLinear(LinearBase):
    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        tp_size, _ = tp_world()
        super().__init__(divide(input_size, tp_size), output_size, bias, 1)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        if param.data.ndim == 1:
            param.data.copy_(loaded_weight)
            return
        shard = param.data.size(1)
        param.data.copy_(loaded_weight.narrow(1, self.tp_rank * shard, shard))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            from fastdms_b200.layers.peer_allreduce import fused_row_parallel, tp_all_reduce_
            fused = fused_row_parallel()
            if fused is not None and _DECODE_LINEAR and fused.fits(x, self.weight, self.bias):
                # decode-sized input: GEMM and all-reduce in one launch (the bias is added once, after the sum)
                return fused.linear_all_reduce(x, self.weight, self.bias)
            y = linear(x, self.weight, self.bias if self.tp_rank == 0 else None)
            tp_all_reduce_(y)
            return y
        return LinearBase.forward(self, x)

"""One-shot all-reduce over NVLink peer memory for the small tensors of tensor-parallel decode (the
library's `fdms_allreduce_oneshot`) and the row-parallel linear layer fused with it
(`fdms_linear_decode_allreduce`), with the plumbing they need: every rank allocates one region, shares its
CUDA IPC handle over the process group and opens its peers' handles with its own device current (the
library's `fdms_ipc_region_*`).  Tensors that do not fit, or that are not 16-byte friendly, go through
`torch.distributed.all_reduce`.

The reference sums tensor-parallel partials with NCCL (fastdms/layers/linear.py:1044-1048); the
result here is the sum in rank order, identical on every rank."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from fastdms_b200 import _lib

_STATE = None
_FUSED = None


class _PeerRegions:
    """One zero-filled device region per rank, mapped into every rank (collective over the group)."""

    def __init__(self, device: torch.device, group, nbytes: int):
        import ctypes
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        if not (2 <= self.world <= 8):
            raise ValueError(f"peer regions support 2..8 ranks, got {self.world}")
        if nbytes <= 0:
            raise ValueError("bad region size")
        lib = _lib.lib()
        self._own = ctypes.c_void_p()
        self._opened: list[int] = []
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):         # everything below happens with this rank's device current
            _lib.check(lib.fdms_ipc_region_create(nbytes, ctypes.byref(self._own), handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(self._own.value)
                    continue
                # The mapping belongs to the device that is current while the handle is opened, so it
                # is opened here, under this rank's device, not under the exporting rank's index.
                p = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                _lib.check(lib.fdms_ipc_region_open(buf, ctypes.byref(p)))
                self._opened.append(p.value)
                ptrs.append(p.value)
        self.ptrs = torch.tensor(ptrs, dtype=torch.int64)      # host array of pointers, indexed by rank
        dist.barrier(group=group)            # every rank has mapped every region before anyone uses them

    def close(self) -> None:
        """Unmaps the peers' regions and frees this rank's (collective: no rank may still be inside a call)."""
        if self._own.value is None:
            return
        dist.barrier(group=self.group)
        lib = _lib.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p in self._opened:
                lib.fdms_ipc_region_close(p)
            self._opened = []
            dist.barrier(group=self.group)
            lib.fdms_ipc_region_destroy(self._own)
        self._own = type(self._own)()



class PeerAllReduce(_PeerRegions):
    def __init__(self, device: torch.device, group=None, max_bytes: int = 1 << 20):
        self.max_bytes = int(max_bytes)
        world = dist.get_world_size(group)
        super().__init__(device, group, _lib.lib().fdms_allreduce_region_bytes(world, self.max_bytes))

    def fits(self, t: torch.Tensor) -> bool:
        nb = t.numel() * t.element_size()
        return (t.is_cuda and t.is_contiguous() and t.dtype in (torch.float32, torch.bfloat16, torch.float16)
                and 0 < nb <= self.max_bytes and nb % 16 == 0 and t.data_ptr() % 16 == 0)

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        """In-place sum over the ranks (the same call, with the same shape, on every rank)."""
        with torch.cuda.device(self.device):
            rc = _lib.lib().fdms_allreduce_oneshot(
                self.ptrs.data_ptr(), self.rank, self.world, self.max_bytes, t.data_ptr(), t.data_ptr(), t.numel(),
                _lib.dtype_code(t.dtype), _lib.status_word(self.device).data_ptr(), _lib.stream_ptr(self.device))
        _lib.check(rc)
        return t


class FusedRowParallel(_PeerRegions):
    """The row-parallel linear layer of tensor-parallel decode and its all-reduce in one launch per rank
    (`fdms_linear_decode_allreduce`): CTAs push float32 partial tiles into every rank's region and sum
    them in rank order, so all ranks hold identical results.  The reference does F.linear followed by
    NCCL's all_reduce (fastdms/layers/linear.py:1044-1048)."""

    def __init__(self, device: torch.device, group=None):
        world = dist.get_world_size(group)
        super().__init__(device, group, _lib.lib().fdms_linear_allreduce_region_bytes(world))

    @staticmethod
    def fits(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> bool:
        n, k = weight.shape
        steps = k // 256
        ks = 1
        while ks * 2 <= 8 and ks * 2 <= steps:
            ks *= 2
        ctas = -(-(n // 16) // (8 // ks)) if k % 256 == 0 and steps > 0 else 1 << 30
        return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype and x.dim() == 2
                and 0 < x.shape[0] <= 8 and x.stride(1) == 1 and weight.is_contiguous() and n % 16 == 0 and k % 256 == 0
                and ctas <= 512 and x.shape[1] == k and (bias is None or bias.dtype == x.dtype)
                and x.data_ptr() % 16 == 0 and (x.stride(0) * 2) % 16 == 0 and weight.data_ptr() % 16 == 0
                and not torch.is_grad_enabled())

    def linear_all_reduce(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        """sum over ranks of x_r @ weight_r.T (+ bias once): the same call on every rank."""
        rows, n = x.shape[0], weight.shape[0]
        y = torch.empty((rows, n), dtype=x.dtype, device=x.device)
        with torch.cuda.device(self.device):
            rc = _lib.lib().fdms_linear_decode_allreduce(
                x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _lib.ptr(bias), y.data_ptr(), y.stride(0),
                _lib.dtype_code(x.dtype), rows, n, weight.shape[1], self.ptrs.data_ptr(), self.rank, self.world,
                _lib.status_word(self.device).data_ptr(), _lib.stream_ptr(self.device))
        _lib.check(rc)
        return y


def init_fused_row_parallel(device, group=None):
    """Sets up the fused linear + all-reduce for this process (collective over the group).  On by
    default under tensor parallelism (measured on two B200s inside a replayed graph: 6.2 us per o_proj call of
    the 8B shape against 15.3 us for the decode linear kernel followed by NCCL, 3.9 us for the linear kernel
    alone; the 8B decode step 2.68 against 3.52 ms); `FDMS_FUSED_ROW_PARALLEL=0` keeps the two-step path."""
    global _FUSED
    _FUSED = None
    if os.environ.get("FDMS_FUSED_ROW_PARALLEL", "1").strip().lower() in {"0", "false", "off", "no"}:
        return None
    if not dist.is_initialized() or dist.get_world_size(group) < 2:
        return None
    _FUSED = FusedRowParallel(device, group)
    return _FUSED


def fused_row_parallel():
    return _FUSED


def init_peer_all_reduce(device, group=None, max_bytes: int = 1 << 20):
    """Sets up the peer all-reduce for this process (collective over the group); returns it, or None
    when it is not switched on (`FDMS_PEER_ALLREDUCE=1`) or there is a single rank.  It serves the
    all-reduces that are not fused into a row-parallel layer (which is the default for o_proj and down_proj at
    decode sizes).  Measured on two B200s for a [8, 4096] bf16 tensor: 9.8 us against NCCL's 17.7 us per eager
    call; inside a replayed graph, after the decode linear kernel, 10.2 us against 15.3 us for the pair."""
    global _STATE
    _STATE = None
    if os.environ.get("FDMS_PEER_ALLREDUCE", "0").strip().lower() not in {"1", "true", "on", "yes"}:
        return None
    if not dist.is_initialized() or dist.get_world_size(group) < 2:
        return None
    _STATE = PeerAllReduce(device, group, max_bytes)
    return _STATE


def tp_all_reduce_(t: torch.Tensor) -> torch.Tensor:
    """Sum over the tensor-parallel ranks, in place: peer kernel when it is set up and the tensor fits,
    NCCL otherwise."""
    if _STATE is not None and _STATE.fits(t):
        return _STATE.all_reduce_(t)
    dist.all_reduce(t)
    return t

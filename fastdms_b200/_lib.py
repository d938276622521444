"""ctypes binding of libfastdms_b200.so (the C ABI declared in include/fastdms_b200.h).

The library is the product: there is no CPU or PyTorch fallback.  `lib()` raises if the shared
object is missing (build it with `python -m fastdms_b200.build` or `__graft_entry__.build()`).
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_double, c_float, c_int32, c_int64, c_void_p
from pathlib import Path

import torch

import os

# FDMS_B200_LIB selects another build of the same library (the probe build of `build.py --probe`)
LIB_PATH = Path(os.environ.get("FDMS_B200_LIB") or Path(__file__).resolve().parent / "libfastdms_b200.so")

FDMS_OK = 0
FDMS_E_ARG, FDMS_E_DTYPE, FDMS_E_WORKSPACE, FDMS_E_CUDA, FDMS_E_CAPACITY = -1, -2, -3, -4, -5
DEV_WAIT_TIMEOUT, DEV_BAD_INDEX = 1, 2
ATTN_OVERLAP_PREVIOUS = 1

F32, BF16, F16, E4M3 = 0, 1, 2, 3
_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16, torch.float8_e4m3fn: E4M3}

P, I32, I64, F, DBL = c_void_p, c_int32, c_int64, c_float, c_double

# name -> (restype, argtypes); the order is the order of the C declaration
_SIGNATURES = {
    "fdms_abi_version": (I32, []),
    "fdms_last_error": (c_char_p, []),
    "fdms_attn_decode_workspace_bytes": (I64, [I32, I32, I32]),
    "fdms_attn_decode": (I32, [P, I32, I64, I64, P, P, I32, I64, P, P, I64, P, I64, I64, I32, P, P,
                               P, I32, I64, I64, I32, I32, I32, I32, F, P, P, I64, I64, P, I64, I32, P, P]),
    "fdms_attn_decode_append": (I32, [P, P, P, I32, I64, I64, I64, I64, I64, I64, P, P, I32, I64, P, P, I64,
                                      P, I64, I64, I32, P, P, P, I64, I64, P, P, I64, DBL, DBL, P, I32, I64, I64,
                                      I32, I32, I32, I32, F, P, I64, I32, P, P]),
    "fdms_attn_decode_noalloc": (I32, [P, I32, I64, I64, P, P, I32, I64, P, P, I64, P, I64, I64, I32, P, P,
                                       P, I32, I64, I64, I32, I32, I32, I32, F, P, P, I64, I64, P, P]),
    "fdms_store_decode": (I32, [P, I64, I64, P, I64, I64, P, I64, I64, I32, P, I64, I64, P, P, P, I32, I64,
                                P, I64, P, I64, P, P, I32, I32, I32, I32, DBL, DBL, I32, I32, I32, I32, P, P]),
    "fdms_extract_decisions": (I32, [P, I32, I64, I64, P, I64, I64, I32, I32, I32, DBL, DBL, P]),
    "fdms_expire_compact": (I32, [P, I64, I64, I64, P, I64, I64, I64, P, P, P, I64, I64, P, P, I64, I32, I64,
                                  P, I64, I64, I64, P, P, I64, P, P, I32, I32, I32, I32, I32, I32, P, P, P, P]),
    "fdms_pack_count": (I32, [P, I64, P, P, P, I32, I32, I32, I32, P]),
    "fdms_pack_scatter": (I32, [P, P, I32, I64, I64, P, I64, P, P, I32, P, P, P, I32, I64, P, I64,
                                P, I64, I64, P, P, I64, I64, P, I64, I64, P, I64, I32, P, P,
                                I32, I32, I32, I32, P, P]),
    "fdms_pack_scatter_append": (I32, [P, P, I32, I64, I64, P, I64, P, P, I32, P, P, P, P, P, I32, I64, P, I64,
                                       P, I64, I64, P, P, I64, I64, P, I64, I64, P, I64, I32, P, P,
                                       I32, I32, I32, I32, P, P]),
    "fdms_prefix_attention": (I32, [P, I32, I64, I64, P, I32, P, P, I32, I64, P, P, I64, P, I64, I64, I32,
                                    P, P, P, P, I64, I64, P, I64, I64, P, I64, I64, I32, I32, I32, I32, F, P, P]),
    "fdms_alloc_pages": (I32, [P, P, I64, I64, I32, P, P, P, I32, I32, P, P]),
    "fdms_grow_pages": (I32, [P, P, P, I64, I64, I32, P, P, P, I32, I32, P, P]),
    "fdms_free_pages": (I32, [P, I64, P, I64, I64, I32, P, P, P, I64, I32, I32, P, P]),
    "fdms_build_decode_metadata": (I32, [P, P, I64, I64, P, I64, I64, I64, I32, P, P, I64, P,
                                         P, P, P, P, I32, I32, I32, P, P]),
    "fdms_record_decisions": (I32, [P, I64, I64, I64, P, I64, I64, I64, P, I64, I64, P, I64, I64, P, P,
                                    I32, I32, I32, I32, P, I32, P]),
    "fdms_kv_quant": (I32, [P, I32, P, P, I64, I32, I32, P]),
    "fdms_kv_dequant": (I32, [P, P, I32, P, I64, I32, I32, P]),
    "fdms_rmsnorm": (I32, [P, I64, P, I64, P, P, I64, P, I64, I32, I64, I32, F, P]),
    "fdms_silu_and_mul": (I32, [P, I64, P, I64, I32, I64, I32, P]),
    "fdms_qk_rmsnorm": (I32, [P, I64, I64, I32, P, P, I64, I64, I32, P, I32, I64, I32, F, P]),
    "fdms_linear_decode": (I32, [P, I64, P, I64, P, P, I64, I32, I32, I32, I32, P]),
    "fdms_linear_decode_gated": (I32, [P, I64, P, I64, P, P, I64, I32, I32, I32, I32, P]),
    "fdms_linear_decode_norm": (I32, [P, I64, P, I64, P, F, P, I64, P, I64, P, P, I64, I32, I32, I32, I32, P]),
    "fdms_argmax_workspace_bytes": (I64, [I64]),
    "fdms_argmax_rows": (I32, [P, I64, I32, I64, I64, P, P, I64, P]),
    "fdms_allreduce_region_bytes": (I64, [I32, I64]),
    "fdms_enable_peer_access": (I32, [I32]),
    "fdms_ipc_region_create": (I32, [I64, P, P]),
    "fdms_ipc_region_open": (I32, [P, P]),
    "fdms_ipc_region_close": (I32, [P]),
    "fdms_ipc_region_destroy": (I32, [P]),
    "fdms_allreduce_oneshot": (I32, [P, I32, I32, I64, P, P, I64, I32, P, P]),
    "fdms_linear_decode_fp8": (I32, [P, I64, P, I64, P, P, P, I64, I32, I32, I32, I32, P]),
    "fdms_linear_allreduce_region_bytes": (I64, [I32]),
    "fdms_linear_decode_allreduce": (I32, [P, I64, P, I64, P, P, I64, I32, I32, I32, I32, P, I32, I32, P, P]),
}

_lib = None


def exported_symbols() -> list[str]:
    return list(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """The loaded library; raises RuntimeError when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: the fastdms_b200 CUDA library has not been built "
                "(run `python -m fastdms_b200.build`); there is no fallback path")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ValueError(f"unsupported dtype {dt}") from None


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def check(status: int) -> None:
    """Maps a C status to the reference's exception classes (ValueError for argument/shape/dtype
    problems, RuntimeError for state/capacity/CUDA problems)."""
    if status == FDMS_OK:
        return
    msg = lib().fdms_last_error().decode("utf-8", "replace")
    if status in (FDMS_E_ARG, FDMS_E_DTYPE, FDMS_E_WORKSPACE):
        raise ValueError(msg)
    raise RuntimeError(msg)


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("fastdms_b200 kernels require CUDA tensors (there is no CPU fallback)")


# ---- per-device scratch owned by the Python layer (the C library allocates nothing) ------------
_status_words: dict[int, torch.Tensor] = {}
_workspaces: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        # an ordinary tensor even when the first caller runs under inference mode (the engine does): callers
        # outside it clear the word in place
        with torch.inference_mode(False):
            w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[idx] = w
    return w


def read_device_status(device: torch.device | str = "cuda", clear: bool = True) -> int:
    """Synchronising read of the device status word (OR of FDMS_DEV_* bits raised by kernels)."""
    device = torch.device(device)
    w = status_word(device)
    v = int(w.item())
    if clear and v:
        w.zero_()
    return v


# Sized for the largest problem the fast kernels accept (65 535 spans, head_dim 256): about 8.7 MB.
_WS_MAX_SPANS, _WS_MAX_HEAD_DIM = 65535, 256
_retired_workspaces: list[torch.Tensor] = []


def attn_workspace(device: torch.device, batch: int, num_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Zero-initialised split-K workspace, one per device (the kernel leaves its counters at zero).

    CUDA graphs captured by the engine hold the workspace's raw address, so the tensor is allocated
    ONCE per device at the size of the largest problem the fast kernels take and is never replaced
    by a bigger one while smaller batches' graphs may still point at it.  A request beyond that size
    (not reachable through the fast kernels) gets a larger tensor and the old one is kept alive.
    Launches that use the workspace are ordered by the stream they run on; callers that drive
    several streams at once must pass their own workspace instead."""
    need = lib().fdms_attn_decode_workspace_bytes(batch, num_kv_heads, head_dim)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None or ws.numel() < need:
        full = lib().fdms_attn_decode_workspace_bytes(_WS_MAX_SPANS, 1, _WS_MAX_HEAD_DIM)
        if ws is not None:
            _retired_workspaces.append(ws)          # graphs captured earlier may still reference it
        with torch.inference_mode(False):
            ws = torch.zeros(max(need, full), dtype=torch.uint8, device=device)
        _workspaces[idx] = ws
    return ws

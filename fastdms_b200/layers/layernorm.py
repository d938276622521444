"""RMSNorm with optional fused residual add (float32 statistics, result in the input dtype), as in
the reference's `fastdms/layers/layernorm.py`.  16-bit CUDA activations take one launch of the
library's `fdms_rmsnorm`; float32 (the reference's CPU-checkable configuration) stays on torch ops
because that path reproduces the reference's aliasing exactly."""
from __future__ import annotations

import torch
from torch import nn

from fastdms_b200 import _lib


def _fused_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype
            and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192 and x.stride(-1) == 1 and x.numel() > 0)


def _rows(t: torch.Tensor) -> torch.Tensor:
    """[rows, hidden] view with a single row stride (copy only if the layout needs one)."""
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.stride(-1) == 1 else t2.contiguous()


def rmsnorm_cuda(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """One launch: returns `out` or `(out, new_residual)` when `residual` is given."""
    x2 = _rows(x)
    rows, hidden = x2.shape
    out = torch.empty((rows, hidden), dtype=x.dtype, device=x.device)
    res2 = res_out = None
    if residual is not None:
        res2 = _rows(residual)
        res_out = torch.empty((rows, hidden), dtype=x.dtype, device=x.device)
    ok = all(t is None or (t.data_ptr() % 16 == 0 and (t.stride(0) * 2) % 16 == 0) for t in (x2, res2)) and \
        weight.data_ptr() % 16 == 0 and weight.is_contiguous()
    if not ok:
        return None
    with torch.cuda.device(x.device):
        rc = _lib.lib().fdms_rmsnorm(
            x2.data_ptr(), x2.stride(0), _lib.ptr(res2), res2.stride(0) if res2 is not None else 0, weight.data_ptr(),
            out.data_ptr(), out.stride(0), _lib.ptr(res_out), res_out.stride(0) if res_out is not None else 0,
            _lib.dtype_code(x.dtype), rows, hidden, float(eps), _lib.stream_ptr(x.device))
    _lib.check(rc)
    out = out.view(x.shape)
    return out if residual is None else (out, res_out.view(x.shape))


def qk_rmsnorm_(q: torch.Tensor, k: torch.Tensor, q_norm: "RMSNorm", k_norm: "RMSNorm") -> bool:
    """Per-head RMSNorm of q [rows, heads, head_dim] and k [rows, kv_heads, head_dim] (views into the fused
    projection output are fine) in ONE launch of `fdms_qk_rmsnorm`, in place.  Returns False, having done
    nothing, when the tensors do not qualify (the caller then applies the two modules)."""
    d = q.shape[-1]
    ok = (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and k.dtype == q.dtype and q.dim() == 3 and k.dim() == 3
          and k.shape[-1] == d and k.shape[0] == q.shape[0] and d % 8 == 0 and d <= 256 and q.stride(2) == 1 and k.stride(2) == 1
          and q_norm.weight.dtype == q.dtype and k_norm.weight.dtype == q.dtype and q_norm.eps == k_norm.eps
          and q_norm.weight.is_contiguous() and k_norm.weight.is_contiguous() and q.numel() > 0
          and not torch.is_grad_enabled()
          and all(v % 16 == 0 for v in (q.data_ptr(), k.data_ptr(), q_norm.weight.data_ptr(), k_norm.weight.data_ptr(),
                                        q.stride(0) * 2, q.stride(1) * 2, k.stride(0) * 2, k.stride(1) * 2)))
    if not ok:
        return False
    with torch.cuda.device(q.device):
        rc = _lib.lib().fdms_qk_rmsnorm(
            q.data_ptr(), q.stride(0), q.stride(1), q.shape[1], q_norm.weight.data_ptr(),
            k.data_ptr(), k.stride(0), k.stride(1), k.shape[1], k_norm.weight.data_ptr(),
            _lib.dtype_code(q.dtype), q.shape[0], d, float(q_norm.eps), _lib.stream_ptr(q.device))
    _lib.check(rc)
    return True


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        dtype = x.dtype
        if _fused_ok(x, self.weight) and (residual is None or (residual.dtype == dtype and residual.shape == x.shape)):
            y = rmsnorm_cuda(x, self.weight, self.eps, residual)
            if y is not None:
                return y
        if residual is None:
            xf = x.float()
            y = (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self.eps)).to(dtype) * self.weight
            if dtype == torch.float32:
                # The reference normalises in place (layernorm.py:16-25); in float32 `.float()` is an
                # alias, so the caller's input -- which it keeps as the residual -- becomes the
                # output.  Reproduced so that float32 models match it exactly.
                x.copy_(y)
                return x
            return y
        xf = x.float() + residual.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self.eps)).to(dtype) * self.weight
        if dtype == torch.float32:
            return y, y                    # same aliasing: the new residual is the normalised output
        return y, xf.to(dtype)

"""RMSNorm with optional fused residual add (float32 statistics, result in the input dtype), as in
the reference's `fastdms/layers/layernorm.py`; plain torch ops (outside the CUDA hot path)."""
from __future__ import annotations

import torch
from torch import nn


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        dtype = x.dtype
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

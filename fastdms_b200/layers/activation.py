import torch
import torch.nn.functional as F
from torch import nn


class SiluAndMul(nn.Module):
    """silu(x[..., :n]) * x[..., n:] on the fused gate/up projection."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a, b = x.chunk(2, -1)
        return F.silu(a) * b

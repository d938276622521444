import torch
import torch.nn.functional as F
from torch import nn

from fastdms_b200 import _lib


class SiluAndMul(nn.Module):
    """silu(x[..., :n]) * x[..., n:] on the fused gate/up projection (reference:
    fastdms/layers/activation.py); one launch of `fdms_silu_and_mul` for 16-bit CUDA activations."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n = x.shape[-1] // 2
        if (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.shape[-1] % 2 == 0 and n % 8 == 0
                and x.stride(-1) == 1 and x.numel() > 0):
            x2 = x.reshape(-1, x.shape[-1])
            if x2.stride(-1) == 1 and x2.data_ptr() % 16 == 0 and (x2.stride(0) * 2) % 16 == 0:
                out = torch.empty((x2.shape[0], n), dtype=x.dtype, device=x.device)
                with torch.cuda.device(x.device):
                    rc = _lib.lib().fdms_silu_and_mul(x2.data_ptr(), x2.stride(0), out.data_ptr(), out.stride(0),
                                                      _lib.dtype_code(x.dtype), x2.shape[0], n, _lib.stream_ptr(x.device))
                _lib.check(rc)
                return out.view(*x.shape[:-1], n)
        a, b = x.chunk(2, -1)
        return F.silu(a) * b

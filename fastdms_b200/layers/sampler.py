import torch
from torch import nn

from fastdms_b200 import _lib


def argmax_workspace(rows: int, device) -> torch.Tensor:
    """Zeroed scratch for `greedy_argmax` on up to `rows` rows; every call leaves it zeroed, so one
    buffer serves all calls of a stream (a captured decode step keeps its own)."""
    return torch.zeros(max(int(_lib.lib().fdms_argmax_workspace_bytes(rows)), 16), dtype=torch.uint8, device=device)


def greedy_argmax(logits: torch.Tensor, workspace: torch.Tensor | None = None,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """`logits.argmax(dim=-1)` of a `[rows, vocab]` CUDA tensor in one launch of the library's
    `fdms_argmax_rows` (lowest index on ties, NaN largest, like torch); other inputs take torch's.
    `out` (int64 [rows], contiguous) receives the result in place, e.g. the token-id buffer the next
    decode step reads."""
    if not (logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1 and 0 < logits.shape[0] < 65536
            and logits.shape[1] > 0 and logits.dtype in (torch.float32, torch.bfloat16, torch.float16)):
        res = logits.argmax(dim=-1)
        return res if out is None else out.copy_(res)
    rows, n = logits.shape
    ws = workspace if workspace is not None else argmax_workspace(rows, logits.device)
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    elif out.dtype != torch.int64 or out.shape != (rows,) or not out.is_contiguous():
        raise ValueError("out must be a contiguous int64 tensor with one element per row")
    with torch.cuda.device(logits.device):
        rc = _lib.lib().fdms_argmax_rows(logits.data_ptr(), logits.stride(0), _lib.dtype_code(logits.dtype), rows, n,
                                         out.data_ptr(), ws.data_ptr(), ws.numel(), _lib.stream_ptr(logits.device))
    _lib.check(rc)
    return out


class Sampler(nn.Module):
    """Temperature sampling with the exponential-race trick (same distribution as the reference's
    `fastdms/layers/sampler.py`); greedy requests bypass it with an argmax."""

    def forward(self, logits: torch.Tensor, temperatures: torch.Tensor) -> torch.Tensor:
        logits = logits.float() / temperatures.unsqueeze(1)
        probs = torch.softmax(logits, dim=-1)
        return (probs / torch.empty_like(probs).exponential_(1).clamp_min_(1e-10)).argmax(dim=-1)

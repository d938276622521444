import torch
from torch import nn


class Sampler(nn.Module):
    """Temperature sampling with the exponential-race trick (same distribution as the reference's
    `fastdms/layers/sampler.py`); greedy requests bypass it with an argmax."""

    def forward(self, logits: torch.Tensor, temperatures: torch.Tensor) -> torch.Tensor:
        logits = logits.float() / temperatures.unsqueeze(1)
        probs = torch.softmax(logits, dim=-1)
        return (probs / torch.empty_like(probs).exponential_(1).clamp_min_(1e-10)).argmax(dim=-1)

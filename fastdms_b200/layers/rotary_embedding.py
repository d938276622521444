"""Rotary position embedding (neox / half-split form) and its cos|sin cache.

Same construction as the reference's `fastdms/layers/rotary_embedding.py`: the cache is
`[max_position, 1, head_dim]` float32 holding cos (first half) and sin (second half); llama3
frequency scaling is supported.  In decode the rotation is applied by the fused store kernel;
this module's forward is the prefill path (plain float32 torch ops, rounded to the input dtype).
"""
from __future__ import annotations

import math

import torch
from torch import nn


def apply_rotary_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    x1, x2 = torch.chunk(x.float(), 2, dim=-1)
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat((y1, y2), dim=-1).to(x.dtype)


def _llama3_scaling(inv_freq, factor, low_freq_factor, high_freq_factor, original_max_position):
    low_wavelen = original_max_position / low_freq_factor
    high_wavelen = original_max_position / high_freq_factor
    wavelen = 2 * math.pi / inv_freq
    scaled = inv_freq / factor
    smooth = (original_max_position / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    mid = (1.0 - smooth) * scaled + smooth * inv_freq
    out = torch.where(wavelen < high_wavelen, inv_freq, mid)
    return torch.where(wavelen > low_wavelen, scaled, out)


class RotaryEmbedding(nn.Module):
    def __init__(self, head_size: int, rotary_dim: int, max_position_embeddings: int, base: float,
                 rope_scaling: dict | None = None) -> None:
        super().__init__()
        assert rotary_dim == head_size
        self.head_size = head_size
        inv_freq = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float, device="cpu") / rotary_dim))
        if rope_scaling is not None:
            kind = rope_scaling.get("rope_type") or rope_scaling.get("type")
            if kind == "llama3":
                inv_freq = _llama3_scaling(
                    inv_freq, float(rope_scaling["factor"]), float(rope_scaling.get("low_freq_factor", 1.0)),
                    float(rope_scaling.get("high_freq_factor", 4.0)),
                    int(rope_scaling["original_max_position_embeddings"]))
            elif kind == "linear":
                inv_freq = inv_freq / float(rope_scaling.get("factor", 1.0))
            elif kind not in (None, "default"):
                raise NotImplementedError(f"rope_type={kind!r} is not implemented")
        t = torch.arange(max_position_embeddings, dtype=torch.float, device="cpu")
        freqs = torch.einsum("i,j -> ij", t, inv_freq)
        cache = torch.cat((freqs.cos(), freqs.sin()), dim=-1).unsqueeze_(1)
        self.register_buffer("cos_sin_cache", cache, persistent=False)

    def forward(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor):
        cos, sin = self.cos_sin_cache[positions].chunk(2, dim=-1)
        return apply_rotary_emb(query, cos, sin), apply_rotary_emb(key, cos, sin)


_ROPE_CACHE: dict[tuple, RotaryEmbedding] = {}


def get_rope(head_size: int, rotary_dim: int, max_position: int, base: float, rope_scaling: dict | None = None):
    key = (head_size, rotary_dim, max_position, base,
           None if rope_scaling is None else tuple(sorted((k, tuple(v) if isinstance(v, list) else v)
                                                          for k, v in rope_scaling.items())))
    rope = _ROPE_CACHE.get(key)
    if rope is None:
        rope = RotaryEmbedding(head_size, rotary_dim, max_position, base, rope_scaling)
        _ROPE_CACHE[key] = rope
    return rope

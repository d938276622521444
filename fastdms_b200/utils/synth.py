"""Deterministic synthetic weights for random-init models.

Values come from an integer hash of (seed, parameter name, element index), so they are
bit-identical on every machine and library version; no checkpoint or random stream is involved.
Used for the benchmark shapes and for the parity fixtures (the same generator fills the
reference's model when the golden traces are made)."""
from __future__ import annotations

import zlib

import numpy as np
import torch


def hashed_uniform(name: str, shape, seed: int = 0) -> np.ndarray:
    """float32 array in [-1, 1) determined by (seed, name, index); splitmix64 finaliser."""
    n = int(np.prod(shape)) if len(shape) else 1
    key = np.uint64(zlib.crc32(name.encode()) ^ (seed * 0x9E3779B1 & 0xFFFFFFFF))
    x = np.arange(n, dtype=np.uint64) + (key << np.uint64(32))
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15))
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        x = x ^ (x >> np.uint64(31))
    u = (x >> np.uint64(40)).astype(np.float64) / float(1 << 24)      # 24 random bits -> [0, 1)
    return (u * 2.0 - 1.0).astype(np.float32).reshape(shape)


def synth_tensor(name: str, shape, std: float, seed: int = 0) -> torch.Tensor:
    """Uniform values with the requested standard deviation (uniform[-a, a] has std a / sqrt(3))."""
    return torch.from_numpy(hashed_uniform(name, tuple(shape), seed) * np.float32(std * 3.0 ** 0.5))


def synth_llama_state_dict(cfg: dict, seed: int = 0, *, evict_rate: float | None = 7.0 / 8.0,
                           alpha_scale: float = 100.0, alpha_offset: float = 5.0) -> dict[str, torch.Tensor]:
    """State dict (HF-style names: q_proj/k_proj/v_proj/o_proj, gate/up/down_proj, norms, embed,
    lm_head) of a Llama/Qwen3-shaped model described by `cfg` (hidden_size, intermediate_size,
    num_hidden_layers, num_attention_heads, num_key_value_heads, head_dim, vocab_size,
    attention_bias, qk_norm).  float32 tensors.

    When `evict_rate` is given the DMS decision channel (last channel of the first q head of every
    GQA group) is wired so that about that fraction of tokens is marked for eviction: its weight
    row is scaled to give a unit-variance pre-activation and its bias is placed at the matching
    quantile above the threshold alpha_offset / alpha_scale (requires attention_bias)."""
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    Hq, Hk, D, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    G = Hq // Hk
    sd: dict[str, torch.Tensor] = {}
    sd["model.embed_tokens.weight"] = synth_tensor("embed", (V, H), 1.0, seed)
    sd["lm_head.weight"] = synth_tensor("lm_head", (V, H), cfg.get("lm_head_std", 0.5), seed)
    if cfg.get("lm_head_factor") is not None:       # float32 product, applied before any cast of the weights
        sd["lm_head.weight"] = sd["lm_head.weight"] * float(cfg["lm_head_factor"])
    sd["model.norm.weight"] = torch.ones(H)
    w_std = H ** -0.5
    for l in range(L):
        p = f"model.layers.{l}."
        q = synth_tensor(p + "q", (Hq * D, H), w_std, seed)
        sd[p + "self_attn.k_proj.weight"] = synth_tensor(p + "k", (Hk * D, H), w_std, seed)
        sd[p + "self_attn.v_proj.weight"] = synth_tensor(p + "v", (Hk * D, H), w_std, seed)
        sd[p + "self_attn.o_proj.weight"] = synth_tensor(p + "o", (H, Hq * D), (Hq * D) ** -0.5, seed)
        if cfg.get("attention_bias", False):
            qb = torch.zeros(Hq * D)
            if evict_rate is not None:
                # inverse normal CDF by bisection on erf (no scipy dependency)
                import math
                lo, hi = -6.0, 6.0
                for _ in range(60):
                    mid = 0.5 * (lo + hi)
                    if 0.5 * (1.0 + math.erf(mid / math.sqrt(2.0))) < evict_rate:
                        lo = mid
                    else:
                        hi = mid
                shift = alpha_offset / alpha_scale + 0.5 * (lo + hi)
                for h in range(Hk):
                    qb[(h * G) * D + D - 1] = shift
            sd[p + "self_attn.q_proj.bias"] = qb
            sd[p + "self_attn.k_proj.bias"] = torch.zeros(Hk * D)
            sd[p + "self_attn.v_proj.bias"] = torch.zeros(Hk * D)
            sd[p + "self_attn.o_proj.bias"] = torch.zeros(H)
        sd[p + "self_attn.q_proj.weight"] = q
        if cfg.get("qk_norm", False):
            sd[p + "self_attn.q_norm.weight"] = torch.ones(D)
            sd[p + "self_attn.k_norm.weight"] = torch.ones(D)
        sd[p + "mlp.gate_proj.weight"] = synth_tensor(p + "gate", (I, H), w_std, seed)
        sd[p + "mlp.up_proj.weight"] = synth_tensor(p + "up", (I, H), w_std, seed)
        sd[p + "mlp.down_proj.weight"] = synth_tensor(p + "down", (H, I), I ** -0.5, seed)
        sd[p + "input_layernorm.weight"] = torch.ones(H)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H)
    return sd

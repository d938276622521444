"""Attention layer: the boundary between the model and the compact-DMS kernels.

Mirrors the reference's `fastdms/layers/attention.py` for the compact path: module attributes
`compact_k_cache`, `compact_v_cache`, `layer_id`; `forward(q, k, v, *, compact_append_stored,
compact_q_rope, positions, cos_sin_cache)`; per-step inputs come from the global Context.
Prefill attention is dense and causal (eviction only decides what is packed into the compact
pool); it runs through torch's scaled_dot_product_attention per sequence.  The reference's dense
paged KV branches do not exist here: compact-DMS mode allocates no dense blocks.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from fastdms_b200.layers.compact_attention import (compact_decode_attention, compact_prefix_attention,
                                                   fused_store_decode_attention, store_compact_kvcache)
from fastdms_b200.utils.context import get_context
from fastdms_b200.utils.profiler import get_profiler


def dense_causal_prefill(q, k, v, cu_seqlens: list[int], scale: float) -> torch.Tensor:
    """q [T, Hq, D], k/v [T, Hk, D] of several packed sequences -> [T, Hq, D]."""
    out = torch.empty_like(q)
    gqa = q.shape[1] != k.shape[1]
    for i in range(len(cu_seqlens) - 1):
        s, e = cu_seqlens[i], cu_seqlens[i + 1]
        if e <= s:
            continue
        o = F.scaled_dot_product_attention(
            q[s:e].transpose(0, 1).unsqueeze(0), k[s:e].transpose(0, 1).unsqueeze(0),
            v[s:e].transpose(0, 1).unsqueeze(0), is_causal=True, scale=scale, enable_gqa=gqa)
        out[s:e] = o.squeeze(0).transpose(0, 1)
    return out


def dense_causal_prefill_lse(q, k, v, cu_seqlens: list[int], scale: float):
    """As `dense_causal_prefill`, also returning the natural-log log-sum-exp of the scaled scores,
    float32 [Hq, T] (what the prefill-tail kernel needs to merge the compact prefix in).  16-bit CUDA
    activations go through torch's flash kernel, which reports it; anything else through plain
    float32 matrix ops."""
    T, Hq, _ = q.shape
    out = torch.empty_like(q)
    lse = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
    G = Hq // k.shape[1]
    for i in range(len(cu_seqlens) - 1):
        s, e = cu_seqlens[i], cu_seqlens[i + 1]
        if e <= s:
            continue
        qq, kk, vv = (x[s:e].transpose(0, 1).unsqueeze(0) for x in (q, k, v))
        if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
            if G > 1:
                kk, vv = kk.repeat_interleave(G, dim=1), vv.repeat_interleave(G, dim=1)
            res = torch.ops.aten._scaled_dot_product_flash_attention(qq, kk, vv, 0.0, True, False, scale=scale)
            out[s:e] = res[0].squeeze(0).transpose(0, 1)
            lse[:, s:e] = res[1].squeeze(0)[:, :e - s]
            continue
        sc = (qq.squeeze(0).float() @ kk.squeeze(0).float().repeat_interleave(G, dim=0).transpose(1, 2)) * scale
        sc = sc.masked_fill(~torch.tril(torch.ones(e - s, e - s, dtype=torch.bool, device=q.device)), float("-inf"))
        lse[:, s:e] = torch.logsumexp(sc, dim=-1)
        out[s:e] = (torch.softmax(sc, dim=-1) @ vv.squeeze(0).float().repeat_interleave(G, dim=0)).transpose(0, 1).to(q.dtype)
    return out, lse


class Attention(nn.Module):
    def __init__(self, num_heads, head_dim, scale, num_kv_heads):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_kv_heads = num_kv_heads
        self.compact_k_cache = self.compact_v_cache = torch.tensor([])
        self.compact_k_scale = self.compact_v_scale = None
        self.layer_id = -1

    def can_fuse_store(self) -> bool:
        """True when decision + RoPE + FP8 store + attention can run as one launch for this layer."""
        return (self.compact_k_cache.numel() > 0 and self.compact_k_cache.dtype == torch.float8_e4m3fn
                and self.head_dim in (64, 128) and self.num_heads // self.num_kv_heads <= 8)

    def forward_fused_store(self, q, k, v, *, positions, cos_sin_cache, evict_out, alpha_scale, alpha_offset):
        """Decode only: q/k/v are pre-RoPE; appends the new row to the compact pool and attends."""
        context = get_context()
        if context.is_prefill or not context.compact_kv_enabled:
            raise RuntimeError("forward_fused_store is a compact-KV decode operation")
        if context.compact_base_offsets is None or context.compact_live_counts is None:
            raise RuntimeError("compact KV decode requires compact_base_offsets and compact_live_counts")
        base, live, bt = context.compact_base_offsets, context.compact_live_counts, context.compact_block_tables
        if base.ndim == 3:
            base, live = base[self.layer_id], live[self.layer_id]
        if bt is not None and bt.ndim == 4:
            bt = bt[self.layer_id]
        with get_profiler().cuda_phase("compact_store_decode_attn"):
            return fused_store_decode_attention(
                q, k, v, cos_sin_cache, self.compact_k_cache, self.compact_v_cache, base, live, evict_out, positions,
                num_kv_heads=self.num_kv_heads, alpha_scale=alpha_scale, alpha_offset=alpha_offset, scale=self.scale,
                block_tables=bt, k_scale=self.compact_k_scale, v_scale=self.compact_v_scale,
                overlap_previous_kernel=context.overlap_store_and_attention)

    def forward(self, q, k, v, *, compact_append_stored: bool = False, compact_q_rope: bool = False,
                positions: torch.Tensor | None = None, cos_sin_cache: torch.Tensor | None = None):
        context = get_context()
        prof = get_profiler()
        if context.is_prefill:
            cu = context.cu_seqlens_host
            if cu is None:
                cu = context.cu_seqlens_q.tolist()
            if context.compact_prefix_slots is not None:
                # a chunk of a longer prompt: its own causal block, then the rows the spans already hold
                m = context.streaming_pack_manager
                with prof.cuda_phase("dense_prefill_attn"):
                    out, lse = dense_causal_prefill_lse(q, k, v, cu, self.scale)
                with prof.cuda_phase("prefix_attn"):
                    l = self.layer_id
                    return compact_prefix_attention(
                        q, self.compact_k_cache, self.compact_v_cache,
                        None if m.paged else m.layer_major_base_offsets[l], m.layer_major_live_counts[l],
                        context.cu_seqlens_q, context.max_seqlen_q, out, lse, self.scale,
                        seq_slots=context.compact_prefix_slots,
                        block_tables=m.block_tables[l] if m.paged else None,
                        k_scale=self.compact_k_scale, v_scale=self.compact_v_scale)
            with prof.cuda_phase("dense_prefill_attn"):
                return dense_causal_prefill(q, k, v, cu, self.scale)
        if not context.compact_kv_enabled:
            raise RuntimeError("decode requires the compact KV path (compact_kv_enabled)")
        if context.compact_base_offsets is None or context.compact_live_counts is None:
            raise RuntimeError("compact KV decode requires compact_base_offsets and compact_live_counts")
        base, live, slot = context.compact_base_offsets, context.compact_live_counts, context.compact_slot_mapping
        bt = context.compact_block_tables
        if base.ndim == 3:
            base, live = base[self.layer_id], live[self.layer_id]
            slot = None if slot is None else slot[self.layer_id]
        if bt is not None and bt.ndim == 4:
            bt = bt[self.layer_id]
        if slot is not None and not compact_append_stored:
            with prof.cuda_phase("compact_append_store"):
                store_compact_kvcache(k, v, self.compact_k_cache, self.compact_v_cache, slot,
                                      k_scale=self.compact_k_scale, v_scale=self.compact_v_scale)
        with prof.cuda_phase("compact_decode_attn"):
            return compact_decode_attention(
                q, self.compact_k_cache, self.compact_v_cache, base, live, scale=self.scale,
                max_live_count=context.compact_max_live_count or None,
                q_rope_positions=positions if compact_q_rope else None,
                q_rope_cos_sin_cache=cos_sin_cache if compact_q_rope else None,
                block_tables=bt, k_scale=self.compact_k_scale, v_scale=self.compact_v_scale,
                overlap_previous_kernel=context.overlap_store_and_attention and compact_append_stored)

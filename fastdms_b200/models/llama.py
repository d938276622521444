"""Llama-family decoder whose attention block runs the compact-DMS decode path.

Module and parameter names follow the reference's `fastdms/models/llama.py`; the attention block's
`forward` reproduces its ordering (llama.py:87-202):
  decode : qkv -> [fused DMS decision + RoPE + FP8 append store] -> compact attention -> o_proj
  prefill: qkv -> decision extraction -> RoPE -> prefill pack into the compact pool -> dense causal
           attention -> o_proj
GEMMs, norms and the activation are torch ops; everything between qkv_proj and o_proj is this
library's CUDA code.
"""
from __future__ import annotations

import torch
from torch import nn

from fastdms_b200.engine.dms import extract_dms_eviction_decisions
from fastdms_b200.layers.activation import SiluAndMul
from fastdms_b200.layers.attention import Attention
from fastdms_b200.layers.compact_attention import (dms_decode_store_transient_k_enabled,
                                                   fused_dms_rope_store_compact_decode,
                                                   fused_store_attention_enabled)
from fastdms_b200.layers.embed_head import ParallelLMHead, VocabParallelEmbedding
from fastdms_b200.layers.layernorm import RMSNorm, qk_rmsnorm_
from fastdms_b200.layers.linear import (MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear,
                                        norm_gated_linear, norm_linear, tp_world)
from fastdms_b200.layers.rotary_embedding import get_rope
from fastdms_b200.utils.context import get_context
from fastdms_b200.utils.profiler import get_profiler


def _rope_config(config) -> tuple[float, dict | None]:
    rope_scaling = getattr(config, "rope_scaling", None) or getattr(config, "rope_parameters", None)
    rope_theta = getattr(config, "rope_theta", None) or 10000
    if isinstance(rope_scaling, dict):
        rope_theta = rope_scaling.get("rope_theta", rope_theta)
        rope_scaling = {k: v for k, v in rope_scaling.items() if k != "rope_theta"}
        if "rope_type" not in rope_scaling and "type" in rope_scaling:
            rope_scaling["rope_type"] = rope_scaling["type"]
        if not rope_scaling or rope_scaling.get("rope_type") in (None, "default"):
            rope_scaling = None
    return rope_theta, rope_scaling


class LlamaAttention(nn.Module):
    qk_norm = False

    def __init__(self, config) -> None:
        super().__init__()
        tp_size, _ = tp_world()
        self.total_num_heads = config.num_attention_heads
        self.total_num_kv_heads = config.num_key_value_heads
        assert self.total_num_heads % tp_size == 0 and self.total_num_kv_heads % tp_size == 0
        self.num_heads = self.total_num_heads // tp_size
        self.num_kv_heads = self.total_num_kv_heads // tp_size
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // self.total_num_heads
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.scaling = self.head_dim ** -0.5
        bias = getattr(config, "attention_bias", False)
        self.qkv_proj = QKVParallelLinear(config.hidden_size, self.head_dim, self.total_num_heads,
                                          self.total_num_kv_heads, bias=bias)
        self.o_proj = RowParallelLinear(self.total_num_heads * self.head_dim, config.hidden_size, bias=bias)
        rope_theta, rope_scaling = _rope_config(config)
        self.rotary_emb = get_rope(self.head_dim, rotary_dim=self.head_dim,
                                   max_position=config.max_position_embeddings, base=rope_theta,
                                   rope_scaling=rope_scaling)
        self.attn = Attention(self.num_heads, self.head_dim, self.scaling, self.num_kv_heads)
        if self.qk_norm:
            self.q_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps)
            self.k_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps)

    def forward(self, positions: torch.Tensor, hidden_states: torch.Tensor | None,
                qkv: torch.Tensor | None = None) -> torch.Tensor:
        """`qkv` given: the projection was already taken (fused with the preceding norm)."""
        if qkv is None:
            qkv = self.qkv_proj(hidden_states)
        q, k, v = qkv.split([self.q_size, self.kv_size, self.kv_size], dim=-1)
        q = q.view(-1, self.num_heads, self.head_dim)
        k = k.view(-1, self.num_kv_heads, self.head_dim)
        v = v.view(-1, self.num_kv_heads, self.head_dim)
        if self.qk_norm:                      # Qwen3: per-head RMSNorm before the decision is read
            if not qk_rmsnorm_(q, k, self.q_norm, self.k_norm):     # one launch, in place in the projection output
                q = self.q_norm(q)
                k = self.k_norm(k)
        context = get_context()
        prof = get_profiler()
        cache = self.rotary_emb.cos_sin_cache
        layer_id = self.attn.layer_id
        fused = False
        evict_mask = None
        if context.dms_capture_enabled:
            if layer_id < 0:
                raise RuntimeError("DMS capture requires assigned attention layer ids")
            evict_out = None
            if context.dms_layer_evictions_buffer is not None:
                evict_out = context.dms_layer_evictions_buffer[layer_id]
            can_fuse = (not context.is_prefill and context.compact_kv_enabled
                        and context.compact_slot_mapping is not None and self.attn.compact_k_cache.numel() > 0)
            if context.dms_layer_evictions is None and evict_out is None and not can_fuse:
                raise RuntimeError("DMS capture requires a layer eviction recorder")
            if can_fuse:
                slot = context.compact_slot_mapping
                if slot.ndim == 3:
                    slot = slot[layer_id]
                if evict_out is None:
                    evict_out = torch.empty((q.shape[0], self.num_kv_heads), device=q.device, dtype=torch.bool)
                if (self.attn.can_fuse_store() and not dms_decode_store_transient_k_enabled()
                        and fused_store_attention_enabled()):
                    if context.dms_layer_evictions is not None:
                        context.dms_layer_evictions[layer_id] = evict_out
                    o = self.attn.forward_fused_store(
                        q, k, v, positions=positions, cos_sin_cache=cache, evict_out=evict_out,
                        alpha_scale=context.dms_alpha_scale, alpha_offset=context.dms_alpha_offset)
                    return self.o_proj(o.flatten(1, -1))
                with prof.cuda_phase("dms_rope_store"):
                    fused_dms_rope_store_compact_decode(
                        q, k, v, cache, self.attn.compact_k_cache, self.attn.compact_v_cache, slot, evict_out,
                        positions, num_kv_heads=self.num_kv_heads, alpha_scale=context.dms_alpha_scale,
                        alpha_offset=context.dms_alpha_offset, store_q=True,
                        store_transient_k=dms_decode_store_transient_k_enabled(),
                        k_scale=self.attn.compact_k_scale, v_scale=self.attn.compact_v_scale)
                evict_mask = evict_out
                fused = True
            else:
                with prof.cuda_phase("dms_capture"):
                    q, evict_mask = extract_dms_eviction_decisions(
                        q, num_kv_heads=self.num_kv_heads, num_qo_heads=self.num_heads, head_dim=self.head_dim,
                        alpha_scale=context.dms_alpha_scale, alpha_offset=context.dms_alpha_offset,
                        inplace=True, out=evict_out)
            if context.dms_layer_evictions is not None:
                context.dms_layer_evictions[layer_id] = evict_mask
        if not fused:
            q, k = self.rotary_emb(positions, q, k)
        pack = (context.is_prefill and context.streaming_pack_manager is not None
                and context.streaming_pack_seq_ids and context.dms_capture_enabled)
        chunked = pack and context.prefill_chunk_starts is not None
        o = None
        if chunked:
            # the chunk attends to what the spans held BEFORE it is packed (expiry + append follow)
            o = self.attn(q, k, v, compact_append_stored=fused, compact_q_rope=False, positions=positions,
                          cos_sin_cache=cache)
        if pack:
            with prof.cuda_phase("streaming_pack"):
                context.streaming_pack_manager.streaming_pack_layer(
                    layer_id=layer_id, k=k, v=v, evict_mask=evict_mask, cu_seqlens_q=context.cu_seqlens_q,
                    seq_ids=context.streaming_pack_seq_ids, window_size=context.streaming_pack_window_size,
                    chunk_starts=context.prefill_chunk_starts, remaining=context.prefill_chunk_remaining)
        if o is None:
            o = self.attn(q, k, v, compact_append_stored=fused, compact_q_rope=False, positions=positions,
                          cos_sin_cache=cache)
        return self.o_proj(o.flatten(1, -1))


class LlamaMLP(nn.Module):
    def __init__(self, config) -> None:
        super().__init__()
        bias = getattr(config, "mlp_bias", False)
        self.gate_up_proj = MergedColumnParallelLinear(config.hidden_size, [config.intermediate_size] * 2, bias=bias)
        self.down_proj = RowParallelLinear(config.intermediate_size, config.hidden_size, bias=bias)
        assert getattr(config, "hidden_act", "silu") == "silu"
        self.act_fn = SiluAndMul()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(self.act_fn(self.gate_up_proj(x)))


class LlamaDecoderLayer(nn.Module):
    attention_cls = LlamaAttention

    def __init__(self, config) -> None:
        super().__init__()
        self.self_attn = self.attention_cls(config)
        self.mlp = LlamaMLP(config)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, positions, hidden_states, residual):
        # norm -> projection pairs go through `norm_linear` (the two modules; one fused launch is an opt-in)
        qkv, residual = norm_linear(hidden_states, residual, self.input_layernorm, self.self_attn.qkv_proj)
        hidden_states = self.self_attn(positions, None, qkv=qkv)
        act, residual = norm_gated_linear(hidden_states, residual, self.post_attention_layernorm, self.mlp.gate_up_proj,
                                          self.mlp.act_fn)
        hidden_states = self.mlp.down_proj(act)
        return hidden_states, residual


class LlamaModel(nn.Module):
    layer_cls = LlamaDecoderLayer

    def __init__(self, config) -> None:
        super().__init__()
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([self.layer_cls(config) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        hidden_states = self.embed_tokens(input_ids)
        residual = None
        for layer in self.layers:
            hidden_states, residual = layer(positions, hidden_states, residual)
        hidden_states, _ = self.norm(hidden_states, residual)
        return hidden_states


class LlamaForCausalLM(nn.Module):
    model_cls = LlamaModel
    packed_modules_mapping = {
        "q_proj": ("qkv_proj", "q"),
        "k_proj": ("qkv_proj", "k"),
        "v_proj": ("qkv_proj", "v"),
        "gate_proj": ("gate_up_proj", 0),
        "up_proj": ("gate_up_proj", 1),
    }

    def __init__(self, config) -> None:
        super().__init__()
        self.model = self.model_cls(config)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size)
        if getattr(config, "tie_word_embeddings", False):
            self.lm_head.weight.data = self.model.embed_tokens.weight.data
        for i, layer in enumerate(self.model.layers):
            layer.self_attn.attn.layer_id = i

    def attention_modules(self) -> list[Attention]:
        return [layer.self_attn.attn for layer in self.model.layers]

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        return self.model(input_ids, positions)

    def compute_logits(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.lm_head(hidden_states)

"""Qwen3 decoder: the Llama block plus per-head RMSNorm of q and k before the DMS decision is read
and before RoPE (reference: fastdms/models/qwen3.py:92-94)."""
from __future__ import annotations

from fastdms_b200.models.llama import LlamaAttention, LlamaDecoderLayer, LlamaForCausalLM, LlamaModel


class Qwen3Attention(LlamaAttention):
    qk_norm = True


class Qwen3DecoderLayer(LlamaDecoderLayer):
    attention_cls = Qwen3Attention


class Qwen3Model(LlamaModel):
    layer_cls = Qwen3DecoderLayer


class Qwen3ForCausalLM(LlamaForCausalLM):
    model_cls = Qwen3Model

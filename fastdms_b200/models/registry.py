from __future__ import annotations

from fastdms_b200.models.llama import LlamaForCausalLM
from fastdms_b200.models.qwen3 import Qwen3ForCausalLM

_MODELS = {"llama": LlamaForCausalLM, "qwen3": Qwen3ForCausalLM}


def build_model(hf_config):
    """Model class by `model_type` (reference: fastdms/models/registry.py)."""
    kind = getattr(hf_config, "model_type", "llama")
    if kind not in _MODELS:
        raise ValueError(f"unsupported model_type {kind!r}; supported: {sorted(_MODELS)}")
    return _MODELS[kind](hf_config)

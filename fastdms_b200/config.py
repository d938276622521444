"""Engine configuration.  Field names follow the reference's `fastdms/config.py` for everything
the compact-DMS path uses; dense-KV, FP8-weight and hub-download options are not carried over.
`model` is a local Hugging Face style directory (config.json, optional *.safetensors, optional
tokenizer files) or, with `hf_config` given, just a label."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from types import SimpleNamespace

import torch

_KV_CACHE_DTYPES = {
    "auto": None,
    "float16": torch.float16,
    "bfloat16": torch.bfloat16,
    "float32": torch.float32,
    "float8_e4m3fn": torch.float8_e4m3fn,
}
_MODEL_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _as_namespace(cfg):
    if isinstance(cfg, dict):
        return SimpleNamespace(**cfg)
    return cfg


@dataclass(slots=True)
class Config:
    model: str
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 512
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    tensor_parallel_size: int = 1
    enforce_eager: bool = False
    hf_config: object | None = None
    eos: int = -1
    kv_cache_dtype: str = "auto"
    compact_kv_enabled: bool = True
    compact_kv_capacity_tokens: int = 0
    compact_kv_retention_mode: str = "dms"
    dms_metadata_path: str | None = None
    dms_window_size: int | None = None
    dms_alpha_scale: float | None = None
    dms_alpha_offset: float | None = None
    compact_kv_budget_bytes: int | None = None
    compact_kv_target_live_tokens_per_seq: int | None = None
    compact_kv_layer_major_metadata: bool = True
    # additions
    compact_kv_paged: bool = False            # 16-row pages + GPU free stack instead of first-fit spans
    dms_expiry_interval: int = 1              # 1 = exact expiry every step; N = when position % N == 0
    compact_kv_row_indirection: bool = True   # expiry compacts metadata only and refills freed K/V rows
    compact_kv_admission: str = "reserve"     # "reserve": worst case per request; "optimistic": estimate + retry
    compact_kv_admission_keep_estimate: float = 0.25
    prefill_chunk_size: int | None = None          # prompts are prefilled in chunks of this many tokens (None: one pass)
    fp8_weights: bool = False                 # linear layers keep an FP8 e4m3 copy (per-column scale) that decode-sized inputs stream
    decode_run_ahead: bool = False            # greedy decode: next step launched from device-resident tokens before this step's are read
    random_init_seed: int | None = None       # synthetic weights when the directory has no safetensors
    dtype: str | None = None                  # overrides the checkpoint's dtype

    def __post_init__(self):
        assert 1 <= self.tensor_parallel_size <= 8
        assert self.kv_cache_dtype in _KV_CACHE_DTYPES, (
            f"kv_cache_dtype must be one of {sorted(_KV_CACHE_DTYPES)}, got {self.kv_cache_dtype!r}")
        if self.compact_kv_retention_mode != "dms" or not self.compact_kv_enabled:
            raise ValueError("only the compact-DMS mode (compact_kv_enabled, retention mode 'dms') is provided")
        if self.dms_window_size is not None:
            assert self.dms_window_size >= 0
        if self.dms_alpha_scale is not None:
            assert self.dms_alpha_scale != 0.0
        if self.hf_config is None:
            path = os.path.join(os.fspath(self.model), "config.json")
            if not os.path.isfile(path):
                raise ValueError(f"model must be a local checkpoint directory with config.json, got {self.model!r}")
            with open(path, encoding="utf-8") as f:
                self.hf_config = SimpleNamespace(**json.load(f))
        else:
            self.hf_config = _as_namespace(self.hf_config)
        hc = self.hf_config
        if not hasattr(hc, "head_dim") or hc.head_dim is None:
            hc.head_dim = hc.hidden_size // hc.num_attention_heads
        self.max_model_len = min(self.max_model_len, hc.max_position_embeddings)

    def model_dtype(self) -> torch.dtype:
        name = self.dtype or getattr(self.hf_config, "torch_dtype", None) or getattr(self.hf_config, "dtype", None) or "bfloat16"
        if isinstance(name, torch.dtype):
            return name
        return _MODEL_DTYPES[str(name).removeprefix("torch.")]

    def resolve_kv_cache_dtype(self) -> torch.dtype:
        return _KV_CACHE_DTYPES[self.kv_cache_dtype] or self.model_dtype()

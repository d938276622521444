"""DMS semantics: decision extraction, live-mask construction and checkpoint metadata.

Mirrors the reference's `fastdms/engine/dms.py`; the extraction runs in the CUDA library.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path

import torch

from fastdms_b200 import _lib


@dataclass(frozen=True, slots=True)
class DMSMetadata:
    """Runtime DMS parameters of a checkpoint (reference: dms.py:45-59)."""
    model_path: str
    source_path: str
    source_kind: str
    packaged_metadata_found: bool
    window_size: int
    alpha_scale: float
    alpha_offset: float
    target_cr: int | None = None
    context_len: int | None = None
    compression_mode: str | None = None

    def to_dict(self) -> dict:
        return asdict(self)


def _from_config(model_path, source_path, kind, packaged, cfg: dict) -> DMSMetadata:
    def pick(*names, default=None):
        for n in names:
            if n in cfg:
                return cfg[n]
        return default

    target_cr = pick("target_cr", "dms_cr")
    context_len = pick("context_len", "max_position_embeddings")
    return DMSMetadata(
        model_path=str(model_path), source_path=str(source_path), source_kind=kind,
        packaged_metadata_found=packaged,
        window_size=int(pick("window_size", "dms_window_size", default=256)),
        alpha_scale=float(pick("alpha_scale", "dms_alpha_scale", default=100.0)),
        alpha_offset=float(pick("alpha_offset", "dms_alpha_offset", "dms_initial_alpha_offset", default=5.0)),
        target_cr=None if target_cr is None else int(target_cr),
        context_len=None if context_len is None else int(context_len),
        compression_mode=cfg.get("compression_mode"),
    )


def load_dms_metadata(model_path, metadata_path=None) -> DMSMetadata:
    """Looks for DMS parameters in, in order: an explicit file, `dms_metadata.json` next to the
    weights, the parent's `training_log.json`, DMS keys of `config.json` (reference: dms.py:92-149)."""
    model_path = Path(model_path)
    if metadata_path is not None:
        path = Path(metadata_path)
        data = json.loads(path.read_text(encoding="utf-8"))
        return _from_config(model_path, path, "explicit_metadata", path.name == "dms_metadata.json",
                            data.get("config", data))
    packaged = model_path / "dms_metadata.json"
    if packaged.exists():
        data = json.loads(packaged.read_text(encoding="utf-8"))
        return _from_config(model_path, packaged, "packaged_metadata", True, data.get("config", data))
    training_log = model_path.parent / "training_log.json"
    if training_log.exists():
        data = json.loads(training_log.read_text(encoding="utf-8"))
        return _from_config(model_path, training_log, "parent_training_log", False, data.get("config", {}))
    hf_config = model_path / "config.json"
    if hf_config.exists():
        data = json.loads(hf_config.read_text(encoding="utf-8"))
        if any(k in data for k in ("dms_window_size", "dms_alpha_scale", "dms_initial_alpha_offset", "dms_cr")):
            return _from_config(model_path, hf_config, "hf_config_dms", False, data)
    raise FileNotFoundError(f"no DMS metadata found for {model_path}; expected {packaged} or {training_log}")


def extract_dms_eviction_decisions(
    q: torch.Tensor,
    *,
    num_kv_heads: int,
    num_qo_heads: int,
    head_dim: int,
    alpha_scale: float,
    alpha_offset: float,
    inplace: bool = False,
    out: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-KV-head eviction decisions from the borrowed q channel (last channel of the first q
    head of each GQA group), which is zeroed.  Returns (q_clean, evict[tokens, kv_heads]); True
    means "evict once outside the window" (reference: dms.py:152-232)."""
    if num_qo_heads % num_kv_heads != 0:
        raise ValueError(f"num_qo_heads={num_qo_heads} must be divisible by num_kv_heads={num_kv_heads}")
    if q.ndim == 2:
        if q.shape[1] != num_qo_heads * head_dim:
            raise ValueError(f"expected flat q width {num_qo_heads * head_dim}, got {q.shape[1]}")
    elif q.ndim == 3:
        if q.shape[1:] != (num_qo_heads, head_dim):
            raise ValueError(f"expected q shape [tokens, {num_qo_heads}, {head_dim}], got {tuple(q.shape)}")
    else:
        raise ValueError(f"expected q as [tokens, heads, dim] or [tokens, heads*dim], got {tuple(q.shape)}")
    _lib.require_cuda(q)
    q_clean = q if inplace else q.clone()
    q_view = q_clean.view(q.shape[0], num_qo_heads, head_dim) if q.ndim == 2 else q_clean
    if q_view.stride(2) != 1:
        raise ValueError("q must be contiguous in its last dimension")
    tokens = q.shape[0]
    if out is not None:
        if tuple(out.shape) != (tokens, num_kv_heads):
            raise ValueError(f"expected DMS output shape {(tokens, num_kv_heads)}, got {tuple(out.shape)}")
        if out.dtype != torch.bool:
            raise ValueError(f"expected DMS output dtype torch.bool, got {out.dtype}")
        if out.device != q_clean.device:
            raise ValueError(f"expected DMS output on {q_clean.device}, got {out.device}")
        if out.stride(1) != 1:
            raise ValueError("DMS output must be contiguous in its last dimension")
    evict = out if out is not None else torch.empty((tokens, num_kv_heads), device=q.device, dtype=torch.bool)
    if tokens:
        ev = evict.view(torch.uint8)
        with torch.cuda.device(q.device):
            rc = _lib.lib().fdms_extract_decisions(
                q_view.data_ptr(), _lib.dtype_code(q_view.dtype), q_view.stride(0), q_view.stride(1),
                ev.data_ptr(), ev.stride(0), tokens, num_qo_heads, num_kv_heads, head_dim,
                float(alpha_scale), float(alpha_offset), _lib.stream_ptr(q.device))
        _lib.check(rc)
    return q_clean, evict


def build_dms_live_mask(evict_mask: torch.Tensor, *, current_position: int, window_size: int,
                        positions: torch.Tensor | None = None) -> torch.Tensor:
    """live = ~evict | (current_position - position <= window); evict_mask is [kv_heads, tokens]
    or [layers, kv_heads, tokens] (reference: dms.py:235-262).  Host-side helper (plain torch)."""
    if evict_mask.ndim not in (2, 3):
        raise ValueError(f"expected evict_mask rank 2 or 3, got {evict_mask.ndim}")
    if window_size < 0:
        raise ValueError(f"window_size must be non-negative, got {window_size}")
    tokens = evict_mask.shape[-1]
    if positions is None:
        positions = torch.arange(tokens, device=evict_mask.device)
    else:
        positions = positions.to(device=evict_mask.device)
    if positions.shape != (tokens,):
        raise ValueError(f"expected positions shape {(tokens,)}, got {tuple(positions.shape)}")
    inside = (int(current_position) - positions.to(torch.long)) <= int(window_size)
    return (~evict_mask.bool()) | inside.view((1,) * (evict_mask.ndim - 1) + (tokens,))

"""Weight loading: safetensors shards with the packed-module mapping (reference:
fastdms/utils/loader.py), or an in-memory state dict (synthetic / random-init models)."""
from __future__ import annotations

import os
from glob import glob

import torch
from torch import nn


def _default_loader(param: nn.Parameter, loaded: torch.Tensor):
    param.data.copy_(loaded)


def load_state_dict(model: nn.Module, state_dict: dict[str, torch.Tensor]) -> None:
    """HF-style names (q_proj, k_proj, v_proj, gate_proj, up_proj, ...) into the packed parameters,
    each through its parameter's `weight_loader` (which takes the tensor-parallel shard)."""
    packed = getattr(model, "packed_modules_mapping", {})
    for name, tensor in state_dict.items():
        for key, (target, shard_id) in packed.items():
            if f".{key}." in name:
                param = model.get_parameter(name.replace(key, target))
                param.weight_loader(param, tensor, shard_id)
                break
        else:
            try:
                param = model.get_parameter(name)
            except AttributeError:
                continue                      # e.g. rotary inv_freq buffers in some checkpoints
            getattr(param, "weight_loader", _default_loader)(param, tensor)


def load_model(model: nn.Module, path: str) -> None:
    from safetensors import safe_open

    files = sorted(glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {path}")
    for file in files:
        with safe_open(file, "pt", "cpu") as f:
            load_state_dict(model, {name: f.get_tensor(name) for name in f.keys()})

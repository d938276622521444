"""Sequence sharding for replica-style multi-GPU serving (Llama-3.2-1B shape: every GPU holds the
whole model and serves its own sequences; there is no collective on the data path).

Request i goes to rank i % world_size.  Results are exchanged once, at the end, as Python objects
over the process group's store-backed object collective (NCCL or gloo)."""
from __future__ import annotations

import torch.distributed as dist


def shard_indices(num_requests: int, world_size: int, rank: int) -> list[int]:
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    return list(range(rank, num_requests, world_size))


def generate_sharded(llm, prompts, sampling_params):
    """Runs `llm.generate` on this rank's share of `prompts` and returns the results of ALL requests
    in request order on every rank.  `llm` is this rank's replica (tensor_parallel_size 1)."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    mine = shard_indices(len(prompts), world, rank)
    sps = sampling_params if isinstance(sampling_params, list) else [sampling_params] * len(prompts)
    local = llm.generate([prompts[i] for i in mine], [sps[i] for i in mine]) if mine else []
    return merge_sharded(dict(zip(mine, local)), len(prompts))


_EXCHANGES = 0


def merge_sharded(local: dict, num_requests: int, timeout_s: float = 600.0) -> list:
    """All-gathers {request index: result} dictionaries and returns the list in request order.

    Before the collective every rank posts a key in the process group's store and waits (bounded)
    for the keys of all peers, so a rank that died or raised earlier is reported as a RuntimeError
    naming it instead of leaving the others blocked in the collective."""
    global _EXCHANGES
    if dist.is_initialized() and dist.get_world_size() > 1:
        from datetime import timedelta
        world, rank = dist.get_world_size(), dist.get_rank()
        store = dist.distributed_c10d._get_default_store()
        _EXCHANGES += 1
        store.set(f"fastdms_b200/merge/{_EXCHANGES}/{rank}", "1")
        for r in range(world):
            try:
                store.wait([f"fastdms_b200/merge/{_EXCHANGES}/{r}"], timedelta(seconds=timeout_s))
            except Exception as e:  # noqa: BLE001  (the store raises its own timeout type)
                raise RuntimeError(f"rank {r} did not reach the result exchange within {timeout_s} s") from e
        parts = [None] * world
        dist.all_gather_object(parts, local)
    else:
        parts = [local]
    merged = {}
    for p in parts:
        merged.update(p)
    missing = [i for i in range(num_requests) if i not in merged]
    if missing:
        raise RuntimeError(f"requests {missing} were not produced by any rank")
    return [merged[i] for i in range(num_requests)]

"""Multi-rank host logic on CPU (gloo, world_size 2): sequence sharding covers every request exactly
once, results come back in request order on every rank, and a rank that fails before the exchange is
reported by its peer through the process-group timeout instead of a hang."""
from __future__ import annotations

import os
import sys
from datetime import timedelta
from pathlib import Path

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _init(rank, world, port, timeout_s=30):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=timeout_s))


class _FakeLLM:
    def generate(self, prompts, sampling_params):
        return [{"text": "", "token_ids": [sum(p), len(p)]} for p in prompts]


def _worker_ok(rank, world, port, q):
    _init(rank, world, port)
    from fastdms_b200.engine.sharding import generate_sharded, shard_indices
    prompts = [[i, i + 1, i + 2] for i in range(7)]
    assert shard_indices(7, world, rank) == list(range(rank, 7, world))
    out = generate_sharded(_FakeLLM(), prompts, None)
    q.put((rank, [o["token_ids"] for o in out]))
    dist.destroy_process_group()


def _worker_fail(rank, world, port, q):
    _init(rank, world, port, timeout_s=5)
    from fastdms_b200.engine.sharding import merge_sharded
    if rank == 1:
        q.put((rank, "raised before the exchange"))
        q.close()
        q.join_thread()                   # flush the message, then leave without joining the collective
        os._exit(0)
    try:
        merge_sharded({0: "a"}, 2, timeout_s=3.0)
        q.put((rank, "no error"))
    except RuntimeError as e:
        q.put((rank, f"error: {e}"))


def _run(target, port):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=target, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    return res


def test_sequence_sharding_world2():
    res = _run(_worker_ok, 29731)
    want = [[3 * i + 3, 3] for i in range(7)]
    assert res[0] == want and res[1] == want


def test_missing_rank_is_an_error_not_a_hang():
    res = _run(_worker_fail, 29733)
    assert res[1] == "raised before the exchange"
    assert res[0].startswith("error: rank 1 did not reach")


def test_shard_indices_errors():
    sys.path.insert(0, str(ROOT))
    from fastdms_b200.engine.sharding import merge_sharded, shard_indices
    assert shard_indices(5, 1, 0) == [0, 1, 2, 3, 4] and shard_indices(2, 4, 3) == []
    with pytest.raises(ValueError):
        shard_indices(5, 2, 2)
    with pytest.raises(RuntimeError):
        merge_sharded({0: "x"}, 2)

"""Row-parallel decode linear layer + all-reduce on N GPUs, per call inside a replayed CUDA graph (as in the
captured decode step): the fused launch (`fdms_linear_decode_allreduce`), the decode linear kernel followed by
NCCL's all-reduce (the reference's F.linear + dist.all_reduce, fastdms/layers/linear.py:1044-1048), the same
followed by the library's peer all-reduce, and the linear kernel alone.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m benchmarks.bench_tp_linear [--hidden 4096 --inter 12288]

Shapes are the o_proj and down_proj shards of a model with the given sizes at N ranks, 8 rows of bf16.  Each
graph holds `--calls` calls that cycle through enough weight copies to exceed L2; times are CUDA events around
the replays, maximum over the ranks.  Prints one JSON line per shape on rank 0."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads-dim", type=int, default=4096, help="q_heads * head_dim (in_features of o_proj before sharding)")
    ap.add_argument("--inter", type=int, default=12288)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--calls", type=int, default=64)
    ap.add_argument("--reps", type=int, default=20)
    args = ap.parse_args()
    os.environ.setdefault("FDMS_FUSED_ROW_PARALLEL", "1")
    os.environ.setdefault("FDMS_PEER_ALLREDUCE", "1")
    from fastdms_b200 import _lib
    from fastdms_b200.layers.linear import linear
    from fastdms_b200.layers.peer_allreduce import init_fused_row_parallel, init_peer_all_reduce
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    with torch.inference_mode():
        fused = init_fused_row_parallel(dev)
        peer = init_peer_all_reduce(dev)
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        for name, n, k in (("o_proj", args.hidden, args.heads_dim // world), ("down_proj", args.hidden, args.inter // world)):
            copies = max(2, int(300e6 // (n * k * 2)) + 1)
            ws = [(torch.randn((n, k), device=dev, generator=g) * (k * world) ** -0.5).to(torch.bfloat16) for _ in range(copies)]
            x = torch.randn((args.rows, k), device=dev, generator=g).to(torch.bfloat16)

            def two_step_nccl(w):
                y = linear(x, w)
                dist.all_reduce(y)

            def two_step_peer(w):
                y = linear(x, w)
                peer.all_reduce_(y)

            variants = {"linear_only": lambda w: linear(x, w), "linear_then_nccl": two_step_nccl}
            if peer is not None:
                variants["linear_then_peer_allreduce"] = two_step_peer
            if fused is not None and fused.fits(x, ws[0], None):
                variants["fused"] = lambda w: fused.linear_all_reduce(x, w, None)
            res = {}
            for vname, fn in variants.items():
                for w in ws[:2]:
                    fn(w)
                torch.cuda.synchronize(dev)
                dist.barrier()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for i in range(args.calls):
                        fn(ws[i % copies])
                for _ in range(3):
                    graph.replay()
                torch.cuda.synchronize(dev)
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.reps):
                    graph.replay()
                e1.record()
                torch.cuda.synchronize(dev)
                t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (args.reps * args.calls)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                res[vname] = round(float(t.item()), 2)
            status = _lib.read_device_status(dev)
            if rank == 0:
                print(json.dumps({"layer": name, "n_gpus": world, "rows": args.rows, "out_features": n, "in_features_per_rank": k,
                                  "weight_bytes_per_rank": n * k * 2, "us_per_call": res, "device_status": status}), flush=True)
        torch.cuda.synchronize(dev)
        dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()

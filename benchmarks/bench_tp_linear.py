"""Row-parallel decode linear layer + all-reduce on N GPUs, per call inside a replayed CUDA graph (as in the
captured decode step): the fused launch (`fdms_linear_decode_allreduce`), the decode linear kernel followed by
NCCL's all-reduce (the reference's F.linear + dist.all_reduce, fastdms/layers/linear.py:1044-1048), the same
followed by the library's peer all-reduce, and the linear kernel alone.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m benchmarks.bench_tp_linear [--hidden 4096 --inter 12288]

Shapes are the o_proj and down_proj shards of a model with the given sizes at N ranks, 8 rows of bf16.  Each
graph holds `--calls` calls that cycle through enough weight copies to exceed L2; times are CUDA events around
the replays, maximum over the ranks.  Prints one JSON line per shape on rank 0.

    python -m benchmarks.bench_tp_linear --staged-world 8

runs the fused launch as rank 0 of 8 on ONE GPU with the peers staged by the host (their partial tiles for the
calls' epochs already sit in rank 0's region, so no wait spins): the single-process form of the kernel for a
profiler, which must not wrap a multi-rank job.  It checks the result against a float32 computation."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def staged(args) -> None:
    """Rank 0 of `--staged-world` on one GPU; eager calls, each on its own weight copy, epochs 1, 2, ..."""
    from fastdms_b200 import _lib
    lib = _lib.lib()
    world = args.staged_world
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    MAXC, SLOT = 512, 1024
    g = torch.Generator(device=dev).manual_seed(3)
    with torch.inference_mode():
        for name, n, k in (("o_proj", args.hidden, args.heads_dim // world), ("down_proj", args.hidden, args.inter // world)):
            steps, ks = k // 256, 1
            while ks * 2 <= 8 and ks * 2 <= steps:
                ks *= 2
            tpc = 8 // ks
            ctas = -(-(n // 16) // tpc)
            nbytes = lib.fdms_linear_allreduce_region_bytes(world)
            regions = [torch.zeros((nbytes,), dtype=torch.uint8, device=dev) for _ in range(world)]
            ptrs = torch.tensor([r.data_ptr() for r in regions], dtype=torch.int64)
            slot_bytes = 2 * world * MAXC * (2 * SLOT) * 4
            mine = regions[0][:slot_bytes].view(torch.int32).view(2, world, MAXC, SLOT, 2)     # [half][source][cta][value][bits, epoch]
            calls = args.staged_calls
            ws = [(torch.randn((n, k), device=dev, generator=g) * (k * world) ** -0.5).to(torch.bfloat16) for _ in range(calls)]
            x = torch.randn((args.rows, k), device=dev, generator=g).to(torch.bfloat16)
            y = torch.empty((args.rows, n), device=dev, dtype=torch.bfloat16)
            npad = ctas * tpc * 16
            worst, times = 0.0, []
            for call in range(1, calls + 1):
                peers = torch.randn((world - 1, args.rows, n), device=dev, generator=g)
                full = torch.zeros((world - 1, 8, npad), device=dev)
                full[:, : args.rows, :n] = peers
                tiles = full.transpose(1, 2).reshape(world - 1, ctas, tpc * 128).contiguous()
                mine[call & 1, 1:, :ctas, : tpc * 128, 0] = tiles.view(torch.int32)
                mine[call & 1, 1:, :ctas, : tpc * 128, 1] = call
                torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                _lib.check(lib.fdms_linear_decode_allreduce(
                    x.data_ptr(), x.stride(0), ws[call - 1].data_ptr(), ws[call - 1].stride(0), None, y.data_ptr(), y.stride(0),
                    _lib.BF16, args.rows, n, k, ptrs.data_ptr(), 0, world, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev)))
                e1.record()
                torch.cuda.synchronize(dev)
                times.append(e0.elapsed_time(e1) * 1e3)
                ref = x.float() @ ws[call - 1].float().t() + peers.sum(0)
                worst = max(worst, float((y.float() - ref).abs().max()) / float(ref.abs().max()))
            print(json.dumps({"layer": name, "staged_world": world, "rows": args.rows, "out_features": n, "in_features_per_rank": k,
                              "ctas": ctas, "us_per_eager_call": [round(t, 2) for t in times], "max_rel_err": worst,
                              "device_status": _lib.read_device_status(dev)}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--staged-world", type=int, default=0, help="run as rank 0 of this many ranks on one GPU, peers staged by the host")
    ap.add_argument("--staged-calls", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads-dim", type=int, default=4096, help="q_heads * head_dim (in_features of o_proj before sharding)")
    ap.add_argument("--inter", type=int, default=12288)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--calls", type=int, default=64)
    ap.add_argument("--reps", type=int, default=20)
    args = ap.parse_args()
    if args.staged_world:
        staged(args)
        return
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

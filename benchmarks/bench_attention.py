"""Op-level sweep of the compact decode attention kernel over span lengths (the counterpart of the
reference's `benchmarks/bench_compact_decode.py`, default lengths `:101`): for every length, `layers`
distinct FP8 pools (so that one replay streams more than L2 holds) with randomly permuted 16-row
pages, one CUDA graph of `layers` launches replayed between two CUDA events.

    python -m benchmarks.bench_attention [--lengths 1280,2048,4096,8192,16384] [--head-dim 64] [--batch 8]

Prints one JSON line per length: µs per launch, achieved GB/s on the algorithmic bytes
(sum of live * 2 * head_dim FP8 bytes) and the fraction of `--peak-gbs`."""
from __future__ import annotations

import argparse
import json

import torch


def sweep(args) -> None:
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, Hk, G, D, L = args.batch, args.kv_heads, args.group, args.head_dim, args.layers
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn((B, Hk * G, D), device=dev, generator=g).to(torch.bfloat16)
    out = torch.empty_like(q)
    scale = torch.full((Hk,), 0.01, device=dev)
    for n in args.lengths:
        jitter = max(1, n // 10)
        pools = []
        for _ in range(L):
            live = (n + torch.randint(-jitter, jitter + 1, (B, Hk), device=dev, generator=g)).to(torch.int32)
            pages = (live + 15) // 16
            total = int(pages.sum().item()) + 8
            perm = torch.randperm(total, device=dev, generator=g).to(torch.int32)
            bt = torch.zeros((B, Hk, int(pages.max().item())), device=dev, dtype=torch.int32)
            flat = bt.view(B * Hk, -1)
            off = 0
            for i, c in enumerate(pages.flatten().tolist()):
                flat[i, :c] = perm[off:off + c]
                off += c
            k = torch.randint(0, 120, (total * 16, D), device=dev, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
            v = torch.randint(0, 120, (total * 16, D), device=dev, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
            pools.append((k, v, bt, live))
        base = torch.zeros((B, Hk), device=dev, dtype=torch.int32)
        res = {}
        for overlap in (False, True):
            def enqueue():
                for k, v, bt, live in pools:
                    compact_decode_attention(q, k, v, base, live, block_tables=bt, k_scale=scale, v_scale=scale, out=out,
                                             overlap_previous_kernel=overlap)
            enqueue()
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                enqueue()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize(dev)
            res[overlap] = e0.elapsed_time(e1) * 1e-3 / (args.reps * L)
        nbytes = sum(float(p[3].sum().item()) for p in pools) * 2 * D / L
        print(json.dumps({
            "length": n, "batch": B, "kv_heads": Hk, "group": G, "head_dim": D, "layers_cycled": L,
            "bytes_per_launch": nbytes, "us_per_launch": res[True] * 1e6, "us_per_launch_ordinary_launches": res[False] * 1e6,
            "achieved_gbs": nbytes / res[True] / 1e9, "frac_of_peak": nbytes / res[True] / 1e9 / args.peak_gbs,
            "peak_gbs": args.peak_gbs}), flush=True)
        del pools


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--lengths", type=lambda s: [int(x) for x in s.split(",")], default=[1280, 2048, 4096, 8192, 16384])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--group", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--peak-gbs", type=float, default=6535.1)
    sweep(ap.parse_args())


if __name__ == "__main__":
    main()

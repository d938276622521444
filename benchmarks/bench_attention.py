"""Op-level sweep of the compact decode attention kernel over span lengths (the counterpart of the
reference's `benchmarks/bench_compact_decode.py`, default lengths `:101`): for every length, `layers`
distinct FP8 pools (so that one replay streams more than L2 holds) with randomly permuted 16-row
pages, one CUDA graph of `layers` launches replayed between two CUDA events.

    python -m benchmarks.bench_attention [--lengths 1280,2048,4096,8192,16384] [--head-dim 64] [--batch 8]

Prints one JSON line per length: µs per launch, achieved GB/s on the algorithmic bytes
(sum of live * 2 * head_dim FP8 bytes) and the fraction of `--peak-gbs`.

`--with-reference` adds, per length, a row for the reference's own Triton kernel
(`fastdms/layers/compact_attention.py:1116-1336`) timed on the same GPU in the same process, the way
its `benchmarks/bench_compact_decode.py:81-92,141-154` does (eager calls between two CUDA events,
`max_live_count` passed so that the call does not synchronise) and also as a CUDA graph of the
same launches.  The reference has contiguous spans and no per-head scale, so its rows use that
layout with the same span lengths and distinct pools per layer.  It is imported from an unmodified
install of the reference under `baseline/_ref` (`python -m pip install --no-index --no-build-isolation --no-deps
--target baseline/_ref <a copy of the reference tree>`) and is a comparison row only: nothing else in this
repository imports it."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent


def _reference_kernel():
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "fastdms").is_dir():
        raise SystemExit(f"--with-reference needs an install of the reference under {ref}")
    sys.path.insert(0, str(ref))
    from fastdms.layers.compact_attention import compact_decode_attention as ref_attention
    return ref_attention


def time_reference(ref_attention, q, pools, reps: int, peak_gbs: float) -> dict:
    """`pools` = [(k, v, base, live)] in span layout; returns eager and graph µs per launch."""
    cap = int(max(int(p[3].max().item()) for p in pools))

    def enqueue():
        for k, v, base, live in pools:
            ref_attention(q, k, v, base, live, max_live_count=cap)
    for _ in range(3):
        enqueue()                      # Triton compiles on the first call
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        enqueue()
    e1.record()
    torch.cuda.synchronize()
    eager = e0.elapsed_time(e1) * 1e-3 / (reps * len(pools))
    graph_s = None
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            enqueue()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        graph_s = e0.elapsed_time(e1) * 1e-3 / (reps * len(pools))
    except Exception as e:                      # a kernel that cannot be captured still has its eager row
        print(json.dumps({"reference_graph_capture_failed": f"{type(e).__name__}: {e}"}), flush=True)
    nbytes = sum(float(p[3].sum().item()) for p in pools) * 2 * q.shape[-1] / len(pools)
    best = min(x for x in (eager, graph_s) if x is not None)
    return {"impl": "reference Triton kernel (span layout, no scale)", "bytes_per_launch": nbytes,
            "us_per_launch_eager": eager * 1e6, "us_per_launch_graph": None if graph_s is None else graph_s * 1e6,
            "achieved_gbs": nbytes / best / 1e9, "frac_of_peak": nbytes / best / 1e9 / peak_gbs}


def sweep(args) -> None:
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, Hk, G, D, L = args.batch, args.kv_heads, args.group, args.head_dim, args.layers
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn((B, Hk * G, D), device=dev, generator=g).to(torch.bfloat16)
    out = torch.empty_like(q)
    scale = torch.full((Hk,), 0.01, device=dev)
    ref_attention = _reference_kernel() if args.with_reference else None
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
        if ref_attention is not None:
            span_pools = []
            for k, v, bt, live in pools:
                rows = live.flatten().to(torch.int64)
                base_r = (torch.cumsum(rows, 0) - rows).to(torch.int32).view(B, Hk)
                total_r = int(rows.sum().item())
                span_pools.append((k[:total_r], v[:total_r], base_r, live))      # same bytes, read as contiguous spans
            row = time_reference(ref_attention, q, span_pools, args.reps, args.peak_gbs)
            row.update(length=n, batch=B, kv_heads=Hk, group=G, head_dim=D, layers_cycled=L, peak_gbs=args.peak_gbs)
            print(json.dumps(row), flush=True)
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
    ap.add_argument("--with-reference", action="store_true",
                    help="also time the reference's Triton kernel (needs the reference installed under baseline/_ref)")
    sweep(ap.parse_args())


if __name__ == "__main__":
    main()

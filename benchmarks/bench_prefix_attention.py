"""Op-level timing of the prefill-tail attention kernel (`fdms_prefix_attention`): one sequence's chunk
of `--queries` tokens against `--rows` FP8 rows per KV-head span (contiguous spans), merged with a
given dense result.  Prints one JSON line per (head_dim, queries, rows): µs per launch and TFLOP/s on
the algorithmic flops 4 * queries * q_heads * rows * head_dim.

    python -m benchmarks.bench_prefix_attention [--cases 64:2048:1280,64:2048:4096,128:2048:4096]"""
from __future__ import annotations

import argparse
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="64:2048:1280,64:2048:4096,128:2048:4096,64:8192:4096",
                    help="comma-separated head_dim:queries:rows")
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--reps", type=int, default=20)
    args = ap.parse_args()
    from fastdms_b200.layers.compact_attention import compact_prefix_attention
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    Hq, Hk = args.q_heads, args.kv_heads
    for case in args.cases.split(","):
        D, T, n = (int(x) for x in case.split(":"))
        q = torch.randn((T, Hq, D), device=dev, generator=g).to(torch.bfloat16)
        out = torch.randn((T, Hq, D), device=dev, generator=g).to(torch.bfloat16)
        lse = torch.randn((Hq, T), device=dev, generator=g)
        ck = torch.randint(0, 120, (Hk * n, D), device=dev, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
        cv = torch.randint(0, 120, (Hk * n, D), device=dev, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
        base = (torch.arange(Hk, device=dev, dtype=torch.int32) * n)[None]
        live = torch.full((1, Hk), n, device=dev, dtype=torch.int32)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        sc = torch.full((Hk,), 0.01, device=dev)

        def launch():
            compact_prefix_attention(q, ck, cv, base, live, cu, T, out, lse, k_scale=sc, v_scale=sc)
        for _ in range(3):
            launch()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            launch()
        e1.record()
        torch.cuda.synchronize(dev)
        sec = e0.elapsed_time(e1) * 1e-3 / args.reps
        flops = 4.0 * T * Hq * n * D
        print(json.dumps({"head_dim": D, "queries": T, "rows_per_span": n, "q_heads": Hq, "kv_heads": Hk,
                          "us_per_launch": sec * 1e6, "tflops": flops / sec / 1e12}), flush=True)


if __name__ == "__main__":
    main()

"""Op-level timing of the decode-sized linear kernels (`fdms_linear_decode`, and `fdms_linear_decode_fp8`
for e4m3 weights with one scale per output row) against `F.linear` (cuBLAS) on the projection shapes of a
decoder block, 8 rows of bf16 activations.  Each shape cycles through
enough distinct weight matrices to exceed L2, inside one CUDA graph replayed between two events.
Prints one JSON line per shape: µs per launch and GB/s on the algorithmic bytes (the weight matrix: 2 bytes
per element for bf16, 1 for FP8).

    python -m benchmarks.bench_linear [--shapes 3072x2048,2048x2048,16384x2048,2048x8192] [--rows 8]"""
from __future__ import annotations

import argparse
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="3072x2048,2048x2048,16384x2048,2048x8192", help="out x in, comma-separated")
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--peak-gbs", type=float, default=6535.1)
    args = ap.parse_args()
    import torch.nn.functional as F
    from fastdms_b200.layers.linear import linear, linear_fp8, quantize_weight_fp8
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    for shape in args.shapes.split(","):
        n, k = (int(v) for v in shape.split("x"))
        copies = max(2, int(400e6 // (n * k * 2)) + 1)                 # > 3 x L2 of weights per replay
        ws = [(torch.randn((n, k), device=dev, generator=g) * k ** -0.5).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn((args.rows, k), device=dev, generator=g).to(torch.bfloat16)
        w8s = [quantize_weight_fp8(w) for w in ws]
        res = {}
        with torch.inference_mode():
            for name, fn, mats in (("fdms_linear_decode", lambda x, w: linear(x, w), ws),
                                   ("fdms_linear_decode_fp8", lambda x, w: linear_fp8(x, w[0], w[1], None), w8s),
                                   ("F.linear", lambda x, w: F.linear(x, w), ws)):
                for w in mats[:2]:
                    fn(x, w)
                torch.cuda.synchronize(dev)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for w in mats:
                        fn(x, w)
                for _ in range(3):
                    graph.replay()
                torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.reps):
                    graph.replay()
                e1.record()
                torch.cuda.synchronize(dev)
                res[name] = e0.elapsed_time(e1) * 1e-3 / (args.reps * copies)
        nbytes = n * k * 2
        print(json.dumps({"out_features": n, "in_features": k, "rows": args.rows, "weight_copies_cycled": copies,
                          "bytes_per_launch": nbytes,
                          "fdms_us": res["fdms_linear_decode"] * 1e6, "fdms_gbs": nbytes / res["fdms_linear_decode"] / 1e9,
                          "fdms_frac_of_peak": nbytes / res["fdms_linear_decode"] / 1e9 / args.peak_gbs,
                          "fp8_us": res["fdms_linear_decode_fp8"] * 1e6, "fp8_gbs": nbytes / 2 / res["fdms_linear_decode_fp8"] / 1e9,
                          "fp8_frac_of_peak": nbytes / 2 / res["fdms_linear_decode_fp8"] / 1e9 / args.peak_gbs,
                          "cublas_us": res["F.linear"] * 1e6, "cublas_gbs": nbytes / res["F.linear"] / 1e9,
                          "peak_gbs": args.peak_gbs}), flush=True)


if __name__ == "__main__":
    main()

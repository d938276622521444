"""Phase timeline of the fused store + attention launch on the benchmark workload (c = 8, 32 q / 8 KV
heads of 64, about 1280 live rows per span, FP8 pools, permuted 16-row pages, 16 layer pools).

Needs the probe build of the library (the production build carries no probe code):

    python -m fastdms_b200.build --probe
    FDMS_B200_LIB=fastdms_b200/libfastdms_b200_probe.so python -m benchmarks.attn_timeline [--loader staged]

The 16 per-layer launches are replayed as one CUDA graph, chained with programmatic dependent launch as
in the decode step; thread 0 of every CTA records the global nanosecond timer at seven phases and the
table of the LAST launch of the graph is printed: per phase the earliest, median and latest CTA,
relative to the moment the launch's first CTA started.  "issued" is the end of the part that runs
before the dependency on the preceding kernel is resolved (metadata, block tables, page loads issued);
"dependency" is when that kernel has completed; the rest is the launch's own critical path.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
PHASES = ["start", "issued", "dependency", "q_ready", "pages_done", "cta_folded", "end"]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--loader", choices=["direct", "staged"], default=None)
    ap.add_argument("--no-overlap", action="store_true", help="ordinary launches instead of programmatic dependent launch")
    args = ap.parse_args()
    if args.loader:
        os.environ["FDMS_ATTN_LOADER"] = args.loader
    import torch

    import bench
    from fastdms_b200 import _lib
    lib = _lib.lib()
    if not hasattr(lib, "fdms_attn_probe_read"):
        raise SystemExit("this library has no probe: build it with `python -m fastdms_b200.build --probe` and set FDMS_B200_LIB")
    lib.fdms_attn_probe_read.restype = ctypes.c_int32
    lib.fdms_attn_probe_read.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    m, seqs, hp, g = bench.build_gpu_workload(dev, seed=1234)
    bench.fill_activations(hp, g, dev)
    hp.set_positions([bench.CTX] * bench.B)
    hp._enqueue()
    torch.cuda.synchronize(dev)
    per_launch, nbytes, _ = bench.time_attention_kernel(hp, dev, reps=20, overlap=not args.no_overlap)
    ctas = 4096
    table = np.zeros((len(PHASES), ctas), dtype=np.uint64)
    _lib.check(lib.fdms_attn_probe_read(table.ctypes.data, len(PHASES), ctas))
    used = table[0] > 0
    n = int(used.sum())
    t = table[:, used].astype(np.int64)
    t0 = int(t[0].min())
    rows = {}
    for i, name in enumerate(PHASES):
        rel = (t[i][t[i] >= t0] - t0) / 1e3          # CTAs that are not cluster leaders never reach the last phase
        if rel.size == 0:
            continue
        rows[name] = {"first_us": round(float(rel.min()), 2), "median_us": round(float(np.median(rel)), 2),
                      "last_us": round(float(rel.max()), 2)}
    print(json.dumps({"loader": os.environ.get("FDMS_ATTN_LOADER", "direct"), "ctas": n, "overlap": not args.no_overlap,
                      "us_per_launch_with_probe": round(per_launch * 1e6, 2), "phases": rows}, indent=1))


if __name__ == "__main__":
    main()

"""Continuous-batching stress of the compact-DMS engine on synthetic traffic: Poisson arrivals, prompt
lengths log-uniform, generation lengths uniform, a cap on concurrent sequences and (optionally) on the
compact KV pool.  Shapes and arrival process follow the reference's serving-style runs
(`benchmarks/soak_compact_dms.py`, `benchmarks/bench_llama_wikitext2.py`); token ids are random.

    python -m benchmarks.bench_serving --shape llama-1b --requests 256 --rate 20 \
        --min-prompt 512 --max-prompt 32768 --min-gen 64 --max-gen 512 --max-concurrent 64 \
        [--kv-gib 8] [--prefill-chunk 2048] [--paged] [--admission optimistic]
    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m benchmarks.bench_serving ...     # N replicas

Under torchrun every rank runs its own engine on its own GPU and serves request i of the one arrival
stream when i mod N is its rank (sequence sharding, no data-path collective); rank 0 prints the
aggregate (wall time = the slowest rank, throughputs summed, latencies over all requests).

Requests are admitted by the scheduler when the token budget and the compact pool allow: charged
their worst case (`--admission reserve`) or an estimate of what DMS keeps, with a retry when a
prefill does not fit (`--admission optimistic`).  With `--paged`, a decode step that could run out of
pages preempts the youngest request (it is prefilled again later); spans own their decode headroom.
Whole prompts are prefilled in one step, or in `--prefill-chunk`-token pieces.  Prints one JSON line: request and token throughput, time to
first token, decode step statistics, peak live rows of the pool, and a check that every page / span
went back to the pool at the end."""
from __future__ import annotations

import argparse
import json
import math
import os
import time

import numpy as np
import torch


def run(args) -> dict:
    from fastdms_b200 import _lib
    from fastdms_b200.utils.shapes import SHAPES
    from fastdms_b200.engine.llm_engine import LLMEngine
    from fastdms_b200.sampling_params import SamplingParams

    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    rng = np.random.default_rng(args.seed)
    n_all = args.requests
    arrivals = np.cumsum(rng.exponential(1.0 / args.rate, size=n_all))
    prompts = np.exp(rng.uniform(math.log(args.min_prompt), math.log(args.max_prompt), size=n_all)).astype(np.int64)
    gens = rng.integers(args.min_gen, args.max_gen + 1, size=n_all)
    mine = np.arange(rank, n_all, world)                 # request i goes to rank i mod N
    arrivals, prompts, gens = arrivals[mine], prompts[mine], gens[mine]
    n = len(mine)
    hf = dict(SHAPES[args.shape])
    max_len = int(args.max_prompt + args.max_gen + 8)
    hf.update(attention_bias=True, torch_dtype="bfloat16", max_position_embeddings=max_len)
    elem_rows = hf["num_hidden_layers"] * 2 * hf["head_dim"]                 # FP8 bytes per pool row over all layers
    budget = int(args.kv_gib * (1 << 30)) if args.kv_gib else None
    engine = LLMEngine(
        f"synthetic-{args.shape}", hf_config=hf, random_init_seed=args.seed, device=dev, max_model_len=max_len,
        max_num_seqs=args.max_concurrent,
        max_num_batched_tokens=max(4 * args.prefill_chunk, 8192) if args.prefill_chunk else max(2 * args.max_prompt, 16384),
        kv_cache_dtype="float8_e4m3fn", compact_kv_paged=args.paged, compact_kv_budget_bytes=budget,
        dms_window_size=args.window, compact_kv_admission=args.admission,
        compact_kv_admission_keep_estimate=args.keep_estimate, prefill_chunk_size=args.prefill_chunk or None,
        decode_run_ahead=args.run_ahead)
    mgr = engine.model_runner.compact_kv_manager
    vocab = hf["vocab_size"]
    g = torch.Generator().manual_seed(args.seed + rank)
    token_lists = [torch.randint(0, vocab, (int(p),), generator=g).tolist() for p in prompts]

    # warm-up: one short request through prefill and a few decode steps
    engine.add_request(token_lists[0][:512], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    while not engine.is_finished():
        engine.step()
    torch.cuda.synchronize(dev)

    seqs, first_token_at, done_at = {}, {}, {}
    nxt = 0
    decode_ms, decode_batch, prefill_tokens, peak_live = [], [], 0, 0
    if world > 1:
        dist.barrier()                                   # the ranks share one arrival clock
    t0 = time.perf_counter()
    while len(done_at) < n:
        now = time.perf_counter() - t0
        while nxt < n and arrivals[nxt] <= now:
            sp = SamplingParams(temperature=0.0, max_tokens=int(gens[nxt]), ignore_eos=True)
            seqs[nxt] = engine.add_request(token_lists[nxt], sp)
            nxt += 1
        if engine.is_finished():
            time.sleep(max(0.0, min(0.01, arrivals[nxt] - now)))
            continue
        ts = time.perf_counter()
        _, num_tokens = engine.step()
        te = time.perf_counter()
        if num_tokens > 0:
            prefill_tokens += num_tokens
        else:
            decode_ms.append((te - ts) * 1e3)
            decode_batch.append(-num_tokens)
        for i, s in seqs.items():
            if i not in first_token_at and s.num_completion_tokens > 0:
                first_token_at[i] = te - t0
            if i not in done_at and s.is_finished:
                done_at[i] = te - t0
        if len(decode_ms) % 64 == 1:
            peak_live = max(peak_live, int(mgr.layer_major_live_counts[0].sum().item()))
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    out_tokens = int(sum(s.num_completion_tokens for s in seqs.values()))
    ttft = np.array([first_token_at[i] - arrivals[i] for i in range(n)])
    lat = np.array([done_at[i] - arrivals[i] for i in range(n)])
    if mgr.paged:
        pool_clean = mgr.free_page_counts.tolist() == [mgr.pages_per_layer] * mgr.num_layers
    else:
        pool_clean = mgr.free_ranges_per_layer == [[(0, mgr.capacity_tokens)]] * mgr.num_layers
    dm = np.array(decode_ms) if decode_ms else np.zeros(1)
    status = int(_lib.read_device_status(dev))
    if world > 1:
        # one exchange after the timed region; every figure below is over all ranks
        part = dict(wall=wall, out=out_tokens, prefill=int(prefill_tokens), ttft=ttft, lat=lat, dm=dm, batch=decode_batch,
                    peak=peak_live, denied=int(mgr.admission_denied_count), retries=int(engine.scheduler.prefill_retries),
                    preempt=int(engine.scheduler.preemptions), clean=bool(pool_clean), status=status, prompts=prompts, gens=gens)
        parts = [None] * world
        dist.all_gather_object(parts, part)
        wall = max(q["wall"] for q in parts)
        out_tokens = sum(q["out"] for q in parts)
        prefill_tokens = sum(q["prefill"] for q in parts)
        ttft = np.concatenate([q["ttft"] for q in parts]); lat = np.concatenate([q["lat"] for q in parts])
        dm = np.concatenate([q["dm"] for q in parts])
        decode_batch = [b for q in parts for b in q["batch"]]
        peak_live = max(q["peak"] for q in parts)
        pool_clean = all(q["clean"] for q in parts)
        status = 0
        for q in parts:
            status |= q["status"]
        prompts = np.concatenate([q["prompts"] for q in parts]); gens = np.concatenate([q["gens"] for q in parts])
        denied, retries, preempt = (sum(q[k] for q in parts) for k in ("denied", "retries", "preempt"))
        n = n_all
    else:
        denied, retries, preempt = int(mgr.admission_denied_count), int(engine.scheduler.prefill_retries), int(engine.scheduler.preemptions)
    return {
        "n_gpus": world, "parallelism": f"replicas x{world}, request i -> rank i mod {world}" if world > 1 else "one GPU",
        "shape": args.shape, "requests": n, "arrival_rate_per_s": args.rate, "max_concurrent": args.max_concurrent,
        "prompt_len": [int(prompts.min()), int(np.median(prompts)), int(prompts.max())],
        "gen_len": [int(gens.min()), int(np.median(gens)), int(gens.max())],
        "wall_s": wall, "requests_per_s": n / wall, "output_tok_s": out_tokens / wall,
        "total_tok_s": (out_tokens + prefill_tokens) / wall, "prefill_tokens": int(prefill_tokens), "output_tokens": out_tokens,
        "ttft_s": {"p50": float(np.median(ttft)), "p90": float(np.quantile(ttft, 0.9)), "max": float(ttft.max())},
        "latency_s": {"p50": float(np.median(lat)), "p90": float(np.quantile(lat, 0.9)), "max": float(lat.max())},
        "decode_steps": len(decode_ms), "decode_ms_per_step": {"p50": float(np.median(dm)), "p90": float(np.quantile(dm, 0.9))},
        "mean_decode_batch": float(np.mean(decode_batch)) if decode_batch else 0.0,
        "pool_rows_per_layer": mgr.capacity_tokens, "pool_gib": mgr.capacity_tokens * elem_rows / (1 << 30),
        "peak_live_rows_layer0_sampled": peak_live, "admission": args.admission, "prefill_chunk": args.prefill_chunk, "run_ahead": bool(args.run_ahead),
        "admission_denied": denied, "prefill_retries": retries, "preemptions": preempt,
        "pool_returned_clean": bool(pool_clean), "layout": "paged" if mgr.paged else "spans",
        "device_status": status,
        "data": "synthetic: random-init bf16 weights, uniform random token ids",
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="llama-1b")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--rate", type=float, default=20.0)
    ap.add_argument("--min-prompt", type=int, default=512)
    ap.add_argument("--max-prompt", type=int, default=32768)
    ap.add_argument("--min-gen", type=int, default=64)
    ap.add_argument("--max-gen", type=int, default=512)
    ap.add_argument("--max-concurrent", type=int, default=64)
    ap.add_argument("--kv-gib", type=float, default=0.0)
    ap.add_argument("--window", type=int, default=256)
    ap.add_argument("--paged", action="store_true")
    ap.add_argument("--admission", choices=["reserve", "optimistic"], default="reserve")
    ap.add_argument("--keep-estimate", type=float, default=0.2)
    ap.add_argument("--prefill-chunk", type=int, default=2048, help="prefill prompts in chunks of this many tokens (0: one pass)")
    ap.add_argument("--run-ahead", action="store_true",
                    help="launch the next decode step from device-resident tokens before this step's are read")
    ap.add_argument("--seed", type=int, default=0)
    out = run(ap.parse_args())
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(out), flush=True)
    import torch.distributed as dist
    if dist.is_initialized():
        torch.cuda.synchronize()
        dist.barrier()
        os._exit(0)           # captured graphs and the process group are not torn down in order by the interpreter


if __name__ == "__main__":
    main()

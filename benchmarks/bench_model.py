"""Whole-model decode throughput on synthetic weights of the shapes the reference is benchmarked on
(its WikiText-2 8192 + 128 runs, `benchmarks/bench_llama_wikitext2.py`; dataset and checkpoints are
replaced by random token ids and random-init weights).

    python -m benchmarks.bench_model --shape llama-1b                       # one GPU, c = 8
    torchrun --nproc-per-node N -m benchmarks.bench_model --shape llama-1b  # N replicas, c = 8 each
    torchrun --nproc-per-node N -m benchmarks.bench_model --shape qwen3-8b --tp N

Replica mode (`--tp 1` under torchrun) shards sequences over the ranks with no data-path collective;
`--tp N` splits KV heads over the ranks with NCCL all-reduces after o_proj and down_proj.
Prints one JSON line on rank 0: prefill and decode tokens/s through `LLMEngine.step()` (host
scheduling, graph replay, token read-back included), the measured KV compression and the per-step
time.  The DMS decision channel of the random-init model is biased so that about 7/8 of the tokens
are marked for eviction (needs a q bias, so the synthetic configs set `attention_bias`)."""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from fastdms_b200.utils.shapes import SHAPES  # noqa: E402


def run(args) -> dict:
    from fastdms_b200 import _lib
    from fastdms_b200.engine.llm_engine import LLMEngine
    from fastdms_b200.sampling_params import SamplingParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    if args.tp not in (1, world):
        raise SystemExit(f"--tp must be 1 (replicas) or the number of ranks ({world})")

    hf = dict(SHAPES[args.shape])
    shard = getattr(args, "shard", 1)
    if shard > 1:
        # one rank's slice of an N-way tensor-parallel model on one GPU, collectives left out: the kernels one
        # rank launches per step, for a launch list of the tensor-parallel step
        for key in ("num_attention_heads", "num_key_value_heads", "intermediate_size", "vocab_size"):
            hf[key] = hf[key] // shard
    hf.update(attention_bias=True, torch_dtype="bfloat16",
              max_position_embeddings=args.prompt_len + args.decode_steps + 8)
    c = args.concurrency
    engine = LLMEngine(
        f"synthetic-{args.shape}", hf_config=hf, random_init_seed=args.seed, device=dev,
        max_model_len=args.prompt_len + args.decode_steps + 8, max_num_seqs=c,
        max_num_batched_tokens=max(c * args.prompt_len, 16384), kv_cache_dtype="float8_e4m3fn",
        tensor_parallel_size=args.tp, compact_kv_paged=args.paged, enforce_eager=args.eager,
        dms_window_size=args.window, dms_expiry_interval=args.expiry_interval,
        prefill_chunk_size=args.prefill_chunk or None, decode_run_ahead=getattr(args, "run_ahead", False),
        fp8_weights=getattr(args, "fp8_weights", False))
    # replicas draw different prompts; tensor-parallel ranks must see the same ones
    g = torch.Generator().manual_seed(args.seed + (rank if args.tp == 1 else 0))
    vocab = hf["vocab_size"]
    if not args.no_warmup:
        # one untimed round (library handles, autotuning, lazy allocations), like the reference's
        # post-warm-up numbers
        wsp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
        for _ in range(c):
            engine.add_request(torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist(), wsp)
        while not engine.is_finished():
            engine.step()
    sp = SamplingParams(temperature=0.0, max_tokens=args.decode_steps + 2, ignore_eos=True)
    seqs = [engine.add_request(torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist(), sp) for _ in range(c)]

    def sync():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()

    sync()
    t0 = time.perf_counter()
    prefill_steps = 0
    while engine.scheduler.waiting or any(s.num_completion_tokens == 0 for s in seqs):
        engine.step()
        prefill_steps += 1
    sync()
    t_prefill = time.perf_counter() - t0
    m = engine.model_runner.compact_kv_manager
    live0 = torch.stack([m.seq_states[s.seq_id].live_counts for s in seqs]).float()
    # two untimed decode steps: the eager warm-up and the graph capture
    warm = 0 if args.eager else 2
    for _ in range(warm):
        engine.step()
    sync()
    steps = args.decode_steps - warm
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    sync()
    t_decode = time.perf_counter() - t0
    live1 = torch.stack([m.seq_states[s.seq_id].live_counts for s in seqs]).float()
    tokens = [s.completion_token_ids[-4:] for s in seqs[:2]]
    while not engine.is_finished():
        engine.step()
    replicas = world if args.tp == 1 else 1
    t = torch.tensor([t_prefill, t_decode], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    t_prefill, t_decode = (float(x) for x in t.tolist())
    ctx_end = args.prompt_len + args.decode_steps
    return {
        "shape": args.shape + (f" (slice 1/{shard})" if shard > 1 else ""), "n_gpus": world, "parallelism": f"tp{args.tp}" if args.tp > 1 else f"replicas x{world}",
        "concurrency_per_replica": c, "prompt_len": args.prompt_len, "decode_steps_timed": steps,
        "decode_tok_s": replicas * c * steps / t_decode, "decode_ms_per_step": t_decode / steps * 1e3,
        "prefill_tok_s": replicas * c * args.prompt_len / t_prefill, "prefill_s": t_prefill, "prefill_steps": prefill_steps,
        "prefill_chunk": args.prefill_chunk, "run_ahead": bool(getattr(args, "run_ahead", False)), "fp8_weights": bool(getattr(args, "fp8_weights", False)), "kv_dtype": "float8_e4m3fn", "layout": "paged" if args.paged else "spans", "window": engine.model_runner.dms_metadata.window_size,
        "mean_live_after_prefill": float(live0.mean()), "mean_live_at_end": float(live1.mean()),
        "compression_at_end": ctx_end / float(live1.mean()), "sample_tokens": tokens,
        "device_status": int(_lib.read_device_status(dev)),
        "data": "synthetic: random-init bf16 weights, uniform random token ids",
    }


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", choices=sorted(SHAPES), default="llama-1b")
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=8192)
    ap.add_argument("--decode-steps", type=int, default=128)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--shard", type=int, default=1, help="run one rank's slice of an N-way tensor-parallel model (no collectives)")
    ap.add_argument("--window", type=int, default=256)
    ap.add_argument("--expiry-interval", type=int, default=1)
    ap.add_argument("--paged", action="store_true")
    ap.add_argument("--prefill-chunk", type=int, default=0, help="prefill in chunks of this many tokens per prompt (0: one pass)")
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--fp8-weights", action="store_true", help="decode streams FP8 e4m3 copies of the linear weights")
    ap.add_argument("--run-ahead", action="store_true",
                    help="launch the next decode step from device-resident tokens before this step's are read")
    ap.add_argument("--no-warmup", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    return ap


def main() -> None:
    args = build_parser().parse_args()
    out = run(args)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(out))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

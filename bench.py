"""Benchmark of the compact-DMS decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the op-level compact decode on Llama-3.2-1B shapes, laid out
as the 16 layers of that model so that a "step" is one decode step of the hot path): 32 q heads,
8 KV heads, head_dim 64, c = 8 sequences at 8192 context; per (layer, sequence, KV head) the
compact span holds 1024 + U(-128, 128) retained prompt tokens plus the 256-token window; K/V ~
N(0,1) stored as FP8 e4m3 with per-(layer, head) absmax scales; 16-row pages, block tables
randomly permuted; q/k/v activations bf16 ~ N(0,1) with the decision channel set for a 7/8
eviction rate.  All data is synthetic (seeded); no dataset or checkpoint is used.

One step = expiry (all layers) -> decode metadata (all layers) -> per layer [fused decision + RoPE
+ FP8 store, compact attention] -> decision recording.  It produces c = 8 tokens' worth of
attention outputs, so value = 8 * n_gpus / step time.  The model's GEMMs are not part of this
path.  With N > 1 GPUs every rank runs its own 8 sequences (sequence sharding, no collective).

The JSON line carries: `value` (inputs resident in HBM, CUDA-graph replay), `e2e` (same step driven
through the public API with host buffers: pinned H2D of q/k/v/positions and D2H of the outputs of
every step inside the timed region, steps pipelined two deep), `roofline` (attention kernel: algorithmic bytes / CUDA-event time per launch
against the measured HBM peak), `cpu_baseline` (the numpy oracle port of the reference's CPU path,
timed on this box's host cores on a bounded sample).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# ---- the workload: op-level compact decode on the 16 layers of the Llama-3.2-1B shape -------------
L, B, HQ, HK, D = 16, 8, 32, 8, 64
CTX, WINDOW = 8192, 256
RETAIN_MEAN, RETAIN_JITTER = 1024, 128
ALPHA_SCALE, ALPHA_OFFSET = 100.0, 5.0
ROPE_THETA = 500000.0
MAX_MODEL_LEN = CTX + 512
EVICT_RATE = 7.0 / 8.0
WORKLOAD = ("configs[1] op-level compact decode, Llama-3.2-1B shape as 16 layer pools: c=8, ctx 8192, "
            "32q/8kv heads, head_dim 64, live=1024+U(-128,128)+256 per (layer,seq,head), FP8 e4m3 + per-head "
            "absmax scale, 16-row pages, permuted block tables")


def workload_config(n_gpus: int) -> dict:
    """The `config` object of the result line: the workload, identical for both arms."""
    return {"workload": WORKLOAD, "layers": L, "sequences_per_gpu": B,
            "parallelism": f"sequence-sharded x{n_gpus}, no collective",
            "l2": "inputs larger than L2: 16 layer pools, 168 MB of K/V cycled per step (L2 is 126 MB)",
            "expiry": "exact, every step"}


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# clocks / throttle sampling (read-only NVML queries)
# ------------------------------------------------------------------------------------------------
# dram__bytes_read.sum + dram__bytes_write.sum of one fused attention launch of this (seeded, hence
# reproducible) workload, from the ncu capture summarised under profiles/
NCU_DRAM_BYTES_PER_LAUNCH = 10_688_512 + 0
NCU_DRAM_SOURCE = ("ncu --set full capture of attn_decode_direct_kernel<64, 3, true> on this workload "
                   "(profiles/attn_decode_direct_fused_config2.md): 10.69 MB read, 0 written")


class ClockSampler:
    def __init__(self, index: int):
        self.index = index
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self) -> dict:
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the numpy oracle port of the reference's CPU path, contiguous-span layout
# ------------------------------------------------------------------------------------------------
def rope_cache(max_pos: int) -> np.ndarray:
    half = D // 2
    inv = 1.0 / (ROPE_THETA ** (np.arange(half, dtype=np.float32) / half))
    ang = np.arange(max_pos, dtype=np.float32)[:, None] * inv[None, :]
    return np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)


def decision_lane(rng, shape):
    """+1 (evict) with probability 7/8, else -1 (keep); the threshold is 0.05."""
    return np.where(rng.random(shape) < EVICT_RATE, 1.0, -1.0).astype(np.float32)


class CpuUnit:
    """Host twin of one (layer, sequence) of the workload in the reference's contiguous-span layout:
    8 KV-head spans, their metadata rows, and the step's q/k/v activations.  Units are independent
    (the path shards by sequence and by layer pool), so they spread over host cores freely."""

    def __init__(self, seed: int):
        from oracle.dtypes import round_to
        rng = np.random.default_rng(seed)
        self.live = (RETAIN_MEAN + rng.integers(-RETAIN_JITTER, RETAIN_JITTER + 1, size=(1, HK)) + WINDOW + 1).astype(np.int32)
        span = int(self.live.max()) + 600
        self.base = (np.arange(HK, dtype=np.int32) * span).reshape(1, HK)
        rows = HK * span
        self.k = rng.integers(0, 0x78, size=(rows, D), dtype=np.uint8)
        self.v = rng.integers(0, 0x78, size=(rows, D), dtype=np.uint8)
        self.pos = np.full((1, HK, MAX_MODEL_LEN), -1, np.int32)
        self.ev = np.zeros((1, HK, MAX_MODEL_LEN), bool)
        for h in range(HK):
            n = int(self.live[0, h])
            kept = np.sort(rng.choice(CTX - 1 - WINDOW, n - WINDOW - 1, replace=False))
            self.pos[0, h, :n] = np.concatenate([kept, np.arange(CTX - 1 - WINDOW, CTX)])
            self.ev[0, h, n - WINDOW - 1:n] = rng.random(WINDOW + 1) < EVICT_RATE
        self.ks = np.full(HK, 5.5 / 448.0, np.float32)
        self.vs = np.full(HK, 5.5 / 448.0, np.float32)
        self.q = round_to(rng.standard_normal((1, HQ, D)).astype(np.float32), "bf16")
        self.q[:, 0::HQ // HK, D - 1] = decision_lane(rng, (1, HK))
        self.kx = round_to(rng.standard_normal((1, HK, D)).astype(np.float32), "bf16")
        self.vx = round_to(rng.standard_normal((1, HK, D)).astype(np.float32), "bf16")

    def step(self, cache: np.ndarray, cur: int):
        from oracle import compact_dms as O
        O.expire_layer(self.pos, self.ev, self.live, self.base, self.k, self.v, [cur], WINDOW)
        _, _, slot = O.prepare_decode_metadata(self.base, self.live)
        q_rot, _, ev = O.rope_store_decode(
            self.q, self.kx, self.vx, cache, self.k, self.v, slot, [cur], num_kv_heads=HK,
            alpha_scale=ALPHA_SCALE, alpha_offset=ALPHA_OFFSET, act_dtype="bf16", pool_dtype="e4m3",
            k_scale=self.ks, v_scale=self.vs)
        out = O.decode_attention(q_rot, self.k, self.v, self.base, self.live, pool_dtype="e4m3", out_dtype="bf16",
                                 k_scale=self.ks, v_scale=self.vs)
        O.record_decisions(self.pos[None], self.ev[None], self.live[None], ev[None], [cur])
        return out


def _cpu_worker(conn, unit_ids):
    """Worker process: owns a set of (layer, sequence) units; 'run n' advances all of them n steps."""
    sys.path.insert(0, str(ROOT))
    cache = rope_cache(MAX_MODEL_LEN)
    units = [CpuUnit(1000 + u) for u in unit_ids]
    cur = CTX
    conn.send("ready")
    while True:
        msg = conn.recv()
        if msg[0] == "stop":
            break
        for _ in range(msg[1]):
            for u in units:
                u.step(cache, cur)
            cur += 1
        conn.send("done")
    conn.close()


def cpu_time_steps(num_units: int, steps: int, warmup: int, procs: int) -> tuple[float, int]:
    """Wall seconds per step in which every one of `num_units` (layer, sequence) units advances by
    one decode step of the oracle port; the units are spread over `procs` single-threaded worker
    processes (spawned, so they are independent of any CUDA state in this process)."""
    import multiprocessing as mp
    procs = max(1, min(procs, num_units))
    os.environ["OMP_NUM_THREADS"] = "1"
    os.environ["OPENBLAS_NUM_THREADS"] = "1"
    os.environ["MKL_NUM_THREADS"] = "1"
    ctx = mp.get_context("spawn")
    workers = []
    for w in range(procs):
        parent, child = ctx.Pipe()
        pr = ctx.Process(target=_cpu_worker, args=(child, list(range(w, num_units, procs))), daemon=True)
        pr.start()
        workers.append((pr, parent))
    for _, c in workers:
        assert c.recv() == "ready"

    def run(n):
        for _, c in workers:
            c.send(("run", n))
        for _, c in workers:
            assert c.recv() == "done"

    if warmup:
        run(warmup)
    t0 = time.perf_counter()
    run(steps)
    dt = time.perf_counter() - t0
    for pr, c in workers:
        c.send(("stop", 0))
        pr.join(timeout=5)
    return dt / steps, procs


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    units = L * B
    per_step, procs = cpu_time_steps(units, args.steps, args.warmup, cores)
    value = B / per_step
    line = {
        "impl": "reference", "metric": "decode tok/s at c=8, 8K ctx (compact-DMS hot path)", "value": value,
        "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "e4m3 KV / bf16 activations, f32 math", "data": "synthetic",
        "config": workload_config(args.gpus),
        "timing": "wall clock around the worker pool's steps on the host cores (rank 0 only)",
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": procs, "kind": "port",
                         "sample": f"{args.steps} full decode steps (16 layers x 8 sequences x 8 KV heads) of the numpy "
                                   f"oracle port of the reference's CPU path (contiguous spans instead of pages), {procs} single-threaded worker processes "
                                   f"on {cores} host cores"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def build_gpu_workload(dev, seed: int):
    """Prefills 8 sequences of 8192 synthetic tokens per layer through the pack kernels so that the
    manager reaches the config's compact shape, then returns (manager, seqs, hot path)."""
    import torch
    from fastdms_b200.engine.compact_kv import CompactKVManager
    from fastdms_b200.engine.hot_path import DecodeHotPath
    from fastdms_b200.engine.sequence import Sequence
    from fastdms_b200.sampling_params import SamplingParams

    g = torch.Generator(device=dev).manual_seed(seed)
    pool_rows = 131072                                     # per layer; ~82k rows live
    k_scale = torch.empty((L, HK), device=dev)
    v_scale = torch.empty((L, HK), device=dev)
    acts = []
    for l in range(L):
        k = torch.randn((B * CTX, HK, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
        v = torch.randn((B * CTX, HK, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
        k_scale[l] = k.float().abs().amax(dim=(0, 2)) / 448.0
        v_scale[l] = v.float().abs().amax(dim=(0, 2)) / 448.0
        acts.append((k, v))
        if l == 0:
            m = None
    m = CompactKVManager(num_layers=L, num_kv_heads=HK, capacity_tokens=pool_rows, max_model_len=MAX_MODEL_LEN,
                         device=dev, head_dim=D, compact_dtype=torch.float8_e4m3fn, max_active_seqs=B, paged=True,
                         k_scale=k_scale, v_scale=v_scale, row_indirection=True)
    # randomly permuted block tables: shuffle every layer's free-page stack before anything is allocated
    for l in range(L):
        perm = torch.randperm(m.pages_per_layer, device=dev, generator=g)
        m.free_pages[l].copy_(m.free_pages[l][perm])
    seqs = [Sequence(list(range(CTX)), SamplingParams(max_tokens=MAX_MODEL_LEN - CTX)) for _ in range(B)]
    for s in seqs:
        m.allocate(s)
    cu = torch.arange(0, (B + 1) * CTX, CTX, dtype=torch.int32)
    old = CTX - 1 - WINDOW
    for l in range(L):
        retain = RETAIN_MEAN + torch.randint(-RETAIN_JITTER, RETAIN_JITTER + 1, (B, HK), device=dev, generator=g)
        order = torch.rand((B, HK, old), device=dev, generator=g).argsort(dim=-1).argsort(dim=-1)
        evict_old = order >= retain.unsqueeze(-1)                                   # keep exactly `retain` old tokens
        evict_new = torch.rand((B, HK, CTX - old), device=dev, generator=g) < EVICT_RATE
        evict = torch.cat([evict_old, evict_new], dim=-1).permute(0, 2, 1).reshape(B * CTX, HK).contiguous()
        k, v = acts[l]
        m.streaming_pack_layer(layer_id=l, k=k, v=v, evict_mask=evict, cu_seqlens_q=cu,
                               seq_ids=[s.seq_id for s in seqs], window_size=WINDOW)
        acts[l] = None
    del acts
    torch.cuda.synchronize(dev)
    cache = torch.from_numpy(rope_cache(MAX_MODEL_LEN)).to(dev).unsqueeze(1)
    hp = DecodeHotPath(m, seqs, num_q_heads=HQ, window_size=WINDOW, alpha_scale=ALPHA_SCALE,
                       alpha_offset=ALPHA_OFFSET, cos_sin_cache=cache)
    return m, seqs, hp, g


def fill_activations(hp, g, dev):
    import torch
    hp.q.copy_(torch.randn(hp.q.shape, device=dev, generator=g).to(hp.q.dtype))
    hp.k.copy_(torch.randn(hp.k.shape, device=dev, generator=g).to(hp.k.dtype))
    hp.v.copy_(torch.randn(hp.v.shape, device=dev, generator=g).to(hp.v.dtype))
    lane = torch.where(torch.rand((L, B, HK), device=dev, generator=g) < EVICT_RATE, 1.0, -1.0)
    hp.q[:, :, 0::HQ // HK, D - 1] = lane.to(hp.q.dtype)


def time_attention_kernel(hp, dev, reps: int, overlap: bool):
    """Average duration of one attention launch: a CUDA graph of the 16 per-layer launches (16
    distinct pools, 168 MB of K/V in total, more than L2) replayed `reps` times between two events."""
    import torch
    from fastdms_b200.layers.compact_attention import compact_decode_attention, fused_store_decode_attention
    m = hp.m

    def enqueue():
        for l in range(L):
            ks, vs = m.layer_scales(l)
            if hp.fuse_store:      # the launch the decode step makes: decision + RoPE + FP8 store + attention
                fused_store_decode_attention(
                    hp.q[l], hp.k[l], hp.v[l], hp.cos_sin_cache, m.compact_k_per_layer[l], m.compact_v_per_layer[l],
                    hp.base[l], hp.live[l], hp.evict_all[l], hp.positions, num_kv_heads=HK, alpha_scale=ALPHA_SCALE,
                    alpha_offset=ALPHA_OFFSET, block_tables=hp.block_tables[l], k_scale=ks, v_scale=vs, out=hp.out[l],
                    overlap_previous_kernel=overlap and l > 0)
                continue
            compact_decode_attention(hp.q[l], m.compact_k_per_layer[l], m.compact_v_per_layer[l], hp.base[l],
                                     hp.live[l], block_tables=hp.block_tables[l], k_scale=ks, v_scale=vs, out=hp.out[l],
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
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    per_launch_s = e0.elapsed_time(e1) * 1e-3 / (reps * L)
    live = hp.live.to(torch.int64)
    bytes_per_launch = float(live.sum().item()) * 2 * D / L        # mean over the 16 layers, FP8 K + V
    return per_launch_s, bytes_per_launch, reps * L


def run_model_block(dev, world: int, steps: int) -> dict:
    """Whole-model context for the hot-path number: the full Llama-3.2-1B shape (16 layers, hidden
    2048, 32 q / 8 KV heads of 64, MLP 8192, vocab 128256; random-init bf16 weights, FP8 compact KV,
    window 256, eviction rate 7/8), c = 8 prompts of 8192 random token ids per GPU, greedy decode
    through `LLMEngine.step()` (scheduler, graph replay and token read-back included)."""
    import torch
    from benchmarks.bench_model import build_parser, run as run_model
    ns = build_parser().parse_args(["--shape", "llama-1b", "--concurrency", str(B), "--prompt-len", str(CTX),
                                    "--decode-steps", str(steps), "--window", str(WINDOW), "--run-ahead"])
    r = run_model(ns)
    params = 16 * (2048 * (32 + 16) * 64 + 2048 * 2048 + 3 * 2048 * 8192) + 128256 * 2048        # streamed once per step
    kv_bytes = r["mean_live_at_end"] * 16 * B * HK * 2 * D
    step_bytes = params * 2 + kv_bytes
    peak, _ = measured_peaks()
    return {"workload": "full Llama-3.2-1B shape, random-init bf16 weights, FP8 compact KV, c=8 per GPU, 8192-token prompts, "
                        f"{r['decode_steps_timed']} greedy decode steps through LLMEngine.step() (next step launched from device-resident "
                        "tokens while this step's are read back)",
            "decode_tok_s": r["decode_tok_s"], "ms_per_step": r["decode_ms_per_step"], "prefill_tok_s": r["prefill_tok_s"],
            "hbm_bytes_per_step": step_bytes, "frac_of_hbm_peak": step_bytes / (r["decode_ms_per_step"] * 1e-3) / 1e9 / peak,
            "compression": r["compression_at_end"], "n_gpus": world, "device_status": r["device_status"]}


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from fastdms_b200 import _lib
    _lib.lib()          # fail loudly if the CUDA library is missing

    m, seqs, hp, g = build_gpu_workload(dev, seed=1234 + rank)
    fill_activations(hp, g, dev)
    hp.set_positions([CTX] * B)
    hp.capture()                                    # one eager step + capture (state advances by one step)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- value: device-resident step, graph replay --------------------------------------------------
    for _ in range(args.warmup):
        hp.step_device()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks = ClockSampler(local)        # samples SM clock and throttle reasons through every timed region below
    clocks.__enter__()
    e0.record()
    for _ in range(args.steps):
        hp.step_device()
    e1.record()
    barrier()
    step_ms = e0.elapsed_time(e1) / args.steps
    t = torch.tensor([step_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms = float(t.item())
    value = B * world / (step_ms * 1e-3)

    # ---- e2e: host buffers in, host buffers out, every step -----------------------------------------
    bank = 4
    # the step's inputs live in pinned host memory, in blocks laid out like the device input block
    # (what a serving process would keep as its staging buffers): one H2D copy per step
    blocks = [hp.new_host_block() for _ in range(bank)]
    for i, (_, bq, bk, bv, _) in enumerate(blocks):
        bq.copy_(torch.randn(hp.q.shape, generator=torch.Generator().manual_seed(100 + i)).to(hp.q.dtype))
        bk.copy_(torch.randn(hp.k.shape, generator=torch.Generator().manual_seed(200 + i)).to(hp.k.dtype))
        bv.copy_(torch.randn(hp.v.shape, generator=torch.Generator().manual_seed(300 + i)).to(hp.v.dtype))
        lane = torch.where(torch.rand((L, B, HK), generator=torch.Generator().manual_seed(400 + i)) < EVICT_RATE, 1.0, -1.0)
        bq[:, :, 0::HQ // HK, D - 1] = lane.to(bq.dtype)
    pos0 = int(hp.positions[0].item())
    # Host-driven steps are pipelined two deep (DecodeHotPath.submit_host_block / wait_host_block):
    # every step still uploads its own inputs from pinned host memory and its outputs are read back
    # on the host, but the upload of step n+1 and the download of step n-1 overlap the kernels of step n.
    def submit(i):
        nonlocal pos0
        blocks[i % bank][4].fill_(pos0); pos0 += 1
        return hp.submit_host_block(blocks[i % bank][0])

    ticket = submit(0)
    for i in range(1, max(3, args.warmup)):
        nxt = submit(i)
        hp.wait_host_block(ticket)
        ticket = nxt
    hp.wait_host_block(ticket)
    barrier()
    t0 = time.perf_counter()
    e0.record()
    ticket = submit(0)
    checksum = 0.0
    for i in range(1, args.steps):
        nxt = submit(i)
        checksum += float(hp.wait_host_block(ticket)[0, 0, 0, 0])      # the host reads every step's result
        ticket = nxt
    checksum += float(hp.wait_host_block(ticket)[0, 0, 0, 0])
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3) / args.steps
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    e2e_value = B * world / (e2e_ms * 1e-3)

    # ---- roofline of the attention kernel -----------------------------------------------------------
    per_launch_s, bytes_per_launch, attn_launches = time_attention_kernel(hp, dev, reps=max(20, args.steps), overlap=False)
    ov_launch_s, _, _ = time_attention_kernel(hp, dev, reps=max(20, args.steps), overlap=True)
    peak, peak_kind = measured_peaks()
    clocks.__exit__()
    achieved = bytes_per_launch / ov_launch_s / 1e9
    status = _lib.read_device_status(dev)
    launches_per_step, h2d_bytes, d2h_bytes = hp.launches_per_step, hp.h2d_bytes_per_step, hp.d2h_bytes_per_step
    staged = os.environ.get("FDMS_ATTN_LOADER", "")[:1] == "s"
    kernel_name = ("attn_decode_staged_kernel<64, %s>" if staged else "attn_decode_direct_kernel<64, 3, %s>") % (
        "true" if hp.fuse_store else "false")

    # ---- whole-model decode on the same shape (context for `value`; does not change it) --------------
    model_block = None
    if not args.no_model:
        del hp, m, seqs
        torch.cuda.empty_cache()
        try:
            model_block = run_model_block(dev, world, args.model_steps)
        except Exception as e:                                  # the hot-path line must still be printed
            model_block = {"error": f"{type(e).__name__}: {e}"}

    if world > 1:
        dist.barrier()
    if rank == 0:
        line = {
            "metric": "decode tok/s at c=8, 8K ctx (compact-DMS hot path)", "value": value, "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "e4m3 KV / bf16 activations, f32 accumulate", "data": "synthetic",
            "config": workload_config(world),
            "timing": "CUDA events around graph replays, max over ranks",
            "expiry_form": "metadata compacted in order, K/V rows refilled through a row index",
            "e2e": {"value": e2e_value, "unit": "tok/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)",
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "traffic_source": NCU_DRAM_SOURCE,
                         "bytes_per_launch": bytes_per_launch, "us_per_launch": ov_launch_s * 1e6,
                         "us_per_launch_without_overlap": per_launch_s * 1e6, "launches_timed": attn_launches,
                         "how": "CUDA events around a graph of the 16 per-layer launches (the fused decision + RoPE + "
                                "FP8 store + attention launch of the decode step) replayed back to back; "
                                "launches use programmatic dependent launch as in the decode step, so a launch's "
                                "preamble and page prefetch overlap the tail of the one before it; "
                                "us_per_launch_without_overlap is the same stream with ordinary launches"},
            "clocks": clocks.summary(),
            "device_status": status,
        }
        if model_block is not None:
            line["model"] = model_block
        if world == 1 and not args.no_cpu_baseline:
            sample_steps = 8
            per_step, procs = cpu_time_steps(L * B, sample_steps, 1, os.cpu_count() or 1)
            line["cpu_baseline"] = {
                "value": B / per_step, "unit": "tok/s", "cores": procs, "kind": "port",
                "sample": f"{sample_steps} full decode steps (16 layers x 8 sequences x 8 KV heads) of the numpy oracle "
                          f"port of the reference's CPU path (contiguous-span layout), {procs} single-threaded worker "
                          f"processes on {os.cpu_count()} host cores"}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-model", action="store_true", help="skip the whole-model block")
    ap.add_argument("--model-steps", type=int, default=64, help="decode steps of the whole-model block")
    args = ap.parse_args()
    # The one JSON line is the only thing on standard output: libraries that print there from native code (NCCL's
    # version banner under NCCL_DEBUG=WARN, for one) are sent to standard error for the length of the run.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
    sys.stdout.flush()


_RESULT_FD = None


def emit(line: dict) -> None:
    """Writes the result line to the process's original standard output."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


if __name__ == "__main__":
    main()

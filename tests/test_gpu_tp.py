"""Tensor parallelism by KV head (the 8B-shape partition) on two GPUs, checked on the tiny CPU-runnable model:
two ranks, one KV head each, NCCL all-reduce after o_proj and down_proj, against the same reference
trace as the single-GPU test.  DMS state is per KV head, so each rank's decisions and compact
lengths must equal that head's columns of the trace; tokens must be identical.  The float32 case
sums the partials with the library's NVLink peer all-reduce, the FP8 case with NCCL.
Skipped on boxes with fewer than two GPUs."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu
PORT = 29731


TP_STEPS = 32        # decode steps of the two-GPU trace runs (the trace's first stretch, free of near-ties)


def _rank_main(rank: int, world: int, kv_dtype: str, out_q) -> None:
    import os
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(PORT), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), FDMS_PEER_ALLREDUCE="1" if kv_dtype == "float32" else "0")
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    import torch.distributed as dist
    import make_golden_model as G
    from fastdms_b200 import LLM, SamplingParams, _lib
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    try:
        with np.load(ROOT / "tests" / "golden" / "model_golden.npz") as z:
            cos_sin = z["cos_sin_cache"]
        llm = LLM("config0-tiny-llama", hf_config=dict(G.MODEL_CFG), random_init_seed=G.SEED, dtype="float32",
                  kv_cache_dtype=kv_dtype, max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=4096,
                  compact_kv_capacity_tokens=8192, dms_window_size=G.WINDOW, dms_alpha_scale=G.ALPHA_SCALE,
                  dms_alpha_offset=G.ALPHA_OFFSET, tensor_parallel_size=world, device=f"cuda:{rank}")
        cache = llm.model_runner.model.model.layers[0].self_attn.rotary_emb.cos_sin_cache
        ref = torch.from_numpy(cos_sin).to(cache.device)
        cache[: ref.shape[0], 0].copy_(ref)
        sp = SamplingParams(temperature=0.0, max_tokens=TP_STEPS + 1, ignore_eos=True)
        seqs = [llm.add_request(p, sp) for p in G.make_prompts()]
        mgr = llm.model_runner.compact_kv_manager
        assert mgr.num_kv_heads == G.MODEL_CFG["num_key_value_heads"] // world
        llm.step()
        tokens = [[s.completion_token_ids[-1] for s in seqs]]
        prefill_live = torch.stack([mgr.seq_states[s.seq_id].live_counts for s in seqs], dim=1).cpu().numpy()
        evict, live, logits = [], [], []
        for _ in range(TP_STEPS):
            llm.step()
            g = llm.model_runner.graphs[len(seqs)]
            evict.append(g.evict_all.cpu().numpy().copy())
            live.append(g.live.cpu().numpy().copy())
            logits.append(g.logits.float().cpu().numpy().copy())
            tokens.append([s.completion_token_ids[-1] for s in seqs])
        out_q.put((rank, dict(tokens=np.array(tokens), prefill_live=prefill_live, evict=np.stack(evict),
                              live=np.stack(live), logits=np.stack(logits),
                              status=_lib.read_device_status(f"cuda:{rank}"), finished=llm.is_finished())))
        out_q.close(); out_q.join_thread()
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        # leave without interpreter teardown: destroying captured graphs that hold NCCL kernels after
        # the peer has gone can block
        sys.stdout.flush(); sys.stderr.flush()
        os._exit(0 if sys.exc_info()[0] is None else 1)


@pytest.mark.parametrize("tag,kv_dtype", [("f32", "float32"), ("fp8", "float8_e4m3fn")])
def test_tp2_by_kv_head_matches_reference_trace(tag, kv_dtype):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, kv_dtype, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(2):
            rank, res = q.get(timeout=180)
            results[rank] = res
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    assert all(p.exitcode == 0 for p in procs)
    with np.load(ROOT / "tests" / "golden" / "model_golden.npz") as z:
        golden = {k: z[k] for k in z.files}
    for rank in range(2):
        r = results[rank]
        assert r["status"] == 0 and r["finished"]
        assert np.array_equal(r["tokens"], golden[f"{tag}_tokens"][: TP_STEPS + 1]), f"rank {rank}: greedy tokens differ"
        assert np.array_equal(r["prefill_live"], golden[f"{tag}_prefill_live"][:, :, rank:rank + 1])
        assert np.array_equal(r["evict"], golden[f"{tag}_evict"][:TP_STEPS, :, :, rank:rank + 1]), f"rank {rank}: decisions differ"
        assert np.array_equal(r["live"], golden[f"{tag}_live"][:TP_STEPS, :, :, rank:rank + 1]), f"rank {rank}: compact lengths differ"
        rows = [i for i, s_ in enumerate(golden["logit_steps"]) if s_ < TP_STEPS]
        assert np.abs(r["logits"][golden["logit_steps"][rows]] - golden[f"{tag}_logits"][rows]).max() < 2e-2


def _allreduce_rank(rank: int, world: int, out_q) -> None:
    import os
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(PORT + 7), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), FDMS_PEER_ALLREDUCE="1")
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    from fastdms_b200 import _lib
    from fastdms_b200.layers.peer_allreduce import init_peer_all_reduce
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    ok, detail = True, ""
    try:
        ar = init_peer_all_reduce(dev, max_bytes=1 << 20)
        assert ar is not None
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        shapes = [(8, 4096), (8, 2048), (1, 8), (64, 4096), (3, 24)]
        calls = 0
        for it in range(60):
            for dtype in (torch.bfloat16, torch.float32, torch.float16):
                shape = shapes[(it + calls) % len(shapes)]
                x = torch.randn(shape, device=dev, generator=g).to(dtype)
                parts = [torch.empty_like(x) for _ in range(world)]
                dist.all_gather(parts, x)
                want = parts[0].float()
                for p in parts[1:]:
                    want = want + p.float()
                want = want.to(dtype)
                got = x.clone()
                assert ar.fits(got)
                ar.all_reduce_(got)
                calls += 1
                if not torch.equal(got, want):
                    ok, detail = False, f"mismatch at call {calls} {shape} {dtype}"
        # back-to-back calls without host synchronisation, then inside a replayed CUDA graph
        x = torch.randn((8, 4096), device=dev, generator=g).to(torch.bfloat16)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        want = sum(p.float() for p in parts).to(torch.bfloat16)
        ys = [x.clone() for _ in range(200)]
        for y in ys:
            ar.all_reduce_(y)
        torch.cuda.synchronize(dev)
        ok = ok and all(torch.equal(y, want) for y in ys)
        static = x.clone()
        out = torch.empty_like(x)
        ar.all_reduce_(static.clone())
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out.copy_(static)
            ar.all_reduce_(out)
        for _ in range(50):
            graph.replay()
        torch.cuda.synchronize(dev)
        ok = ok and torch.equal(out, want)
        # timing of the two paths for the decode-sized tensor
        def timeit(fn, n=200):
            for _ in range(20):
                fn()
            torch.cuda.synchronize(dev); dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record(); torch.cuda.synchronize(dev)
            return e0.elapsed_time(e1) / n * 1e3
        buf = x.clone()
        t_peer = timeit(lambda: ar.all_reduce_(buf))
        t_nccl = timeit(lambda: dist.all_reduce(buf))
        status = _lib.read_device_status(dev)
        out_q.put((rank, ok and status == 0, detail, t_peer, t_nccl))
        out_q.close(); out_q.join_thread()
        torch.cuda.synchronize(dev)
        dist.barrier()
    finally:
        sys.stdout.flush(); sys.stderr.flush()
        os._exit(0 if sys.exc_info()[0] is None else 1)


def test_peer_allreduce_two_gpus():
    """The NVLink peer all-reduce against the sum of all-gathered inputs in rank order: bit-exact for
    bf16 / f16 / f32, alternating shapes, 200 unsynchronised calls in a row and 50 replays of a captured
    graph.  Also prints its latency next to NCCL's for the decode-sized [8, 4096] bf16 tensor."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_allreduce_rank, args=(r, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(2):
            rank, ok, detail, t_peer, t_nccl = q.get(timeout=180)
            results[rank] = (ok, detail, t_peer, t_nccl)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    print("peer all-reduce us / NCCL us per call:", {r: (round(v[2], 2), round(v[3], 2)) for r, v in results.items()})
    assert all(p.exitcode == 0 for p in procs)
    for rank in range(2):
        assert results[rank][0], f"rank {rank}: {results[rank][1]}"


def _fused_linear_rank(rank: int, world: int, out_q) -> None:
    import os
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(PORT + 13), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), FDMS_FUSED_ROW_PARALLEL="1")
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    from fastdms_b200 import _lib
    from fastdms_b200.layers.linear import linear
    from fastdms_b200.layers.peer_allreduce import init_fused_row_parallel
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    ok, detail = True, ""
    try:
      with torch.inference_mode():
          fused = init_fused_row_parallel(dev)
          assert fused is not None
          g = torch.Generator(device=dev).manual_seed(500 + rank)
          # (rows, out_features, this rank's share of in_features): o_proj / down_proj shards of the 8B shape at 2, 4, 8 ranks
          shapes = [(8, 4096, 2048), (8, 4096, 6144), (8, 4096, 1024), (3, 4096, 1536), (8, 4096, 512), (1, 2048, 256)]
          weights = {s: (torch.randn((s[1], s[2]), device=dev, generator=g) * (world * s[2]) ** -0.5).to(torch.bfloat16) for s in shapes}
          bias = {s: torch.randn((s[1],), device=dev, generator=torch.Generator(device=dev).manual_seed(9)).to(torch.bfloat16) for s in shapes}
          calls = 0
          for it in range(40):
              for s in shapes:
                  rows, n, k = s
                  x = torch.randn((rows, k), device=dev, generator=g).to(torch.bfloat16)
                  b = bias[s] if (it + calls) % 2 else None
                  assert fused.fits(x, weights[s], b)
                  y = fused.linear_all_reduce(x, weights[s], b)
                  calls += 1
                  # float32 reference: every rank's partial, summed in rank order
                  part = x.float() @ weights[s].float().t()
                  parts = [torch.empty_like(part) for _ in range(world)]
                  dist.all_gather(parts, part)
                  ref = parts[0]
                  for p in parts[1:]:
                      ref = ref + p
                  if b is not None:
                      ref = ref + b.float()
                  ys = [torch.empty_like(y) for _ in range(world)]
                  dist.all_gather(ys, y)
                  if not all(torch.equal(ys[0], o) for o in ys[1:]):
                      ok, detail = False, f"ranks disagree at call {calls} {s}"
                  err = float((y.float() - ref).abs().max())
                  if not err <= 2.0 ** -7 * float(ref.abs().max()):
                      ok, detail = False, f"error {err} at call {calls} {s}"
          # 300 calls without host synchronisation, then a replayed CUDA graph of a two-layer chain
          s = shapes[0]
          x = torch.randn((8, s[2]), device=dev, generator=g).to(torch.bfloat16)
          want = fused.linear_all_reduce(x, weights[s], None).clone()
          outs = [fused.linear_all_reduce(x, weights[s], None) for _ in range(300)]
          torch.cuda.synchronize(dev)
          ok = ok and all(torch.equal(o, want) for o in outs)
          s2 = shapes[1]
          x2 = torch.randn((8, s2[2]), device=dev, generator=g).to(torch.bfloat16)
          want2 = fused.linear_all_reduce(x2, weights[s2], None).clone()
          torch.cuda.synchronize(dev)
          graph = torch.cuda.CUDAGraph()
          with torch.cuda.graph(graph):
              o1 = fused.linear_all_reduce(x, weights[s], None)
              o2 = fused.linear_all_reduce(x2, weights[s2], None)
          for _ in range(50):
              graph.replay()
          torch.cuda.synchronize(dev)
          ok = ok and torch.equal(o1, want) and torch.equal(o2, want2)

          def timeit(fn, n=200):
              for _ in range(20):
                  fn()
              torch.cuda.synchronize(dev); dist.barrier()
              e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
              e0.record()
              for _ in range(n):
                  fn()
              e1.record(); torch.cuda.synchronize(dev)
              return e0.elapsed_time(e1) / n * 1e3

          def two_step():
              y = linear(x, weights[s])
              dist.all_reduce(y)
          t_fused = timeit(lambda: fused.linear_all_reduce(x, weights[s], None))
          t_two = timeit(two_step)
          status = _lib.read_device_status(dev)
          out_q.put((rank, ok and status == 0, detail, t_fused, t_two))
          out_q.close(); out_q.join_thread()
          torch.cuda.synchronize(dev)
          dist.barrier()
    except BaseException:
        import traceback
        traceback.print_exc()
        out_q.put((rank, False, traceback.format_exc()[-400:], 0.0, 0.0))
        out_q.close(); out_q.join_thread()
        raise
    finally:
        sys.stdout.flush(); sys.stderr.flush()
        os._exit(0 if sys.exc_info()[0] is None else 1)


def test_fused_linear_allreduce_two_gpus():
    """The row-parallel linear layer fused with its all-reduce on two GPUs, for the o_proj / down_proj shard
    shapes of the 8B model at 2, 4 and 8 ranks: identical bits on both ranks, within one 16-bit rounding of
    the float32 sum of the ranks' partials, 300 unsynchronised calls and 50 replays of a captured graph of
    two chained calls.  Prints its latency next to the two-step path (decode linear kernel, then NCCL)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_fused_linear_rank, args=(r, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(2):
            rank, ok, detail, t_fused, t_two = q.get(timeout=240)
            results[rank] = (ok, detail, t_fused, t_two)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    print("fused linear+all-reduce us / linear then NCCL us per call:", {r: (round(v[2], 2), round(v[3], 2)) for r, v in results.items()})
    assert all(p.exitcode == 0 for p in procs)
    for rank in range(2):
        assert results[rank][0], f"rank {rank}: {results[rank][1]}"


def _tp_bf16_rank(rank: int, world: int, out_q) -> None:
    import os
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(PORT + 21), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), FDMS_PEER_ALLREDUCE="0")
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    import torch.distributed as dist
    import make_golden_model as G
    from fastdms_b200 import LLM, SamplingParams, _lib
    from fastdms_b200.layers import peer_allreduce
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    try:
        try:
            runs = {}
            for fused in ("1", "0"):
                os.environ["FDMS_FUSED_ROW_PARALLEL"] = fused
                cfg = dict(G.MODEL_CFG)
                cfg.update(torch_dtype="bfloat16", lm_head_factor=G.BF16_LM_HEAD_FACTOR)
                llm = LLM("config0-tiny-llama", hf_config=cfg, random_init_seed=G.SEED, dtype="bfloat16",
                          kv_cache_dtype="float8_e4m3fn", max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=4096,
                          compact_kv_capacity_tokens=8192, dms_window_size=G.WINDOW, dms_alpha_scale=G.ALPHA_SCALE,
                          dms_alpha_offset=G.ALPHA_OFFSET, tensor_parallel_size=world, device=f"cuda:{rank}")
                assert (peer_allreduce.fused_row_parallel() is not None) == (fused == "1")
                sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
                seqs = [llm.add_request(p, sp) for p in G.make_prompts()]
                llm.step()
                logits = []
                for _ in range(4):
                    llm.step()
                    logits.append(llm.model_runner.graphs[len(seqs)].logits.float().cpu().numpy().copy())
                    # follow the same history in both runs: a near-tie must not send them apart
                    if fused == "1":
                        runs.setdefault("tokens", []).append([s.completion_token_ids[-1] for s in seqs])
                    else:
                        for s, tok in zip(seqs, runs["tokens"][len(logits) - 1]):
                            s.token_ids[-1] = tok
                            s.last_token = tok
                runs[fused] = np.stack(logits)
                torch.cuda.synchronize()
                dist.barrier()
            out_q.put((rank, True, "", runs["1"], runs["0"], _lib.read_device_status(f"cuda:{rank}")))
        except BaseException:
            import traceback
            traceback.print_exc()
            out_q.put((rank, False, traceback.format_exc()[-600:], None, None, -1))
            raise
        finally:
            out_q.close(); out_q.join_thread()
    finally:
        sys.stdout.flush(); sys.stderr.flush()
        os._exit(0 if sys.exc_info()[0] is None else 1)


def test_tp2_bf16_fused_row_parallel_matches_nccl_path():
    """The tiny model in bf16 on two GPUs, decode steps with the row-parallel layers fused with their all-reduce
    against the same steps with the linear kernel followed by NCCL, on the same token history: logits within
    16-bit rounding of each other (the fused path rounds the sum once, NCCL adds rounded partials), identical
    on both ranks."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_tp_bf16_rank, args=(r, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(2):
            rank, ok, detail, fused, nccl, status = q.get(timeout=240)
            results[rank] = (ok, detail, fused, nccl, status)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    for rank in range(2):
        ok, detail, fused, nccl, status = results[rank]
        assert ok, f"rank {rank}: {detail}"
        assert status == 0
        scale = float(np.abs(nccl).max())
        assert np.abs(fused - nccl).max() <= 3e-2 * scale, (np.abs(fused - nccl).max(), scale)
    assert np.array_equal(results[0][2], results[1][2]), "ranks disagree on the fused path's logits"
    assert all(p.exitcode == 0 for p in procs)

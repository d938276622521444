"""The engine loop (`LLMEngine.step` + `Scheduler`) over a simulated page pool, no GPU: a stand-in
manager that counts pages per request (kept rows = a fraction of the tokens + the window) and a
stand-in runner that takes pages for prefill chunks and decode tokens.  Properties checked for
continuous-batching workloads of config-5 shape on pools from roomy to tight, with admission
estimates that are right, low and far too low: every request finishes (no livelock, bounded number
of steps), no decode step runs dry, the pool returns to its initial state, and with chunked prefill
no prompt token is computed twice unless a request was preempted."""
from __future__ import annotations

import math
import random
from types import SimpleNamespace

import pytest

from fastdms_b200.engine.llm_engine import LLMEngine
from fastdms_b200.engine.scheduler import Scheduler
from fastdms_b200.engine.sequence import Sequence
from fastdms_b200.sampling_params import SamplingParams

PAGE = 16


class SimManager:
    def __init__(self, pages, keep_true, keep_est, hk=8, window=256):
        self.total = self.free = pages
        self.hk, self.window, self.keep_true, self.keep_est = hk, window, keep_true, keep_est
        self.held: dict[int, int] = {}

    def pages_for(self, tokens):
        rows = min(tokens, int(tokens * self.keep_true) + self.window)
        return -(-rows // PAGE) * self.hk

    def admission_need(self, seq):                       # the optimistic estimate of CompactKVManager
        est = int(seq.num_tokens * self.keep_est) + self.window + max(seq.max_tokens - seq.num_completion_tokens, 0) + 1
        rows = min(seq.num_prompt_tokens + seq.max_tokens, est)
        return -(-rows // PAGE) * PAGE * self.hk

    def can_allocate(self, seq, pending=0):
        return self.admission_need(seq) + pending <= self.free * PAGE

    def decode_pages_guaranteed(self, batch):
        return self.free >= batch * self.hk

    def prefill_pages_guaranteed(self, tokens, num_seqs):
        return self.free >= (-(-tokens // PAGE) + num_seqs) * self.hk

    def take(self, sid, tokens):
        need = self.pages_for(tokens) - self.held.get(sid, 0)
        if need > self.free:
            return False
        self.free -= need
        self.held[sid] = self.held.get(sid, 0) + need
        return True


class SimRunner:
    def __init__(self, mgr, chunk):
        self.compact_kv_manager, self.chunk = mgr, chunk

    def run(self, seqs, is_prefill):
        m = self.compact_kv_manager
        for s in seqs:
            if is_prefill:
                upto = s.num_cached_tokens + s.num_scheduled_tokens if self.chunk else len(s)
                if not m.take(s.seq_id, upto):
                    raise RuntimeError("compact KV capacity exhausted (simulated pool)")
            else:
                assert m.take(s.seq_id, len(s) + 1), "a decode step ran dry despite the guard"
        return [1] * len(seqs)

    def free_compact(self, ids):
        m = self.compact_kv_manager
        for i in ids:
            m.free += m.held.pop(i, 0)


def simulate(seed, pages, keep_true, keep_est, chunk, n=24, max_seqs=12, max_prompt=16384, max_steps=30000):
    rng = random.Random(seed)
    cfg = SimpleNamespace(max_num_seqs=max_seqs, max_num_batched_tokens=8192 if chunk else 2 * max_prompt, eos=-1,
                          prefill_chunk_size=chunk)
    mgr = SimManager(pages, keep_true, keep_est)
    eng = LLMEngine.__new__(LLMEngine)
    eng.config, eng.model_runner = cfg, SimRunner(mgr, chunk)
    eng.scheduler = Scheduler(cfg, can_allocate=mgr.can_allocate, admission_need=mgr.admission_need,
                              prefill_guard=mgr.prefill_pages_guaranteed if chunk else None)
    seqs = [Sequence(list(range(int(math.exp(rng.uniform(math.log(512), math.log(max_prompt)))))),
                     SamplingParams(temperature=0.0, max_tokens=rng.randint(64, 256), ignore_eos=True)) for _ in range(n)]
    todo, steps, prefill_tokens = list(seqs), 0, 0
    while todo or not eng.is_finished():
        for _ in range(2):                               # two arrivals per step
            if todo:
                eng.scheduler.add(todo.pop(0))
        _, nt = eng.step()
        steps += 1
        prefill_tokens += max(nt, 0)
        assert steps <= max_steps, "the engine loop does not terminate"
    assert all(s.is_finished and s.num_completion_tokens == s.max_tokens for s in seqs)
    assert mgr.free == mgr.total and not mgr.held, "pages were leaked"
    return eng.scheduler, prefill_tokens, sum(s.num_prompt_tokens for s in seqs)


@pytest.mark.parametrize("chunk", [2048, None])
@pytest.mark.parametrize("pages", [20000, 6000, 4000])
@pytest.mark.parametrize("keep_true,keep_est", [(0.16, 0.2), (0.3, 0.05), (0.4, 0.02)])
def test_engine_loop_terminates_and_returns_the_pool(chunk, pages, keep_true, keep_est):
    for seed in (1, 2):
        sched, prefill_tokens, prompt_tokens = simulate(seed, pages, keep_true, keep_est, chunk)
        if chunk:
            assert sched.prefill_retries == 0, "with the page guard a chunk is only launched when it fits"
            if sched.preemptions == 0:
                assert prefill_tokens == prompt_tokens


def test_a_request_that_cannot_fit_alone_is_an_error_not_a_hang():
    with pytest.raises(RuntimeError):
        simulate(1, 1500, 0.9, 0.02, 2048)
    with pytest.raises(RuntimeError):
        simulate(1, 1500, 0.9, 0.02, None)

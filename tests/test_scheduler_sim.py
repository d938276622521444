"""The engine loop (`LLMEngine.step` + `Scheduler`) over a simulated page pool, no GPU: a stand-in
manager that counts pages per request (kept rows = a fraction of the tokens + the window) and a
stand-in runner that takes pages for prefill chunks and decode tokens.  Properties checked for
continuous-batching workloads of config-5 shape on pools from roomy to tight, with admission
estimates that are right, low and far too low: every request finishes (no livelock, bounded number
of steps), no decode step runs dry, the pool returns to its initial state, and with chunked prefill
no prompt token is computed twice unless a request was preempted.  With run-ahead decode (the next
step launched before this step's tokens are read) the same workloads must give the same tokens as
the synchronous loop, never free a request's pages while a step in flight still reads them, and
leave nothing in flight at the end."""
from __future__ import annotations

import itertools
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


EOS = 7


def sim_token(seq_id, length):
    """The token a request emits when it holds `length` tokens (a fixed function, so that the
    synchronous and the run-ahead loop can be compared); the value 7 is the end-of-sequence id."""
    return (seq_id * 31 + length * 17) % 23


class SimRunner:
    """Stand-in for ModelRunner.  In run-ahead mode it keeps what the real runner keeps on the
    device: the batch of the last launched step and every request's length as that step saw it."""

    def __init__(self, mgr, chunk, run_ahead=False):
        self.compact_kv_manager, self.chunk, self.run_ahead = mgr, chunk, run_ahead
        self.sync_steps_of_batch: dict[int, int] = {}     # a batch size needs two synchronous steps (warm-up, capture)
        self.device_batch: list[int] = []
        self.device_len: dict[int, int] = {}
        self.in_flight: list[list[int]] = []
        self.ahead_launches = 0

    def run(self, seqs, is_prefill):
        m = self.compact_kv_manager
        for s in seqs:
            if is_prefill:
                upto = s.num_cached_tokens + s.num_scheduled_tokens if self.chunk else len(s)
                if not m.take(s.seq_id, upto):
                    raise RuntimeError("compact KV capacity exhausted (simulated pool)")
            else:
                assert m.take(s.seq_id, len(s) + 1), "a decode step ran dry despite the guard"
        if not is_prefill:
            self.sync_steps_of_batch[len(seqs)] = self.sync_steps_of_batch.get(len(seqs), 0) + 1
        return [sim_token(s.seq_id, len(s)) for s in seqs]

    def can_run_ahead(self, seqs):
        return self.run_ahead and self.sync_steps_of_batch.get(len(seqs), 0) >= 2 and all(s.temperature <= 1e-10 for s in seqs)

    def launch_decode(self, seqs, device_fed):
        m = self.compact_kv_manager
        ids = [s.seq_id for s in seqs]
        if device_fed:
            assert ids == self.device_batch, "a device-fed step must repeat the previous batch"
            assert len(self.in_flight) == 1, "the step before a device-fed one has not been read yet"
            lens = [self.device_len[i] + 1 for i in ids]
            self.ahead_launches += 1
        else:
            assert not self.in_flight
            lens = [len(s) for s in seqs]
        for s, n in zip(seqs, lens):
            assert m.take(s.seq_id, n + 1), "a decode step ran dry despite the guard"
        self.device_batch, self.device_len = ids, dict(zip(ids, lens))
        self.in_flight.append(ids)
        return ids, [sim_token(i, n) for i, n in zip(ids, lens)]

    def resolve_decode(self, handle):
        ids, tokens = handle
        assert self.in_flight and self.in_flight[0] is ids, "steps are read in launch order"
        self.in_flight.pop(0)
        return tokens

    def free_compact(self, ids):
        m = self.compact_kv_manager
        for i in ids:
            assert all(i not in step for step in self.in_flight), "pages freed under a step that still reads them"
            m.free += m.held.pop(i, 0)


def simulate(seed, pages, keep_true, keep_est, chunk, n=24, max_seqs=12, max_prompt=16384, max_steps=30000,
             run_ahead=False, eos_every=0, result=None):
    rng = random.Random(seed)
    cfg = SimpleNamespace(max_num_seqs=max_seqs, max_num_batched_tokens=8192 if chunk else 2 * max_prompt,
                          eos=EOS if eos_every else -1, prefill_chunk_size=chunk, decode_run_ahead=run_ahead)
    mgr = SimManager(pages, keep_true, keep_est)
    eng = LLMEngine.__new__(LLMEngine)
    eng.config, eng.model_runner = cfg, SimRunner(mgr, chunk, run_ahead)
    eng.scheduler = Scheduler(cfg, can_allocate=mgr.can_allocate, admission_need=mgr.admission_need,
                              prefill_guard=mgr.prefill_pages_guaranteed if chunk else None)
    seqs = [Sequence(list(range(int(math.exp(rng.uniform(math.log(512), math.log(max_prompt)))))),
                     SamplingParams(temperature=0.0, max_tokens=rng.randint(64, 256),
                                    ignore_eos=not (eos_every and i % eos_every == 0))) for i in range(n)]
    todo, steps, prefill_tokens = list(seqs), 0, 0
    while todo or not eng.is_finished():
        for _ in range(2):                               # two arrivals per step
            if todo:
                eng.scheduler.add(todo.pop(0))
        _, nt = eng.step()
        steps += 1
        prefill_tokens += max(nt, 0)
        assert steps <= max_steps, "the engine loop does not terminate"
    for s in seqs:
        assert s.is_finished
        if s.ignore_eos:
            assert s.num_completion_tokens == s.max_tokens
        else:
            done = s.completion_token_ids
            assert (done[-1] == EOS and EOS not in done[:-1]) or (len(done) == s.max_tokens and EOS not in done[:-1])
    assert mgr.free == mgr.total and not mgr.held, "pages were leaked"
    assert eng._ahead is None and not eng._deferred_free and not eng.model_runner.in_flight
    if result is not None:
        result["tokens"] = [list(s.completion_token_ids) for s in seqs]
        result["ahead_launches"] = eng.model_runner.ahead_launches
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


@pytest.mark.parametrize("chunk", [2048, None])
@pytest.mark.parametrize("pages,keep_true,keep_est", [(20000, 0.16, 0.2), (6000, 0.3, 0.05), (4000, 0.4, 0.02)])
def test_run_ahead_loop_gives_the_tokens_of_the_synchronous_loop(chunk, pages, keep_true, keep_est):
    """Every third request may stop on the end-of-sequence id, i.e. at a step whose successor has
    already been launched; the others stop on their token limit, which is known in advance."""
    for seed in (1, 2):
        sync, ahead = {}, {}
        saved = Sequence.counter
        try:
            # the simulated tokens depend on the request id: give both runs the same ids
            Sequence.counter = itertools.count(1000)
            simulate(seed, pages, keep_true, keep_est, chunk, eos_every=3, result=sync)
            Sequence.counter = itertools.count(1000)
            simulate(seed, pages, keep_true, keep_est, chunk, eos_every=3, run_ahead=True, result=ahead)
        finally:
            Sequence.counter = saved
        assert sync["tokens"] == ahead["tokens"]
        assert any(t[-1] == EOS and len(t) < 64 for t in sync["tokens"]), "no request stopped on the end-of-sequence id"
        assert ahead["ahead_launches"] > 100 and sync["ahead_launches"] == 0


def test_a_request_that_cannot_fit_alone_is_an_error_not_a_hang():
    with pytest.raises(RuntimeError):
        simulate(1, 1500, 0.9, 0.02, 2048)
    with pytest.raises(RuntimeError):
        simulate(1, 1500, 0.9, 0.02, None)

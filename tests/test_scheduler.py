"""Host-side scheduler logic (no GPU): admission accounting within one pass, and the retry policy of
optimistic admission (requeue at the front, halved prefill batch, hold while requests are running)."""
from __future__ import annotations

from types import SimpleNamespace

import pytest

from fastdms_b200.engine.scheduler import Scheduler
from fastdms_b200.engine.sequence import Sequence, SequenceStatus
from fastdms_b200.sampling_params import SamplingParams


class Pool:
    """Stand-in for the manager's admission interface: every request is charged its prompt length."""

    def __init__(self, free):
        self.free = free
        self.denied = 0

    def need(self, seq):
        return seq.num_prompt_tokens

    def can_allocate(self, seq, pending=0):
        ok = self.need(seq) + pending <= self.free
        self.denied += not ok
        return ok


def _sched(pool, max_seqs=8, budget=10_000):
    cfg = SimpleNamespace(max_num_seqs=max_seqs, max_num_batched_tokens=budget, eos=-1)
    return Scheduler(cfg, can_allocate=pool.can_allocate, admission_need=pool.need)


def _seq(n, max_tokens=2):
    return Sequence(list(range(n)), SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True))


def test_rows_promised_earlier_in_the_pass_count():
    pool = Pool(free=100)
    s = _sched(pool)
    a, b = _seq(60), _seq(60)
    s.add(a); s.add(b)
    batch, is_prefill = s.schedule()
    assert is_prefill and batch == [a] and list(s.waiting) == [b] and pool.denied == 1
    pool.free -= 60                                   # the prefill took its rows
    batch, is_prefill = s.schedule()                  # b still does not fit: decode a
    assert not is_prefill and batch == [a]
    s.postprocess([a], [7], False); s.postprocess([a], [7], False)
    assert a.status == SequenceStatus.FINISHED and s.consume_freed_seq_ids() == [a.seq_id]
    pool.free += 60
    batch, is_prefill = s.schedule()
    assert is_prefill and batch == [b]


def test_failed_prefill_is_requeued_in_order_and_the_batch_halves():
    pool = Pool(free=10_000)
    s = _sched(pool)
    seqs = [_seq(10 + i) for i in range(4)]
    for q in seqs:
        s.add(q)
    batch, _ = s.schedule()
    assert batch == seqs
    s.requeue(batch)
    assert list(s.waiting) == seqs and not s.running and s.prefill_retries == 1
    assert all(q.status == SequenceStatus.WAITING for q in seqs)
    batch, is_prefill = s.schedule()
    assert is_prefill and batch == seqs[:2]           # half the failed batch
    s.prefill_succeeded()
    batch, is_prefill = s.schedule()
    assert is_prefill and batch == seqs[2:]           # the limit is gone after a success


def test_single_failure_waits_for_a_running_request_to_finish():
    pool = Pool(free=10_000)
    s = _sched(pool)
    a, b = _seq(10, max_tokens=2), _seq(20)
    s.add(a)
    assert s.schedule() == ([a], True)
    s.prefill_succeeded()
    s.postprocess([a], [1], True)
    s.add(b)
    assert s.schedule() == ([b], True)
    s.requeue([b])                                     # did not fit while a is running
    assert s.hold_prefill and list(s.waiting) == [b]
    assert s.schedule() == ([a], False)                # no new prefill attempt: decode
    s.postprocess([a], [1], False)                     # a finishes -> capacity came back
    assert a.status == SequenceStatus.FINISHED and not s.hold_prefill
    assert s.schedule() == ([b], True)


def test_request_that_cannot_fit_alone_raises():
    pool = Pool(free=10_000)
    s = _sched(pool)
    a = _seq(10)
    s.add(a)
    batch, _ = s.schedule()
    with pytest.raises(RuntimeError, match="even alone"):
        s.requeue(batch)


def test_nothing_admissible_and_nothing_running_raises():
    pool = Pool(free=5)
    s = _sched(pool)
    s.add(_seq(10))
    with pytest.raises(RuntimeError, match="no request fits"):
        s.schedule()


def test_chunked_prefill_schedules_prompts_in_pieces():
    """prefill_chunk_size: continuing prompts first, new ones while the token budget lasts; only the
    chunk that ends a prompt yields a token; decode starts when no prompt is pending."""
    pool = Pool(free=10_000)
    cfg = SimpleNamespace(max_num_seqs=8, max_num_batched_tokens=100, eos=-1, prefill_chunk_size=64)
    s = Scheduler(cfg, can_allocate=pool.can_allocate, admission_need=pool.need)
    a, b = _seq(150), _seq(40)
    s.add(a)
    s.add(b)
    batch, is_prefill = s.schedule()                     # a: 64 of 150; b: 36 left in the budget < 40 -> waits
    assert is_prefill and batch == [a] and a.num_scheduled_tokens == 64
    s.postprocess(batch, [7], True)
    assert a.num_cached_tokens == 64 and a.num_completion_tokens == 0
    batch, is_prefill = s.schedule()                     # a continues (64), b does not fit beside it (36 < 40)
    assert is_prefill and batch == [a] and a.num_scheduled_tokens == 64
    s.postprocess(batch, [7], True)
    batch, is_prefill = s.schedule()                     # a's last 22 tokens + b's 40
    assert is_prefill and batch == [a, b] and (a.num_scheduled_tokens, b.num_scheduled_tokens) == (22, 40)
    s.postprocess(batch, [11, 12], True)
    assert a.completion_token_ids == [11] and b.completion_token_ids == [12]
    assert a.num_cached_tokens == a.num_tokens == 151
    batch, is_prefill = s.schedule()
    assert not is_prefill and batch == [a, b]
    s.postprocess(batch, [1, 2], False)
    assert a.is_finished and b.is_finished and s.is_finished()
    with pytest.raises(ValueError):
        Scheduler(SimpleNamespace(max_num_seqs=8, max_num_batched_tokens=100, eos=-1, prefill_chunk_size=128))


def test_requeue_restarts_a_chunked_prompt():
    pool = Pool(free=10_000)
    cfg = SimpleNamespace(max_num_seqs=8, max_num_batched_tokens=100, eos=-1, prefill_chunk_size=64)
    s = Scheduler(cfg, can_allocate=pool.can_allocate, admission_need=pool.need)
    a, b = _seq(100), _seq(30)
    s.add(a)
    s.add(b)
    batch, _ = s.schedule()
    assert batch == [a, b]
    s.postprocess(batch, [5, 6], True)                   # b is done prefilling, a is half way
    batch, _ = s.schedule()
    assert batch == [a]
    s.requeue([a])                                       # its second chunk did not fit the pool
    assert a.num_cached_tokens == 0 and a.status == SequenceStatus.WAITING and s.waiting[0] is a


def test_preempt_youngest_requeues_for_recompute():
    pool = Pool(free=10_000)
    s = _sched(pool)
    a, b, c = _seq(10, max_tokens=5), _seq(20, max_tokens=5), _seq(30, max_tokens=5)
    for x in (a, b, c):
        s.add(x)
    batch, _ = s.schedule()
    s.postprocess(batch, [1, 2, 3], True)
    batch, is_prefill = s.schedule()
    assert not is_prefill and batch == [a, b, c]
    victim = s.preempt_youngest(batch)
    assert victim is c and c.status == SequenceStatus.WAITING and s.waiting[0] is c
    assert c.num_cached_tokens == 0 and c.num_preemptions == 1 and c.num_tokens == 31
    assert list(s.running) == [a, b] and s.hold_prefill
    batch, is_prefill = s.schedule()                     # held while others run
    assert not is_prefill and batch == [a, b]
    for _ in range(4):
        batch, _ = s.schedule()
        s.postprocess(batch, [4] * len(batch), False)
    assert a.is_finished and b.is_finished
    batch, is_prefill = s.schedule()                     # capacity came back: prompt + generated token again
    assert is_prefill and batch == [c] and c.num_scheduled_tokens == 31
    with pytest.raises(RuntimeError):
        s.preempt_youngest([c])

"""Prefill-first scheduler for compact-DMS serving (reference: fastdms/engine/scheduler.py).

A waiting request is admitted when the token budget allows its whole prompt (the DMS prefill packs
a prompt in one step, as in the reference) and the compact pool can take the rows it is charged in
every layer (`CompactKVManager.can_allocate`, which the reference defines but never calls).  Rows
promised to requests admitted earlier in the same pass count against later ones.

Two admission modes (the manager's `admission`):
  * `reserve`   - a request is charged its worst case, so a prefill can never fail;
  * `optimistic` - a request is charged an estimate of what DMS keeps.  If a prefill then does not
    fit, the engine releases what it had taken and calls `requeue`: the requests go back to the front
    of the queue, the next prefill batch is at most half as large, and while requests are running no
    new prefill is tried until one of them finishes (its spans come back).  Running requests own
    their spans including the decode headroom, so decode itself never runs out: nothing that has
    started is ever preempted."""
from __future__ import annotations

from collections import deque

from fastdms_b200.engine.sequence import Sequence, SequenceStatus


class Scheduler:
    def __init__(self, config, can_allocate=None, admission_need=None):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = config.eos
        self.can_allocate = can_allocate or (lambda seq, pending=0: True)
        self.admission_need = admission_need or (lambda seq: 0)
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()
        self.freed_seq_ids: list[int] = []
        self.prefill_batch_limit: int | None = None     # set after a prefill that did not fit
        self.hold_prefill = False                        # wait for a running request to finish first
        self.prefill_retries = 0

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def schedule(self) -> tuple[list[Sequence], bool]:
        scheduled: list[Sequence] = []
        budget = self.max_num_batched_tokens
        pending = 0
        limit = self.prefill_batch_limit if self.prefill_batch_limit is not None else self.max_num_seqs
        hold = self.hold_prefill and bool(self.running)
        while (not hold and self.waiting and len(scheduled) < limit
               and len(self.running) + len(scheduled) < self.max_num_seqs):
            seq = self.waiting[0]
            n = seq.num_tokens
            if n > self.max_num_batched_tokens:
                raise RuntimeError(f"prompt of {n} tokens exceeds max_num_batched_tokens={self.max_num_batched_tokens}")
            if n > budget or not self.can_allocate(seq, pending):
                break
            pending += self.admission_need(seq)
            seq.num_scheduled_tokens = n
            seq.status = SequenceStatus.RUNNING
            self.waiting.popleft()
            scheduled.append(seq)
            budget -= n
        if scheduled:
            self.running.extend(scheduled)
            return scheduled, True
        if not self.running:
            raise RuntimeError("no request fits the compact KV pool / token budget")
        batch = list(self.running)[: self.max_num_seqs]
        for seq in batch:
            seq.num_scheduled_tokens = 1
        return batch, False

    def requeue(self, seqs: list[Sequence]) -> None:
        """A prefill of `seqs` did not fit: put them back at the front, in order, and back off."""
        if len(seqs) == 1 and len(self.running) == 1:
            raise RuntimeError(f"request {seqs[0].seq_id} does not fit the compact KV pool even alone")
        for seq in reversed(seqs):
            self.running.remove(seq)
            seq.status = SequenceStatus.WAITING
            seq.num_scheduled_tokens = 0
            self.waiting.appendleft(seq)
        self.prefill_retries += 1
        if len(seqs) > 1:
            self.prefill_batch_limit = max(1, len(seqs) // 2)
        else:
            self.hold_prefill = True

    def prefill_succeeded(self) -> None:
        self.prefill_batch_limit = None

    def postprocess(self, seqs: list[Sequence], token_ids: list[int], is_prefill: bool) -> None:
        for seq, token_id in zip(seqs, token_ids):
            seq.append_token(token_id)
            seq.num_cached_tokens = seq.num_tokens
            seq.num_scheduled_tokens = 0
            if (not seq.ignore_eos and token_id == self.eos) or seq.num_completion_tokens >= seq.max_tokens:
                seq.status = SequenceStatus.FINISHED
                self.freed_seq_ids.append(seq.seq_id)
                self.running.remove(seq)
                self.hold_prefill = False            # capacity came back

    def consume_freed_seq_ids(self) -> list[int]:
        out, self.freed_seq_ids = self.freed_seq_ids, []
        return out

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
    their spans including the decode headroom, so decode itself never runs out.  With the paged
    layout pages are taken during decode: before a decode step the engine asks the manager whether every
    span could take a page (`decode_pages_guaranteed`); if not, `preempt_youngest` sends the request
    that started last back to the queue (preempt-by-recompute: it is prefilled again later over prompt
    + generated tokens) until the step is safe.

With `prefill_chunk_size` set, a prompt enters the pool in chunks of that many tokens (an extension:
the reference prefills in one pass).  A step then carries the next chunk of every request whose
prompt is only partly in, plus first chunks of newly admitted requests while the token budget
lasts; decode steps run when no prompt is pending.  Only the chunk that ends a prompt yields a
token."""
from __future__ import annotations

from collections import deque

from fastdms_b200.engine.sequence import Sequence, SequenceStatus


class Scheduler:
    def __init__(self, config, can_allocate=None, admission_need=None, prefill_guard=None):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = config.eos
        self.can_allocate = can_allocate or (lambda seq, pending=0: True)
        self.admission_need = admission_need or (lambda seq: 0)
        # chunked prefill over a paged pool: prefill_guard(tokens, seqs) says whether a prefill step of
        # that size is certain to find its pages (None: prefills are tried and retried instead)
        self.prefill_guard = prefill_guard
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()
        self.freed_seq_ids: list[int] = []
        self.prefill_batch_limit: int | None = None     # set after a prefill that did not fit
        self.hold_prefill = False                        # wait for a running request to finish first
        self.prefill_retries = 0
        self.preemptions = 0
        self.prefill_chunk_size = getattr(config, "prefill_chunk_size", None) or None
        if self.prefill_chunk_size is not None and not 0 < self.prefill_chunk_size <= self.max_num_batched_tokens:
            raise ValueError("prefill_chunk_size must be positive and at most max_num_batched_tokens")

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
        chunk = self.prefill_chunk_size
        continuing: list[Sequence] = []
        guard = self.prefill_guard if chunk else None
        taken = 0                                        # tokens of this prefill step so far
        blocked = False                                  # the page guard stopped the batch from growing
        if chunk:
            for seq in self.running:
                left = seq.num_tokens - seq.num_cached_tokens
                if left <= 0:
                    continue
                n = min(chunk, left)
                if n > budget:
                    break
                if guard is not None and not guard(taken + n, len(continuing) + 1):
                    blocked = True
                    break
                seq.num_scheduled_tokens = n
                continuing.append(seq)
                budget -= n
                taken += n
        hold = hold or blocked
        while (not hold and self.waiting and len(scheduled) < limit
               and len(self.running) + len(scheduled) < self.max_num_seqs):
            seq = self.waiting[0]
            n = min(chunk, seq.num_tokens) if chunk else seq.num_tokens
            if n > self.max_num_batched_tokens:
                raise RuntimeError(f"prompt of {n} tokens exceeds max_num_batched_tokens={self.max_num_batched_tokens}")
            if n > budget or not self.can_allocate(seq, pending):
                break
            if guard is not None and not guard(taken + n, len(continuing) + len(scheduled) + 1):
                blocked = True
                break
            taken += n
            pending += self.admission_need(seq)
            seq.num_scheduled_tokens = n
            seq.status = SequenceStatus.RUNNING
            self.waiting.popleft()
            scheduled.append(seq)
            budget -= n
        if scheduled or continuing:
            self.running.extend(scheduled)
            return continuing + scheduled, True
        if not self.running:
            raise RuntimeError("no request fits the compact KV pool / token budget")
        batch = [seq for seq in self.running if not chunk or seq.num_cached_tokens >= seq.num_tokens][: self.max_num_seqs]
        if not batch:
            # only partly prefilled prompts are running and the pool cannot take another chunk: the one
            # that started last gives its pages back (the caller frees them) and waits
            partly = list(self.running)
            if len(partly) <= 1:
                raise RuntimeError("the compact KV pool cannot take the next chunk of a lone request")
            self._send_back(partly[-1])
            self.freed_seq_ids.append(partly[-1].seq_id)
            return [], True
        for seq in batch:
            seq.num_scheduled_tokens = 1
        return batch, False

    def _send_back(self, seq: Sequence) -> None:
        self.running.remove(seq)
        seq.status = SequenceStatus.WAITING
        seq.num_scheduled_tokens = 0
        seq.num_cached_tokens = 0
        seq.num_preemptions += 1
        self.waiting.appendleft(seq)
        self.hold_prefill = True                     # wait for a running request to finish before retrying
        self.preemptions += 1

    def requeue(self, seqs: list[Sequence]) -> None:
        """A prefill of `seqs` did not fit: put them back at the front, in order, and back off."""
        if len(seqs) == 1 and len(self.running) == 1:
            raise RuntimeError(f"request {seqs[0].seq_id} does not fit the compact KV pool even alone")
        for seq in reversed(seqs):
            self.running.remove(seq)
            seq.status = SequenceStatus.WAITING
            seq.num_scheduled_tokens = 0
            seq.num_cached_tokens = 0
            self.waiting.appendleft(seq)
        self.prefill_retries += 1
        if len(seqs) > 1:
            self.prefill_batch_limit = max(1, len(seqs) // 2)
        else:
            self.hold_prefill = True

    def preempt_youngest(self, batch: list[Sequence]) -> Sequence:
        """Preempt-by-recompute (paged layout, when a decode step could run out of pages): the request
        that started last leaves the running set, its pages are freed by the caller, and it goes to the
        front of the queue to be prefilled again later over prompt + generated tokens."""
        if len(batch) <= 1:
            raise RuntimeError("the compact KV pool cannot hold even one running request")
        seq = batch[-1]
        self._send_back(seq)
        return seq

    def prefill_succeeded(self) -> None:
        self.prefill_batch_limit = None

    def postprocess(self, seqs: list[Sequence], token_ids: list[int], is_prefill: bool) -> None:
        for seq, token_id in zip(seqs, token_ids):
            if is_prefill and self.prefill_chunk_size:
                seq.num_cached_tokens += seq.num_scheduled_tokens
                if seq.num_cached_tokens < seq.num_tokens:             # more of the prompt to come: no token yet
                    seq.num_scheduled_tokens = 0
                    continue
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

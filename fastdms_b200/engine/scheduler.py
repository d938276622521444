"""Prefill-first scheduler for compact-DMS serving (reference: fastdms/engine/scheduler.py).

A waiting request is admitted when the token budget allows its whole prompt (the DMS prefill packs
a prompt in one step, as in the reference) and the compact pool can hold its worst-case
reservation in every layer (`CompactKVManager.can_allocate`, which the reference defines but never
calls).  Running requests decode one token per step; because admission is conservative a running
request never has to be preempted."""
from __future__ import annotations

from collections import deque

from fastdms_b200.engine.sequence import Sequence, SequenceStatus


class Scheduler:
    def __init__(self, config, can_allocate=None):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = config.eos
        self.can_allocate = can_allocate or (lambda seq: True)
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()
        self.freed_seq_ids: list[int] = []

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def schedule(self) -> tuple[list[Sequence], bool]:
        scheduled: list[Sequence] = []
        budget = self.max_num_batched_tokens
        while self.waiting and len(self.running) + len(scheduled) < self.max_num_seqs:
            seq = self.waiting[0]
            n = seq.num_tokens
            if n > self.max_num_batched_tokens:
                raise RuntimeError(f"prompt of {n} tokens exceeds max_num_batched_tokens={self.max_num_batched_tokens}")
            if n > budget or not self.can_allocate(seq):
                break
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

    def postprocess(self, seqs: list[Sequence], token_ids: list[int], is_prefill: bool) -> None:
        for seq, token_id in zip(seqs, token_ids):
            seq.append_token(token_id)
            seq.num_cached_tokens = seq.num_tokens
            seq.num_scheduled_tokens = 0
            if (not seq.ignore_eos and token_id == self.eos) or seq.num_completion_tokens >= seq.max_tokens:
                seq.status = SequenceStatus.FINISHED
                self.freed_seq_ids.append(seq.seq_id)
                self.running.remove(seq)

    def consume_freed_seq_ids(self) -> list[int]:
        out, self.freed_seq_ids = self.freed_seq_ids, []
        return out

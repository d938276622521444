"""Request loop: scheduler + model runner (reference: fastdms/engine/llm_engine.py)."""
from __future__ import annotations

from dataclasses import fields
from time import perf_counter

from fastdms_b200.config import Config
from fastdms_b200.engine.model_runner import ModelRunner
from fastdms_b200.engine.scheduler import Scheduler
from fastdms_b200.engine.sequence import Sequence
from fastdms_b200.sampling_params import SamplingParams


class LLMEngine:
    # run-ahead decode state (class-level defaults: "nothing in flight")
    _ahead = None
    _deferred_free: list = []

    def __init__(self, model, **kwargs):
        names = {f.name for f in fields(Config)}
        config = Config(model, **{k: v for k, v in kwargs.items() if k in names})
        self.config = config
        self.model_runner = ModelRunner(config, device=kwargs.get("device"))
        self.tokenizer = None
        config.eos = int(getattr(config.hf_config, "eos_token_id", -1) or -1)
        mgr = self.model_runner.compact_kv_manager
        guard = mgr.prefill_pages_guaranteed if (mgr.paged and config.prefill_chunk_size) else None
        self.scheduler = Scheduler(config, can_allocate=mgr.can_allocate, admission_need=mgr.admission_need,
                                   prefill_guard=guard)
        self.last_decode_tok_s = 0.0
        self.last_prefill_tok_s = 0.0
        # run-ahead decode (Config.decode_run_ahead): the step launched during the previous call,
        # as (sequences, read-back handle), and finished requests whose spans it may still be using
        self._ahead = None
        self._deferred_free: list[int] = []

    def _tokenizer(self):
        if self.tokenizer is None:
            from transformers import AutoTokenizer
            self.tokenizer = AutoTokenizer.from_pretrained(self.config.model, use_fast=True)
            if self.tokenizer.eos_token_id is not None:
                self.scheduler.eos = self.config.eos = self.tokenizer.eos_token_id
        return self.tokenizer

    def add_request(self, prompt: str | list[int], sampling_params: SamplingParams) -> Sequence:
        if isinstance(prompt, str):
            prompt = self._tokenizer().encode(prompt)
        if len(prompt) + sampling_params.max_tokens > self.config.max_model_len:
            raise ValueError(f"prompt ({len(prompt)}) + max_tokens ({sampling_params.max_tokens}) exceeds "
                             f"max_model_len={self.config.max_model_len}")
        seq = Sequence(prompt, sampling_params)
        self.scheduler.add(seq)
        return seq

    def _may_launch_next(self, seqs) -> bool:
        """Whether the step AFTER the one in flight can be launched before its tokens are known:
        same batch for certain (nobody reaches max_tokens, nothing waits to be prefilled, nobody has
        finished), greedy, graph captured, and -- paged layout -- a page certain for every span."""
        mgr = self.model_runner.compact_kv_manager
        return (not self.scheduler.waiting
                and all(not s.is_finished and s.num_completion_tokens + 1 < s.max_tokens for s in seqs)
                and self.model_runner.can_run_ahead(seqs)
                and mgr.decode_pages_guaranteed(len(seqs)))

    def _finish_decode(self, seqs, handle):
        """Second half of a run-ahead decode step: launch the following step from the tokens that
        are still on the device, then read this step's tokens and do the host bookkeeping."""
        runner = self.model_runner
        nxt = (seqs, runner.launch_decode(seqs, device_fed=True)) if self._may_launch_next(seqs) else None
        tokens = runner.resolve_decode(handle)
        # a request that ended on EOS one call ago is still part of a step launched before that was known
        kept = [(s, t) for s, t in zip(seqs, tokens) if not s.is_finished]
        self.scheduler.postprocess([s for s, _ in kept], [t for _, t in kept], False)
        done, self._deferred_free = self._deferred_free, []          # the step that used them has completed
        freed = self.scheduler.consume_freed_seq_ids()
        if nxt is not None:
            self._deferred_free = freed                              # the step in flight still reads their spans
        else:
            done += freed
        if done:
            runner.free_compact(done)
        self._ahead = nxt
        return [(s.seq_id, s.completion_token_ids) for s, _ in kept if s.is_finished], -len(kept)

    def step(self):
        if self._ahead is not None:
            seqs, handle = self._ahead
            self._ahead = None
            return self._finish_decode(seqs, handle)
        seqs, is_prefill = self.scheduler.schedule()
        if not seqs:                      # a partly prefilled request was sent back to free its pages
            self.model_runner.free_compact(self.scheduler.consume_freed_seq_ids())
            return [], 0
        num_tokens = sum(seq.num_scheduled_tokens for seq in seqs) if is_prefill else -len(seqs)
        if is_prefill:
            try:
                token_ids = self.model_runner.run(seqs, True)
            except RuntimeError as e:
                if "capacity exhausted" not in str(e):
                    raise
                # optimistic admission charged less than the prompts kept: give everything back and retry later
                self.model_runner.free_compact([seq.seq_id for seq in seqs])
                self.scheduler.requeue(seqs)
                return [], 0
            self.scheduler.prefill_succeeded()
        else:
            mgr = self.model_runner.compact_kv_manager
            while not mgr.decode_pages_guaranteed(len(seqs)):
                victim = self.scheduler.preempt_youngest(seqs)
                seqs.remove(victim)
                self.model_runner.free_compact([victim.seq_id])
            num_tokens = -len(seqs)
            if getattr(self.config, "decode_run_ahead", False) and self.model_runner.can_run_ahead(seqs):
                return self._finish_decode(seqs, self.model_runner.launch_decode(seqs, device_fed=False))
            token_ids = self.model_runner.run(seqs, False)
        self.scheduler.postprocess(seqs, token_ids, is_prefill)
        freed = self.scheduler.consume_freed_seq_ids()
        if freed:
            self.model_runner.free_compact(freed)
        outputs = [(seq.seq_id, seq.completion_token_ids) for seq in seqs if seq.is_finished]
        return outputs, num_tokens

    def is_finished(self) -> bool:
        # a run-ahead step still in flight has to be resolved (and its requests' spans released)
        return self.scheduler.is_finished() and self._ahead is None

    def generate(self, prompts, sampling_params, use_tqdm: bool = False) -> list[dict]:
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params] * len(prompts)
        order = [self.add_request(p, sp).seq_id for p, sp in zip(prompts, sampling_params)]
        outputs: dict[int, list[int]] = {}
        while not self.is_finished():
            t = perf_counter()
            finished, num_tokens = self.step()
            dt = max(perf_counter() - t, 1e-9)
            if num_tokens > 0:
                self.last_prefill_tok_s = num_tokens / dt
            else:
                self.last_decode_tok_s = -num_tokens / dt
            for seq_id, token_ids in finished:
                outputs[seq_id] = token_ids
        result = []
        for seq_id in order:
            ids = outputs[seq_id]
            text = self.tokenizer.decode(ids) if self.tokenizer is not None else ""
            result.append({"text": text, "token_ids": ids})
        return result

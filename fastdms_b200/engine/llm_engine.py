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

    def step(self):
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
            token_ids = self.model_runner.run(seqs, False)
        self.scheduler.postprocess(seqs, token_ids, is_prefill)
        freed = self.scheduler.consume_freed_seq_ids()
        if freed:
            self.model_runner.free_compact(freed)
        outputs = [(seq.seq_id, seq.completion_token_ids) for seq in seqs if seq.is_finished]
        return outputs, num_tokens

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

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

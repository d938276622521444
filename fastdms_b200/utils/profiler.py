"""CUDA-event phase timer.  The phase names used by the runner and the layers are the reference's
(`dms_decode_expire`, `prepare_decode_metadata`, `dms_rope_store`, `compact_decode_attn`,
`record_dms_decode_decisions`, `streaming_pack`, `dms_capture`, `model_forward_decode`), so that
reports built on them keep working.  Disabled (the default) it costs one attribute test."""
from __future__ import annotations

import time
from contextlib import contextmanager

import torch


class PhaseProfiler:
    def __init__(self) -> None:
        self.enabled = False
        self.totals_ms: dict[str, float] = {}
        self.counts: dict[str, int] = {}
        self._pending: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []

    def enable(self) -> None:
        self.enabled = True

    def disable(self) -> None:
        self.enabled = False

    def reset(self) -> None:
        self.totals_ms.clear()
        self.counts.clear()
        self._pending.clear()

    @contextmanager
    def cuda_phase(self, name: str):
        if not self.enabled or not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
            yield
            return
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        try:
            yield
        finally:
            end.record()
            self._pending.append((name, start, end))
            self.counts[name] = self.counts.get(name, 0) + 1

    @contextmanager
    def wall_phase(self, name: str):
        if not self.enabled:
            yield
            return
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.totals_ms[name] = self.totals_ms.get(name, 0.0) + (time.perf_counter() - t0) * 1e3
            self.counts[name] = self.counts.get(name, 0) + 1

    def summarize(self) -> dict:
        if self._pending:
            torch.cuda.synchronize()
            for name, start, end in self._pending:
                self.totals_ms[name] = self.totals_ms.get(name, 0.0) + start.elapsed_time(end)
            self._pending.clear()
        return {"totals_ms": dict(self.totals_ms), "counts": dict(self.counts)}


_PROFILER = PhaseProfiler()


def get_profiler() -> PhaseProfiler:
    return _PROFILER

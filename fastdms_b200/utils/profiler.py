"""Phase timing for the runner and the layers.

The public surface is the reference's (`fastdms/utils/profiler.py`: `get_profiler()`, `enable`,
`disable`, `reset`, `cuda_phase`, `wall_phase`, `summarize`) and so are the phase names used at the
call sites (`dms_decode_expire`, `dms_rope_store`, `compact_decode_attn`, `streaming_pack`,
`dms_capture`, `model_forward_decode`, ...), so reports built on them keep working.  The
implementation is this package's own: device phases are pairs of CUDA events collected in a flat
list and resolved in one pass when a summary is asked for; nothing is recorded while a CUDA graph is
being captured (events inside a capture would become graph nodes), and a disabled profiler costs one
attribute test per phase.
"""
from __future__ import annotations

import time
from collections import defaultdict

import torch


class _Phase:
    """Context manager of one timed region; `device=True` brackets it with CUDA events."""

    __slots__ = ("owner", "name", "device", "t0", "events")

    def __init__(self, owner: "PhaseProfiler", name: str, device: bool):
        self.owner, self.name, self.device = owner, name, device
        self.t0 = 0.0
        self.events = None

    def __enter__(self):
        if not self.owner.enabled:
            return self
        if not self.device:
            self.t0 = time.perf_counter()
        elif torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
            self.events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self.events[0].record()
        return self

    def __exit__(self, *exc):
        if not self.owner.enabled:
            return False
        if not self.device:
            self.owner._add(self.name, (time.perf_counter() - self.t0) * 1e3)
        elif self.events is not None:
            self.events[1].record()
            self.owner._unresolved.append((self.name, *self.events))
            self.owner.counts[self.name] += 1
        return False


class PhaseProfiler:
    def __init__(self) -> None:
        self.enabled = False
        self.totals_ms: dict[str, float] = defaultdict(float)
        self.counts: dict[str, int] = defaultdict(int)
        self._unresolved: list[tuple] = []          # (name, start event, end event) of device phases

    def enable(self) -> None:
        self.enabled = True

    def disable(self) -> None:
        self.enabled = False

    def reset(self) -> None:
        self.totals_ms.clear()
        self.counts.clear()
        self._unresolved.clear()

    def _add(self, name: str, ms: float) -> None:
        self.totals_ms[name] += ms
        self.counts[name] += 1

    def cuda_phase(self, name: str) -> _Phase:
        """Times the device work enqueued inside the `with` block (CUDA events on the current stream)."""
        return _Phase(self, name, device=True)

    def wall_phase(self, name: str) -> _Phase:
        """Times the host wall clock of the `with` block."""
        return _Phase(self, name, device=False)

    def summarize(self) -> dict:
        """{"totals_ms": {phase: ms}, "counts": {phase: n}}; waits for the device if phases are pending."""
        if self._unresolved:
            torch.cuda.synchronize()
            for name, start, end in self._unresolved:
                self.totals_ms[name] += start.elapsed_time(end)
            self._unresolved.clear()
        return {"totals_ms": dict(self.totals_ms), "counts": dict(self.counts)}


_PROFILER = PhaseProfiler()


def get_profiler() -> PhaseProfiler:
    return _PROFILER

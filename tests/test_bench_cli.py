"""Host-side checks of the benchmark entry points that need no GPU: the model block of `bench.py` drives
`benchmarks.bench_model.run` with that module's own parser, so every option `run` reads has a value."""
from __future__ import annotations

import ast
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def test_model_block_arguments_cover_what_run_reads():
    from benchmarks.bench_model import build_parser
    ns = build_parser().parse_args(["--shape", "llama-1b", "--concurrency", "8", "--prompt-len", "8192",
                                    "--decode-steps", "64", "--window", "256", "--run-ahead"])
    src = (ROOT / "benchmarks" / "bench_model.py").read_text()
    read = {n.attr for n in ast.walk(ast.parse(src))
            if isinstance(n, ast.Attribute) and isinstance(n.value, ast.Name) and n.value.id == "args"}
    missing = sorted(a for a in read if not hasattr(ns, a))
    assert not missing, f"bench_model.run reads options its parser does not define: {missing}"
    assert ns.run_ahead and ns.shard == 1 and ns.tp == 1
    # bench.py builds its arguments with the same parser
    assert "build_parser().parse_args(" in (ROOT / "bench.py").read_text()


def test_cached_scratch_is_not_an_inference_tensor():
    """The per-device status word is created on first use, possibly by the engine under inference mode; code
    outside inference mode clears it in place, which an inference tensor would refuse."""
    import torch
    from fastdms_b200 import _lib
    saved = dict(_lib._status_words)
    _lib._status_words.clear()
    try:
        with torch.inference_mode():
            w = _lib.status_word(torch.device("cpu", 0))
        assert not w.is_inference()
        w.zero_()
    finally:
        _lib._status_words.clear()
        _lib._status_words.update(saved)

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


def test_reference_arm_prints_one_line_with_the_shared_config():
    """`bench.py --impl reference` (the CPU arm) writes exactly one JSON line to standard output and names the
    workload with the same `config` object as the GPU arm."""
    import json
    import subprocess
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-400:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    import bench
    assert d["impl"] == "reference" and d["config"] == bench.workload_config(1)
    assert d["unit"] == "tok/s" and d["higher_is_better"] is True and d["value"] > 0
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["cpu_baseline"]["kind"] == "port"
    src = (ROOT / "bench.py").read_text()
    assert src.count('"config": workload_config(') == 2          # both arms

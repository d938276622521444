"""The two ways of switching application code over:

* `install_as_fastdms()`: imports written against the reference (`from fastdms.layers... import`) resolve
  to this package (CPU test: importing needs no GPU).
* the operator rebinding recipe applied to an unmodified install of the reference (under
  `baseline/_ref`, skipped when absent): the reference's own modules then run this library's kernels,
  called exactly as the reference calls them (positional arguments, span layout, no scales), and are
  checked against the reference's own torch oracles `compact_decode_attention_ref` and the
  extract -> rotary_emb -> indexed-store chain."""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def test_install_as_fastdms_resolves_reference_style_imports():
    saved = {k: v for k, v in sys.modules.items() if k == "fastdms" or k.startswith("fastdms.")}
    for k in saved:
        del sys.modules[k]
    try:
        import fastdms_b200
        fastdms_b200.install_as_fastdms()
        from fastdms.engine.compact_kv import CompactKVManager                      # noqa: F401
        from fastdms.engine.dms import build_dms_live_mask, extract_dms_eviction_decisions   # noqa: F401
        from fastdms.layers.compact_attention import (compact_decode_attention,    # noqa: F401
                                                      fused_dms_rope_store_compact_decode, store_compact_kvcache)
        from fastdms.utils.context import get_context, set_context                  # noqa: F401
        import fastdms
        assert fastdms.SamplingParams is fastdms_b200.SamplingParams
        assert compact_decode_attention.__module__ == "fastdms_b200.layers.compact_attention"
        with pytest.raises(RuntimeError):                                            # never shadows silently
            sys.modules["fastdms"] = importlib.import_module("types")
            fastdms_b200.install_as_fastdms()
    finally:
        for k in [k for k in sys.modules if k == "fastdms" or k.startswith("fastdms.")]:
            del sys.modules[k]
        sys.modules.update(saved)


@pytest.mark.gpu
@pytest.mark.skipif(not (REF / "fastdms").is_dir(), reason="the reference is not installed under baseline/_ref")
def test_reference_modules_run_the_library_after_rebinding():
    saved = {k: v for k, v in sys.modules.items() if k == "fastdms" or k.startswith("fastdms.")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, str(REF))
    try:
        import fastdms.engine.dms as ref_dms
        import fastdms.layers.compact_attention as ref_ops
        from fastdms.layers.rotary_embedding import apply_rotary_emb, get_rope
        import fastdms_b200.engine.dms as b200_dms
        import fastdms_b200.layers.compact_attention as b200_ops
        assert ref_ops.__file__.startswith(str(REF))
        oracle_attention = ref_ops.compact_decode_attention_ref
        oracle_extract = ref_dms.extract_dms_eviction_decisions                     # its CPU branch is plain torch
        # ---- the recipe ----
        for name in ("compact_decode_attention", "fused_dms_rope_store_compact_decode", "store_compact_kvcache",
                     "dms_expiry_one_layer", "dms_expiry_incremental_one_layer"):
            setattr(ref_ops, name, getattr(b200_ops, name))
        ref_dms.extract_dms_eviction_decisions = b200_dms.extract_dms_eviction_decisions
        # ---- the reference's decode attention call (benchmarks/bench_compact_decode.py:141-154) ----
        dev = torch.device("cuda:0")
        g = torch.Generator(device=dev).manual_seed(3)
        B, Hq, Hk, D, live = 4, 32, 8, 64, 333
        q = torch.randn((B, Hq, D), device=dev, generator=g).to(torch.bfloat16)
        ck = torch.randn((B * Hk * live, D), device=dev, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn)
        cv = torch.randn((B * Hk * live, D), device=dev, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn)
        base = torch.arange(B * Hk, device=dev, dtype=torch.int32).reshape(B, Hk) * live
        lens = torch.randint(1, live + 1, (B, Hk), device=dev, generator=g, dtype=torch.int32)
        out = ref_ops.compact_decode_attention(q, ck, cv, base, lens, None, live, 128, True)
        want = oracle_attention(q, ck, cv, base, lens)
        assert float((out.float() - want.float()).abs().max()) < 2e-2
        # ---- the reference's fused decode preprocess call (models/llama.py:138-154) against its torch chain ----
        rope = get_rope(D, D, 4096, 500000.0, None)
        cache = rope.cos_sin_cache.to(dev)
        k = torch.randn((B, Hk, D), device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn((B, Hk, D), device=dev, generator=g).to(torch.bfloat16)
        positions = torch.tensor([5, 100, 0, 777], device=dev)
        slot = (base + lens).clamp(max=B * Hk * live - 1).to(torch.int32)
        slot[:, :] = base + torch.minimum(lens, torch.full_like(lens, live - 1))
        q_in = q.clone()
        q_in[:, 0::Hq // Hk, -1] = torch.linspace(-0.2, 0.3, B * Hk, device=dev).view(B, Hk).to(torch.bfloat16)
        ck2, cv2 = ck.clone(), cv.clone()
        ev = torch.empty((B, Hk), dtype=torch.bool, device=dev)
        q_fused = q_in.clone()
        ref_ops.fused_dms_rope_store_compact_decode(q_fused, k.clone(), v, cache, ck2, cv2, slot, ev, positions,
                                                    num_kv_heads=Hk, alpha_scale=100.0, alpha_offset=5.0)
        q_cpu, ev_cpu = oracle_extract(q_in.cpu().clone(), num_kv_heads=Hk, num_qo_heads=Hq, head_dim=D,
                                       alpha_scale=100.0, alpha_offset=5.0, inplace=True)
        cos, sin = rope.cos_sin_cache.cpu()[positions.cpu()].chunk(2, dim=-1)
        q_rot, k_rot = apply_rotary_emb(q_cpu, cos, sin), apply_rotary_emb(k.cpu(), cos, sin)
        assert torch.equal(ev.cpu(), ev_cpu)
        assert torch.equal(q_fused.cpu().view(torch.int16), q_rot.view(torch.int16)), "rotated q differs from the reference chain"
        flat = slot.reshape(-1).long().cpu()
        want_k = k_rot.reshape(-1, D).to(torch.float8_e4m3fn).view(torch.uint8)
        want_v = v.cpu().reshape(-1, D).to(torch.float8_e4m3fn).view(torch.uint8)
        assert torch.equal(ck2.cpu().view(torch.uint8)[flat], want_k) and torch.equal(cv2.cpu().view(torch.uint8)[flat], want_v)
        from fastdms_b200 import _lib
        assert _lib.read_device_status(dev) == 0
    finally:
        sys.path.remove(str(REF))
        for k in [k for k in sys.modules if k == "fastdms" or k.startswith("fastdms.")]:
            del sys.modules[k]
        sys.modules.update(saved)

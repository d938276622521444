"""Generate the op-level golden fixtures by running the reference implementation on CPU.

Run in a container that has the reference checkout (it is imported, never copied):

    PYTHONDONTWRITEBYTECODE=1 TORCHDYNAMO_DISABLE=1 FASTDMS_DMS_EXPIRY_TRITON=0 \
    FASTDMS_DMS_FUSED_DECODE_PREPROCESS=0 \
    python tests/golden/make_golden_ops.py --reference /path/to/FastDMS

Every fixture stores the INPUTS next to the reference OUTPUTS, so the tests never depend
on reproducing a random stream.  FP8 tensors are stored as their raw bytes (uint8).

Reference functions exercised (paths inside the reference project):
  fastdms/engine/dms.py                 extract_dms_eviction_decisions (CPU branch), build_dms_live_mask
  fastdms/engine/compact_kv.py          CompactKVManager.{allocate, streaming_pack_layer,
                                        apply_dms_evictions (python path), prepare_decode_metadata,
                                        record_appended_dms_decisions, free}, pack_compact_kv
  fastdms/layers/compact_attention.py   compact_decode_attention_ref
  fastdms/layers/rotary_embedding.py    get_rope, apply_rotary_emb
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _u8(t: torch.Tensor) -> np.ndarray:
    """Raw bytes of an fp8 tensor / plain numpy of anything else."""
    if t.dtype in (torch.float8_e4m3fn,):
        return t.contiguous().view(torch.uint8).numpy().copy()
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().copy()
    return t.contiguous().numpy().copy()


def gen_extract(ref, out: dict) -> None:
    from fastdms.engine.dms import extract_dms_eviction_decisions

    g = torch.Generator().manual_seed(101)
    # fp32 case with values exactly at / one ulp around the 0.05 threshold
    q = torch.randn(11, 32, 64, generator=g, dtype=torch.float32)
    q[:, 0::4, -1] = torch.linspace(-0.1, 0.2, q.shape[0]).view(-1, 1)
    q[0, 0::4, -1] = 0.05
    q[1, 0::4, -1] = torch.nextafter(torch.tensor(0.05), torch.tensor(1.0))
    q[2, 0::4, -1] = torch.nextafter(torch.tensor(0.05), torch.tensor(0.0))
    q_out, ev = extract_dms_eviction_decisions(
        q.clone(), num_kv_heads=8, num_qo_heads=32, head_dim=64,
        alpha_scale=100.0, alpha_offset=5.0, inplace=True)
    out["extract_f32_q"] = _u8(q)
    out["extract_f32_q_out"] = _u8(q_out)
    out["extract_f32_evict"] = _u8(ev)
    # bf16 case (the dtype the engine feeds), odd token count, group size 2
    qb = (torch.randn(37, 4, 64, generator=g) * 0.2).to(torch.bfloat16)
    qb_out, evb = extract_dms_eviction_decisions(
        qb.clone(), num_kv_heads=2, num_qo_heads=4, head_dim=64,
        alpha_scale=100.0, alpha_offset=5.0, inplace=True)
    out["extract_bf16_q"] = _u8(qb)
    out["extract_bf16_q_out"] = _u8(qb_out)
    out["extract_bf16_evict"] = _u8(evb)
    # negative alpha_scale takes the other comparison branch
    qn = torch.randn(9, 8, 32, generator=g, dtype=torch.float32) * 0.1
    qn_out, evn = extract_dms_eviction_decisions(
        qn.clone(), num_kv_heads=4, num_qo_heads=8, head_dim=32,
        alpha_scale=-50.0, alpha_offset=1.0, inplace=True)
    out["extract_neg_q"] = _u8(qn)
    out["extract_neg_q_out"] = _u8(qn_out)
    out["extract_neg_evict"] = _u8(evn)


def gen_live_mask(ref, out: dict) -> None:
    from fastdms.engine.dms import build_dms_live_mask

    g = torch.Generator().manual_seed(102)
    ev = torch.rand(2, 3, 40, generator=g) > 0.4
    out["livemask_evict"] = _u8(ev)
    out["livemask_cur39_w8"] = _u8(build_dms_live_mask(ev, current_position=39, window_size=8))
    out["livemask_cur50_w0"] = _u8(build_dms_live_mask(ev, current_position=50, window_size=0))
    pos = torch.arange(40) * 2
    out["livemask_positions"] = _u8(pos)
    out["livemask_cur60_w16_pos"] = _u8(
        build_dms_live_mask(ev, current_position=60, window_size=16, positions=pos))


def gen_pack_known_answer(ref, out: dict) -> None:
    from fastdms.engine.compact_kv import pack_compact_kv
    from fastdms.layers.compact_attention import compact_decode_attention_ref

    k = torch.arange(1 * 5 * 2 * 4, dtype=torch.float32).reshape(1, 5, 2, 4)
    v = k + 100
    live_mask = torch.tensor([[[True, False, True, False, True], [False, True, True, False, False]]])
    ck, cv, meta = pack_compact_kv(k, v, live_mask)
    out["packka_k"] = _u8(k)
    out["packka_v"] = _u8(v)
    out["packka_live_mask"] = _u8(live_mask)
    out["packka_compact_k"] = _u8(ck)
    out["packka_compact_v"] = _u8(cv)
    out["packka_base"] = _u8(meta.base_offsets)
    out["packka_live"] = _u8(meta.live_counts)
    out["packka_positions"] = _u8(meta.token_positions)
    q = torch.ones((1, 4, 4), dtype=torch.float32)
    o = compact_decode_attention_ref(q, ck, cv, meta.base_offsets, meta.live_counts, scale=1.0)
    out["packka_q"] = _u8(q)
    out["packka_attn_out"] = _u8(o)


def gen_attention_ref(ref, out: dict) -> None:
    from fastdms.layers.compact_attention import compact_decode_attention_ref

    g = torch.Generator().manual_seed(103)
    # the reference's own split-K test shape (fp32, D=16, 2 seqs, 8 q heads, 2 kv heads)
    q = torch.randn((2, 8, 16), generator=g)
    ck = torch.randn((96, 16), generator=g)
    cv = torch.randn((96, 16), generator=g)
    base = torch.tensor([[0, 24], [48, 72]], dtype=torch.int32)
    live = torch.tensor([[17, 13], [19, 11]], dtype=torch.int32)
    o = compact_decode_attention_ref(q, ck, cv, base, live)
    for name, t in (("q", q), ("k", ck), ("v", cv), ("base", base), ("live", live), ("out", o)):
        out[f"attn_f32d16_{name}"] = _u8(t)
    # fp8 K/V, bf16 q, D=64, 3 seqs x 2 kv heads x group 4, ragged lengths incl. 1 and non-multiples of 16
    q = torch.randn((3, 8, 64), generator=g).to(torch.bfloat16)
    lens = [[1, 37], [300, 16], [255, 129]]
    base_l, cur = [], 0
    for row in lens:
        b = []
        for n in row:
            b.append(cur)
            cur += n + 5
        base_l.append(b)
    ck = torch.randn((cur, 64), generator=g).to(torch.float8_e4m3fn)
    cv = torch.randn((cur, 64), generator=g).to(torch.float8_e4m3fn)
    base = torch.tensor(base_l, dtype=torch.int32)
    live = torch.tensor(lens, dtype=torch.int32)
    o = compact_decode_attention_ref(q, ck, cv, base, live)
    for name, t in (("q", q), ("k", ck), ("v", cv), ("base", base), ("live", live), ("out", o)):
        out[f"attn_fp8d64_{name}"] = _u8(t)
    # fp8 K/V, bf16 q, D=128 (Qwen3-8B head size), group 4
    q = torch.randn((2, 8, 128), generator=g).to(torch.bfloat16)
    lens = [[200, 77], [513, 64]]
    base_l, cur = [], 0
    for row in lens:
        b = []
        for n in row:
            b.append(cur)
            cur += n
        base_l.append(b)
    ck = torch.randn((cur, 128), generator=g).to(torch.float8_e4m3fn)
    cv = torch.randn((cur, 128), generator=g).to(torch.float8_e4m3fn)
    base = torch.tensor(base_l, dtype=torch.int32)
    live = torch.tensor(lens, dtype=torch.int32)
    o = compact_decode_attention_ref(q, ck, cv, base, live, scale=0.11)
    for name, t in (("q", q), ("k", ck), ("v", cv), ("base", base), ("live", live), ("out", o)):
        out[f"attn_fp8d128_{name}"] = _u8(t)


def gen_rope_store(ref, out: dict) -> None:
    """extract -> apply_rotary_emb -> indexed store: the reference chain the fused decode
    kernel is tested against (reference tests/test_compact_kv.py, fused store test)."""
    from fastdms.engine.dms import extract_dms_eviction_decisions
    from fastdms.layers.rotary_embedding import RotaryEmbedding, apply_rotary_emb

    g = torch.Generator().manual_seed(104)
    for tag, dtype, cdtype, (B, Hk, G, D), theta in (
        ("f32d32", torch.float32, torch.float32, (3, 2, 2, 32), 10000.0),
        ("bf16d64", torch.bfloat16, torch.float8_e4m3fn, (5, 2, 4, 64), 500000.0),
        ("bf16d128", torch.bfloat16, torch.float8_e4m3fn, (4, 2, 4, 128), 1000000.0),
    ):
        Hq = Hk * G
        q = torch.randn((B, Hq, D), generator=g).to(dtype)
        k = torch.randn((B, Hk, D), generator=g).to(dtype)
        v = torch.randn((B, Hk, D), generator=g).to(dtype)
        dec = torch.tensor([0.01, 0.06, 0.05, 0.08, 0.10, -0.01, 0.049, 0.051, 0.2, -0.3])
        q[:, 0::G, -1] = dec[: B * Hk].view(B, Hk).to(dtype)
        positions = torch.tensor([0, 3, 7, 100, 8191][:B], dtype=torch.int64)
        slots = (torch.arange(B * Hk, dtype=torch.int32) * 3).view(B, Hk)
        rope = RotaryEmbedding(D, D, 8192 + 8, theta)
        cache = rope.cos_sin_cache
        q_ref, ev = extract_dms_eviction_decisions(
            q.clone(), num_kv_heads=Hk, num_qo_heads=Hq, head_dim=D,
            alpha_scale=100.0, alpha_offset=5.0, inplace=True)
        cos, sin = cache[positions].chunk(2, dim=-1)
        q_rot = apply_rotary_emb(q_ref, cos, sin)
        k_rot = apply_rotary_emb(k.clone(), cos, sin)
        ck = torch.zeros((B * Hk * 3, D), dtype=cdtype)
        cv = torch.zeros_like(ck)
        flat = slots.view(-1).long()
        ck[flat] = k_rot.reshape(B * Hk, D).to(cdtype)
        cv[flat] = v.reshape(B * Hk, D).to(cdtype)
        out[f"ropestore_{tag}_q"] = _u8(q)
        out[f"ropestore_{tag}_k"] = _u8(k)
        out[f"ropestore_{tag}_v"] = _u8(v)
        out[f"ropestore_{tag}_positions"] = _u8(positions)
        out[f"ropestore_{tag}_slots"] = _u8(slots)
        out[f"ropestore_{tag}_theta"] = np.array([theta], dtype=np.float64)
        out[f"ropestore_{tag}_cos_sin_rows"] = _u8(cache[positions, 0])
        out[f"ropestore_{tag}_q_out"] = _u8(q_rot)
        out[f"ropestore_{tag}_k_out"] = _u8(k_rot)
        out[f"ropestore_{tag}_evict"] = _u8(ev)
        out[f"ropestore_{tag}_compact_k"] = _u8(ck)
        out[f"ropestore_{tag}_compact_v"] = _u8(cv)


def _mk_manager(**kw):
    from fastdms.engine.compact_kv import CompactKVManager

    return CompactKVManager(**kw)


def gen_manager_known_answers(ref, out: dict) -> None:
    from fastdms.engine.sequence import Sequence
    from fastdms.sampling_params import SamplingParams

    m = _mk_manager(num_layers=2, num_kv_heads=2, capacity_tokens=32, max_model_len=16, device="cpu")
    seq = Sequence([10, 11], SamplingParams(max_tokens=4))
    st = m.allocate(seq)
    for l in range(2):
        m._allocate_layer_ranges_for_seq(st, l, torch.full((2,), 2, dtype=torch.int32))
    m.mark_all_heads_live(seq.seq_id, 2)
    base, live, slot, cap = m.prepare_decode_metadata([seq])
    out["meta_base"] = _u8(base)
    out["meta_live"] = _u8(live)
    out["meta_slot"] = _u8(slot)
    out["meta_cap"] = np.array([cap])
    out["meta_free_after"] = np.array(m.free_ranges_per_layer[0])
    m.free(seq.seq_id)
    out["meta_free_end"] = np.array(m.free_ranges_per_layer[0])

    m = _mk_manager(num_layers=2, num_kv_heads=2, capacity_tokens=32, max_model_len=16, device="cpu",
                    layer_major_metadata=True, max_active_seqs=2)
    s0 = Sequence([10, 11], SamplingParams(max_tokens=4))
    s1 = Sequence([20, 21], SamplingParams(max_tokens=4))
    st0, st1 = m.allocate(s0), m.allocate(s1)
    st0.live_counts.fill_(1)
    st1.live_counts.fill_(1)
    ev = torch.tensor([[[True, False], [False, True]], [[False, False], [True, True]]])
    stats = m.record_appended_dms_decisions([s0, s1], [10, 20], ev)
    out["record_evict_in"] = _u8(ev)
    out["record_positions"] = _u8(m.layer_major_token_positions)
    out["record_evict_mask"] = _u8(m.layer_major_evict_mask)
    out["record_stats"] = np.array([stats["eviction_decisions_true"], stats["eviction_decisions_total"]])


def gen_streaming_pack(ref, out: dict) -> None:
    """Prefill pack through the manager's CPU path, two ragged sequences in one batch."""
    from fastdms.engine.sequence import Sequence
    from fastdms.sampling_params import SamplingParams

    g = torch.Generator().manual_seed(105)
    for tag, cdtype in (("f32", torch.float32), ("fp8", torch.float8_e4m3fn)):
        L, Hk, D, W = 2, 3, 16, 31
        lens = [37, 541]
        m = _mk_manager(num_layers=L, num_kv_heads=Hk, capacity_tokens=4096, max_model_len=1024,
                        device="cpu", head_dim=D, compact_dtype=cdtype, per_layer_storage=True)
        seqs = [Sequence(list(range(n)), SamplingParams(max_tokens=8)) for n in lens]
        for s in seqs:
            m.allocate(s)
        cu = torch.tensor([0, lens[0], lens[0] + lens[1]], dtype=torch.int32)
        T = int(cu[-1])
        for l in range(L):
            k = torch.randn((T, Hk, D), generator=g).to(torch.bfloat16)
            v = torch.randn((T, Hk, D), generator=g).to(torch.bfloat16)
            ev = torch.rand((T, Hk), generator=g) > 0.5
            m.streaming_pack_layer(layer_id=l, k=k, v=v, evict_mask=ev, cu_seqlens_q=cu,
                                   seq_ids=[s.seq_id for s in seqs], window_size=W)
            out[f"pack_{tag}_k_l{l}"] = _u8(k)
            out[f"pack_{tag}_v_l{l}"] = _u8(v)
            out[f"pack_{tag}_evict_l{l}"] = _u8(ev)
            out[f"pack_{tag}_compact_k_l{l}"] = _u8(m.compact_k_per_layer[l])
            out[f"pack_{tag}_compact_v_l{l}"] = _u8(m.compact_v_per_layer[l])
        out[f"pack_{tag}_cu"] = _u8(cu)
        out[f"pack_{tag}_window"] = np.array([W])
        out[f"pack_{tag}_max_tokens"] = np.array([8])
        for i, s in enumerate(seqs):
            st = m.seq_states[s.seq_id]
            out[f"pack_{tag}_base_s{i}"] = _u8(st.base_offsets)
            out[f"pack_{tag}_cap_s{i}"] = _u8(st.range_capacity)
            out[f"pack_{tag}_live_s{i}"] = _u8(st.live_counts)
            out[f"pack_{tag}_pos_s{i}"] = _u8(st.token_positions)
            out[f"pack_{tag}_ev_s{i}"] = _u8(st.evict_mask)


def _expiry_case(cdtype, layer_major):
    """CPU twin of the reference's CUDA expiry fixture (capacity 9, window 3)."""
    from fastdms.engine.sequence import Sequence
    from fastdms.sampling_params import SamplingParams

    m = _mk_manager(num_layers=2, num_kv_heads=2, capacity_tokens=128, max_model_len=9, device="cpu",
                    head_dim=4, compact_dtype=cdtype, per_layer_storage=True,
                    layer_major_metadata=layer_major, max_active_seqs=2)
    seq = Sequence([1, 2, 3, 4], SamplingParams(max_tokens=5))
    st = m.allocate(seq)
    for l in range(2):
        m._ensure_layer_storage(l, 64)
        m.compact_k_per_layer[l].zero_()
        m.compact_v_per_layer[l].zero_()
        lc = torch.tensor([6, 7], dtype=torch.int32)
        m._allocate_layer_ranges_for_seq(st, l, lc)
        st.live_counts[l].copy_(lc)
        for h in range(2):
            n = int(lc[h])
            pos = torch.arange(n, dtype=torch.int32)
            st.token_positions[l, h, :n] = pos
            st.evict_mask[l, h, :n] = pos % 2 == 0
            b = int(st.base_offsets[l, h])
            vals = (l * 10.0 + h + torch.arange(n, dtype=torch.float32) * 0.01).view(n, 1).expand(n, 4)
            m.compact_k_per_layer[l][b:b + n] = vals.to(cdtype)
            m.compact_v_per_layer[l][b:b + n] = (vals + 0.5).to(cdtype)
    return m, [seq]


def _append_expiry_token(m, position, cdtype):
    for st in m.seq_states.values():
        for l in range(m.num_layers):
            for h in range(m.num_kv_heads):
                idx = int(st.live_counts[l, h])
                b = int(st.base_offsets[l, h])
                st.token_positions[l, h, idx] = position
                st.evict_mask[l, h, idx] = (position % 2) == 0
                val = torch.full((m.head_dim,), l * 10.0 + h + position * 0.01).to(cdtype)
                m.compact_k_per_layer[l][b + idx] = val
                m.compact_v_per_layer[l][b + idx] = (val.float() + 0.5).to(cdtype)
                st.live_counts[l, h] += 1


def _snap(m, out, prefix):
    st = next(iter(m.seq_states.values()))
    out[f"{prefix}_live"] = _u8(st.live_counts.clone())
    out[f"{prefix}_pos"] = _u8(st.token_positions.clone())
    out[f"{prefix}_ev"] = _u8(st.evict_mask.clone())
    out[f"{prefix}_base"] = _u8(st.base_offsets.clone())
    for l in range(m.num_layers):
        out[f"{prefix}_k_l{l}"] = _u8(m.compact_k_per_layer[l].clone())
        out[f"{prefix}_v_l{l}"] = _u8(m.compact_v_per_layer[l].clone())


def gen_expiry(ref, out: dict) -> None:
    for tag, cdtype in (("f32", torch.float32), ("fp8", torch.float8_e4m3fn)):
        m, seqs = _expiry_case(cdtype, False)
        _snap(m, out, f"expiry_{tag}_s0")
        stats = m.apply_dms_evictions(seqs, [8], window_size=3)
        out[f"expiry_{tag}_stats8"] = np.array([stats[k] for k in (
            "evicted_tokens", "live_tokens_before_min", "live_tokens_before_max",
            "live_tokens_after_min", "live_tokens_after_max")])
        _snap(m, out, f"expiry_{tag}_s1")
        _append_expiry_token(m, 8, cdtype)
        m.apply_dms_evictions(seqs, [9], window_size=3)
        _snap(m, out, f"expiry_{tag}_s2")
        _append_expiry_token(m, 9, cdtype)
        m.apply_dms_evictions(seqs, [10], window_size=3)
        _snap(m, out, f"expiry_{tag}_s3")


def gen_expiry_random(ref, out: dict) -> None:
    """Larger random multi-step expiry: 2 layers x 3 heads, one sequence, 12 decode steps with
    per-step exact expiry (python path), window 16, spans long enough to need several tiles."""
    from fastdms.engine.sequence import Sequence
    from fastdms.sampling_params import SamplingParams

    g = torch.Generator().manual_seed(106)
    L, Hk, D, W = 2, 3, 64, 16
    cdtype = torch.float8_e4m3fn
    T0, steps = 700, 12
    m = _mk_manager(num_layers=L, num_kv_heads=Hk, capacity_tokens=8192, max_model_len=1024, device="cpu",
                    head_dim=D, compact_dtype=cdtype, per_layer_storage=True)
    seq = Sequence(list(range(T0)), SamplingParams(max_tokens=steps + 1))
    m.allocate(seq)
    cu = torch.tensor([0, T0], dtype=torch.int32)
    for l in range(L):
        k = torch.randn((T0, Hk, D), generator=g).to(torch.bfloat16)
        v = torch.randn((T0, Hk, D), generator=g).to(torch.bfloat16)
        ev = torch.rand((T0, Hk), generator=g) > 0.3
        m.streaming_pack_layer(layer_id=l, k=k, v=v, evict_mask=ev, cu_seqlens_q=cu,
                               seq_ids=[seq.seq_id], window_size=W)
    st = m.seq_states[seq.seq_id]
    _snap(m, out, "expiryrand_s0")
    app_k = torch.randn((steps, L, Hk, D), generator=g).to(cdtype)
    app_v = torch.randn((steps, L, Hk, D), generator=g).to(cdtype)
    app_ev = torch.rand((steps, L, Hk), generator=g) > 0.3
    out["expiryrand_app_k"] = _u8(app_k)
    out["expiryrand_app_v"] = _u8(app_v)
    out["expiryrand_app_ev"] = _u8(app_ev)
    out["expiryrand_T0"] = np.array([T0])
    out["expiryrand_window"] = np.array([W])
    for s in range(steps):
        cur = T0 + s  # position of the token being fed this step
        seq.append_token(0) if s > 0 else None
        m.apply_dms_evictions([seq], [cur], window_size=W)
        base, live, slot, _ = m.prepare_decode_metadata([seq])
        for l in range(L):
            for h in range(Hk):
                sl = int(slot[l, 0, h])
                m.compact_k_per_layer[l][sl] = app_k[s, l, h]
                m.compact_v_per_layer[l][sl] = app_v[s, l, h]
        m.record_appended_dms_decisions([seq], [cur], app_ev[s].view(L, 1, Hk))
        out[f"expiryrand_slot_{s}"] = _u8(slot.clone())
        out[f"expiryrand_live_{s}"] = _u8(st.live_counts.clone())
    _snap(m, out, "expiryrand_end")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a FastDMS checkout (the directory that holds the fastdms package)")
    args = ap.parse_args()
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    os.environ.setdefault("FASTDMS_DMS_EXPIRY_TRITON", "0")
    os.environ.setdefault("FASTDMS_DMS_FUSED_DECODE_PREPROCESS", "0")
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    torch.set_num_threads(1)
    out: dict[str, np.ndarray] = {}
    for fn in (gen_extract, gen_live_mask, gen_pack_known_answer, gen_attention_ref, gen_rope_store,
               gen_manager_known_answers, gen_streaming_pack, gen_expiry, gen_expiry_random):
        fn(args.reference, out)
        print(f"{fn.__name__}: {len(out)} arrays so far")
    path = HERE / "ops_golden.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size / 1024:.1f} KiB, {len(out)} arrays)")


if __name__ == "__main__":
    main()

"""GPU parity tests of CompactKVManager (prefill pack, expiry, decode metadata, decision recording,
allocation) against vectors produced by the reference's CPU manager and against the numpy oracle.
All comparisons are bit-exact."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import compact_dms as O
from oracle.dtypes import bf16_bits_to_f32, decode_e4m3, encode_e4m3

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _status_clean(dev):
    from fastdms_b200 import _lib
    _lib.read_device_status(dev)
    yield
    assert _lib.read_device_status(dev) == 0, "a kernel raised a device status bit"


def _mgr(dev, **kw):
    from fastdms_b200.engine.compact_kv import CompactKVManager
    return CompactKVManager(device=dev, **kw)


def _seq(tokens, max_tokens):
    from fastdms_b200.engine.sequence import Sequence
    from fastdms_b200.sampling_params import SamplingParams
    return Sequence(list(tokens), SamplingParams(max_tokens=max_tokens))


def t_bf16(a, dev):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(dev)


def n_u8(t):
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def test_allocate_free_and_metadata_known_answers(ops_golden, dev):
    """reference tests/test_compact_kv.py:162-249."""
    z = ops_golden
    m = _mgr(dev, num_layers=3, num_kv_heads=2, capacity_tokens=64, max_model_len=32, head_dim=16,
             compact_dtype=torch.float32, max_active_seqs=4)
    seq = _seq([1, 2, 3], 5)
    st = m.allocate(seq)
    assert st.max_capacity_per_lh == 8 and st.base_offsets.tolist() == [[-1, -1]] * 3
    assert st.range_capacity.tolist() == [[0, 0]] * 3 and st.live_counts.sum().item() == 0
    assert m.free_tokens == 3 * 64 and m.allocate(seq) is st
    m.free(seq.seq_id)
    assert m.free_tokens == 3 * 64 and m.free_ranges_per_layer == [[(0, 64)]] * 3

    m = _mgr(dev, num_layers=2, num_kv_heads=2, capacity_tokens=32, max_model_len=16, head_dim=16,
             compact_dtype=torch.float32, max_active_seqs=2)
    seq = _seq([10, 11], 4)
    st = m.allocate(seq)
    for l in range(2):
        m._allocate_layer_ranges_for_seq(st, l, torch.full((2,), 2, dtype=torch.int32))
    m.mark_all_heads_live(seq.seq_id, 2)
    base, live, slot, cap = m.prepare_decode_metadata([seq])
    assert base.tolist() == z["meta_base"].tolist() == [[[0, 6]], [[0, 6]]]
    assert slot.tolist() == z["meta_slot"].tolist() == [[[2, 8]], [[2, 8]]]
    assert live.tolist() == z["meta_live"].tolist() and st.live_counts.tolist() == [[3, 3], [3, 3]]
    assert cap == st.max_capacity_per_lh == int(z["meta_cap"][0])
    assert m.last_cu_live.tolist() == [[0, 3, 6], [0, 3, 6]]
    assert [list(r) for r in m.free_ranges_per_layer[0]] == z["meta_free_after"].tolist()
    m.free(seq.seq_id)
    assert [list(r) for r in m.free_ranges_per_layer[0]] == z["meta_free_end"].tolist()
    with pytest.raises(RuntimeError):
        m.prepare_decode_metadata([seq])

    # active-slot reuse (reference :189-222) and slot exhaustion
    s0, s1 = _seq([1, 2, 3], 4), _seq([4, 5], 4)
    a0, a1 = m.allocate(s0), m.allocate(s1)
    assert (a0.active_slot, a1.active_slot) == (0, 1)
    a0.live_counts[0, 1] = 7
    assert m.layer_major_live_counts[0, 0, 1].item() == 7
    with pytest.raises(RuntimeError):
        m.allocate(_seq([9], 4))
    m.free(s0.seq_id)
    a2 = m.allocate(_seq([6], 4))
    assert a2.active_slot == 0 and a2.live_counts.sum().item() == 0 and a2.token_positions.max().item() == -1


def test_record_decisions_known_answer(ops_golden, dev):
    """reference tests/test_compact_kv.py:252-320."""
    z = ops_golden
    m = _mgr(dev, num_layers=2, num_kv_heads=2, capacity_tokens=32, max_model_len=16, head_dim=16,
             compact_dtype=torch.float32, max_active_seqs=2)
    s0, s1 = _seq([10, 11], 4), _seq([20, 21], 4)
    m.allocate(s0).live_counts.fill_(1)
    m.allocate(s1).live_counts.fill_(1)
    ev = torch.from_numpy(z["record_evict_in"]).to(dev)
    stats = m.record_appended_dms_decisions([s0, s1], [10, 20], ev)
    assert stats == {"eviction_decisions_true": 4, "eviction_decisions_total": 8}
    assert np.array_equal(m.layer_major_token_positions.cpu().numpy(), z["record_positions"])
    assert np.array_equal(m.layer_major_evict_mask.cpu().numpy(), z["record_evict_mask"])
    # tensor positions and dict-of-layers decisions give the same result
    m.layer_major_token_positions.fill_(-1)
    m.layer_major_evict_mask.zero_()
    m.record_appended_dms_decisions([s0, s1], torch.tensor([10, 20], device=dev), {0: ev[0], 1: ev[1]})
    assert np.array_equal(m.layer_major_token_positions.cpu().numpy(), z["record_positions"])
    with pytest.raises(RuntimeError):
        m.record_appended_dms_decisions([s0, s1], [10, 20], ev[:1])


@pytest.mark.parametrize("tag,pool", [("f32", torch.float32), ("fp8", torch.float8_e4m3fn)])
def test_streaming_pack_golden(ops_golden, dev, tag, pool):
    """Two ragged prompts (37 and 541 tokens, window 31): spans, positions, evict bits, live counts
    and pool bytes equal the reference's CPU pack; the first-fit bases are identical too."""
    z = ops_golden
    g = lambda n: z[f"pack_{tag}_{n}"]
    cu = g("cu")
    L, Hk, D = 2, 3, 16
    m = _mgr(dev, num_layers=L, num_kv_heads=Hk, capacity_tokens=4096, max_model_len=1024, head_dim=D,
             compact_dtype=pool, max_active_seqs=4)
    seqs = [_seq(range(int(cu[i + 1] - cu[i])), int(g("max_tokens")[0])) for i in range(2)]
    for s in seqs:
        m.allocate(s)
    for l in range(L):
        m.streaming_pack_layer(layer_id=l, k=t_bf16(g(f"k_l{l}"), dev), v=t_bf16(g(f"v_l{l}"), dev),
                               evict_mask=torch.from_numpy(g(f"evict_l{l}")).to(dev),
                               cu_seqlens_q=torch.from_numpy(cu), seq_ids=[s.seq_id for s in seqs],
                               window_size=int(g("window")[0]))
    for i, s in enumerate(seqs):
        st = m.seq_states[s.seq_id]
        assert np.array_equal(st.base_offsets.cpu().numpy(), g(f"base_s{i}"))
        assert np.array_equal(st.range_capacity.cpu().numpy(), g(f"cap_s{i}"))
        assert np.array_equal(st.live_counts.cpu().numpy(), g(f"live_s{i}"))
        assert np.array_equal(st.token_positions.cpu().numpy(), g(f"pos_s{i}"))
        assert np.array_equal(st.evict_mask.cpu().numpy(), g(f"ev_s{i}"))
        for l in range(L):
            ck, cv = n_u8(m.compact_k_per_layer[l]), n_u8(m.compact_v_per_layer[l])
            rk = g(f"compact_k_l{l}").view(np.uint8).reshape(-1, ck.shape[1])
            rv = g(f"compact_v_l{l}").view(np.uint8).reshape(-1, ck.shape[1])
            for h in range(Hk):
                b, n = int(g(f"base_s{i}")[l, h]), int(g(f"live_s{i}")[l, h])
                assert np.array_equal(ck[b:b + n], rk[b:b + n]) and np.array_equal(cv[b:b + n], rv[b:b + n])
    for s in seqs:
        m.free(s.seq_id)
    assert m.free_ranges_per_layer == [[(0, 4096)]] * L


def _load_expiry_state(m, seq, z, prefix, pool, dev):
    st = m.seq_states[seq.seq_id]
    live, base = z[f"{prefix}_live"], z[f"{prefix}_base"]
    L, Hk = live.shape
    for l in range(L):
        st.base_offsets[l].copy_(torch.from_numpy(base[l]))
        for h in range(Hk):
            m.free_ranges_per_layer[l] = []          # spans are placed by hand; the allocator is bypassed
    st.live_counts.copy_(torch.from_numpy(live))
    st.token_positions.copy_(torch.from_numpy(z[f"{prefix}_pos"]))
    st.evict_mask.copy_(torch.from_numpy(z[f"{prefix}_ev"]))
    for l in range(L):
        k = torch.from_numpy(z[f"{prefix}_k_l{l}"].copy())
        v = torch.from_numpy(z[f"{prefix}_v_l{l}"].copy())
        if pool == torch.float8_e4m3fn:
            k, v = k.view(torch.float8_e4m3fn), v.view(torch.float8_e4m3fn)
        n = min(k.shape[0], m.capacity_tokens)   # the reference grows its pools in 256-row steps
        m.compact_k_per_layer[l][:n].copy_(k[:n])
        m.compact_v_per_layer[l][:n].copy_(v[:n])
    return st


def _check_expiry_state(m, st, z, prefix, rows_only=False):
    assert np.array_equal(st.live_counts.cpu().numpy(), z[f"{prefix}_live"])
    assert np.array_equal(st.token_positions.cpu().numpy(), z[f"{prefix}_pos"])
    assert np.array_equal(st.evict_mask.cpu().numpy(), z[f"{prefix}_ev"])
    L, Hk = z[f"{prefix}_live"].shape
    for l in range(L):
        ck, cv = n_u8(m.compact_k_per_layer[l]), n_u8(m.compact_v_per_layer[l])
        rk = z[f"{prefix}_k_l{l}"].view(np.uint8).reshape(-1, ck.shape[1])
        rv = z[f"{prefix}_v_l{l}"].view(np.uint8).reshape(-1, ck.shape[1])
        for h in range(Hk):
            b, n = int(z[f"{prefix}_base"][l, h]), int(z[f"{prefix}_live"][l, h])
            assert np.array_equal(ck[b:b + n], rk[b:b + n]) and np.array_equal(cv[b:b + n], rv[b:b + n])


@pytest.mark.parametrize("tag,pool", [("f32", torch.float32), ("fp8", torch.float8_e4m3fn)])
def test_expiry_capacity9_window3(ops_golden, dev, tag, pool):
    """The reference's expiry fixture (tests/test_compact_kv.py:1283-1329): non power-of-two capacity
    9, window 3, positions 8 -> 10; float32 rows of 16 bytes and FP8 rows of 4 bytes."""
    z = ops_golden
    m = _mgr(dev, num_layers=2, num_kv_heads=2, capacity_tokens=128, max_model_len=9, head_dim=4,
             compact_dtype=pool, max_active_seqs=2)
    seq = _seq([1, 2, 3, 4], 5)
    m.allocate(seq)
    st = _load_expiry_state(m, seq, z, f"expiry_{tag}_s0", pool, dev)

    def append(p):
        live = st.live_counts.cpu().numpy()
        for l in range(2):
            for h in range(2):
                i, b = int(live[l, h]), int(st.base_offsets[l, h])
                st.token_positions[l, h, i] = p
                st.evict_mask[l, h, i] = p % 2 == 0
                val = torch.full((4,), l * 10.0 + h + p * 0.01).to(pool)
                m.compact_k_per_layer[l][b + i] = val.to(dev)
                m.compact_v_per_layer[l][b + i] = (val.float() + 0.5).to(pool).to(dev)
                st.live_counts[l, h] += 1

    stats = m.apply_dms_evictions([seq], [8], window_size=3)
    assert [stats[k] for k in ("evicted_tokens", "live_tokens_before_min", "live_tokens_before_max",
                               "live_tokens_after_min", "live_tokens_after_max")] == z[f"expiry_{tag}_stats8"].tolist()
    _check_expiry_state(m, st, z, f"expiry_{tag}_s1")
    append(8)
    m.apply_dms_evictions([seq], [9], window_size=3)
    _check_expiry_state(m, st, z, f"expiry_{tag}_s2")
    append(9)
    m.apply_dms_evictions([seq], [10], window_size=3, incremental=True)      # steady-state variant
    _check_expiry_state(m, st, z, f"expiry_{tag}_s3")


def test_expiry_one_layer_functions(ops_golden, dev):
    """The per-layer operator entry points (reference compact_attention.py:861-965)."""
    from fastdms_b200.layers.compact_attention import dms_expiry_incremental_one_layer, dms_expiry_one_layer
    z = ops_golden
    for fn, cur, src, dst in ((dms_expiry_one_layer, 8, "s0", "s1"),):
        for l in range(2):
            pos = torch.from_numpy(z[f"expiry_f32_{src}_pos"][l][None].copy()).to(dev)
            ev = torch.from_numpy(z[f"expiry_f32_{src}_ev"][l][None].copy()).to(dev)
            live = torch.from_numpy(z[f"expiry_f32_{src}_live"][l][None].copy()).to(dev)
            base = torch.from_numpy(z[f"expiry_f32_{src}_base"][l][None].copy()).to(dev)
            ck = torch.from_numpy(z[f"expiry_f32_{src}_k_l{l}"].copy()).to(dev)
            cv = torch.from_numpy(z[f"expiry_f32_{src}_v_l{l}"].copy()).to(dev)
            fn(positions_per_lh=pos, evict_per_lh=ev, live_counts=live, base_offsets=base, compact_k=ck,
               compact_v=cv, current_positions=torch.tensor([cur], device=dev), window_size=3)
            assert np.array_equal(pos[0].cpu().numpy(), z[f"expiry_f32_{dst}_pos"][l])
            assert np.array_equal(ev[0].cpu().numpy(), z[f"expiry_f32_{dst}_ev"][l])
            assert np.array_equal(live[0].cpu().numpy(), z[f"expiry_f32_{dst}_live"][l])
            for h in range(2):
                b, n = int(base[0, h]), int(live[0, h])
                assert np.array_equal(ck[b:b + n].cpu().numpy(), z[f"expiry_f32_{dst}_k_l{l}"][b:b + n])
    # incremental drops only the first expired slot even when two qualify
    pos = torch.tensor([[[0, 1, 2, 3, 4, 5, -1, -1]]], dtype=torch.int32, device=dev)
    ev = torch.tensor([[[1, 1, 0, 1, 0, 0, 0, 0]]], dtype=torch.bool, device=dev)
    live = torch.tensor([[6]], dtype=torch.int32, device=dev)
    base = torch.tensor([[2]], dtype=torch.int32, device=dev)
    ck = torch.arange(16 * 4, dtype=torch.float32, device=dev).view(16, 4).clone()
    cv = ck + 100
    k0 = ck.clone()
    dms_expiry_incremental_one_layer(positions_per_lh=pos, evict_per_lh=ev, live_counts=live, base_offsets=base,
                                     compact_k=ck, compact_v=cv, current_positions=torch.tensor([10], device=dev),
                                     window_size=3)
    assert pos[0, 0].tolist() == [1, 2, 3, 4, 5, -1, -1, -1] and ev[0, 0].tolist() == [True, False, True] + [False] * 5
    assert live.item() == 5 and torch.equal(ck[2:7], k0[3:8]) and torch.equal(ck[:2], k0[:2])


@pytest.mark.parametrize("paged", [False, True])
def test_expiry_random_multistep(ops_golden, dev, paged):
    """700-token prompt packed by the reference, then 12 decode steps of
    expire -> metadata -> append -> record; spans need several 256-slot tiles.  The paged layout
    must give the same logical contents as the contiguous one."""
    z = ops_golden
    L, Hk, D = 2, 3, 64
    W, T0 = int(z["expiryrand_window"][0]), int(z["expiryrand_T0"][0])
    steps = z["expiryrand_app_k"].shape[0]
    m = _mgr(dev, num_layers=L, num_kv_heads=Hk, capacity_tokens=8192, max_model_len=1024, head_dim=D,
             compact_dtype=torch.float8_e4m3fn, max_active_seqs=2, paged=paged)
    seq = _seq(range(T0), steps + 1)
    m.allocate(seq)
    st = m.seq_states[seq.seq_id]
    live0, base0 = z["expiryrand_s0_live"], z["expiryrand_s0_base"]
    if not paged:
        _load_expiry_state(m, seq, z, "expiryrand_s0", torch.float8_e4m3fn, dev)
    else:
        # re-home the reference spans into pages popped from the GPU free stack
        from fastdms_b200 import _lib
        st.live_counts.copy_(torch.from_numpy(live0))
        st.token_positions.copy_(torch.from_numpy(z["expiryrand_s0_pos"]))
        st.evict_mask.copy_(torch.from_numpy(z["expiryrand_s0_ev"]))
        slot_t = torch.tensor([st.active_slot], dtype=torch.int32, device=dev)
        for l in range(L):
            need = torch.from_numpy(live0[l][None].copy()).to(dev)
            bt = m.block_tables[l]
            _lib.check(_lib.lib().fdms_alloc_pages(
                need.data_ptr(), bt.data_ptr(), bt.stride(0), bt.stride(1), m.max_pages, slot_t.data_ptr(),
                m.free_pages[l].data_ptr(), m.free_page_counts[l:].data_ptr(), 1, Hk,
                _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev)))
            btc = m.block_tables[l, st.active_slot].cpu().numpy()
            rk, rv = z[f"expiryrand_s0_k_l{l}"], z[f"expiryrand_s0_v_l{l}"]
            for h in range(Hk):
                n, b = int(live0[l, h]), int(base0[l, h])
                rows = torch.from_numpy(O.gather_span(np.arange(m.capacity_tokens), 0, n, btc[h])).to(dev)
                m.compact_k_per_layer[l].view(torch.uint8)[rows] = torch.from_numpy(rk[b:b + n].copy()).to(dev)
                m.compact_v_per_layer[l].view(torch.uint8)[rows] = torch.from_numpy(rv[b:b + n].copy()).to(dev)
        free0 = m.free_page_counts.clone()
    app_k = torch.from_numpy(z["expiryrand_app_k"].copy()).view(torch.float8_e4m3fn).to(dev)
    app_v = torch.from_numpy(z["expiryrand_app_v"].copy()).view(torch.float8_e4m3fn).to(dev)
    app_ev = torch.from_numpy(z["expiryrand_app_ev"]).to(dev)
    for s in range(steps):
        cur = T0 + s
        m.apply_dms_evictions([seq], [cur], window_size=W, sync_stats=False)
        base, live, slot, _ = m.prepare_decode_metadata([seq])
        if not paged:
            assert np.array_equal(slot.cpu().numpy(), z[f"expiryrand_slot_{s}"])
        for l in range(L):
            idx = slot[l, 0].long()
            m.compact_k_per_layer[l][idx] = app_k[s, l]
            m.compact_v_per_layer[l][idx] = app_v[s, l]
        m.record_appended_dms_decisions([seq], [cur], app_ev[s].view(L, 1, Hk), sync_stats=False)
        assert np.array_equal(st.live_counts.cpu().numpy(), z[f"expiryrand_live_{s}"])
    assert np.array_equal(st.token_positions.cpu().numpy(), z["expiryrand_end_pos"])
    assert np.array_equal(st.evict_mask.cpu().numpy(), z["expiryrand_end_ev"])
    end_live, end_base = z["expiryrand_end_live"], z["expiryrand_end_base"]
    for l in range(L):
        ck, cv = n_u8(m.compact_k_per_layer[l]), n_u8(m.compact_v_per_layer[l])
        btc = m.block_tables[l, st.active_slot].cpu().numpy() if paged else None
        for h in range(Hk):
            b, n = int(end_base[l, h]), int(end_live[l, h])
            rows = O.gather_span(np.arange(m.capacity_tokens), b, n, None if btc is None else btc[h])
            assert np.array_equal(ck[rows], z[f"expiryrand_end_k_l{l}"][b:b + n])
            assert np.array_equal(cv[rows], z[f"expiryrand_end_v_l{l}"][b:b + n])
            if paged:   # exactly the pages that hold live rows stay in the table
                assert int((btc[h] >= 0).sum()) == -(-n // 16)
    if paged:
        pages_now = sum(-(-int(n) // 16) for n in end_live[0])
        assert int(m.free_page_counts[0]) == m.pages_per_layer - pages_now
        m.free(seq.seq_id)
        assert m.free_page_counts.tolist() == [m.pages_per_layer] * L
        assert sorted(m.free_pages[0].tolist()) == list(range(m.pages_per_layer))       # no page lost or duplicated
    else:
        m.free(seq.seq_id)


def test_windowed_cadence_matches_oracle_with_same_cadence(dev):
    """expiry_interval = W (the reference's default cadence for batched decode): evict-marked tokens
    survive until the next multiple of W; compare live counts with the oracle driven the same way."""
    rng = np.random.default_rng(3)
    L, Hk, D, W, T0, steps = 1, 2, 64, 8, 40, 20
    m = _mgr(dev, num_layers=L, num_kv_heads=Hk, capacity_tokens=1024, max_model_len=128, head_dim=D,
             compact_dtype=torch.float8_e4m3fn, max_active_seqs=1, dms_expiry_interval=W)
    seq = _seq(range(T0), steps + 1)
    m.allocate(seq)
    ev0 = rng.random((T0, Hk)) > 0.4
    k = torch.randn((T0, Hk, D), device=dev, dtype=torch.bfloat16)
    m.streaming_pack_layer(layer_id=0, k=k, v=k, evict_mask=torch.from_numpy(ev0).to(dev),
                           cu_seqlens_q=torch.tensor([0, T0], dtype=torch.int32), seq_ids=[seq.seq_id], window_size=W)
    st = m.seq_states[seq.seq_id]
    o_pos, o_ev = st.token_positions.cpu().numpy().copy(), st.evict_mask.cpu().numpy().copy()
    o_live, o_base = st.live_counts.cpu().numpy().copy(), st.base_offsets.cpu().numpy().copy()
    o_k = np.zeros((1024, D), np.uint8)
    for s in range(steps):
        cur = T0 + s
        m.apply_dms_evictions([seq], [cur], window_size=W, sync_stats=False)
        if s == 0 or cur % W == 0:
            O.expire_layer(o_pos[0][None], o_ev[0][None], o_live[0][None], o_base[0][None], o_k, o_k.copy(), [cur], W)
        m.prepare_decode_metadata([seq])
        O.prepare_decode_metadata(o_base, o_live)
        e = rng.random((L, 1, Hk)) > 0.4
        m.record_appended_dms_decisions([seq], [cur], torch.from_numpy(e).to(dev), sync_stats=False)
        O.record_decisions(o_pos[:, None], o_ev[:, None], o_live[:, None], e, [cur])
        assert np.array_equal(st.live_counts.cpu().numpy(), o_live)
    assert np.array_equal(st.token_positions.cpu().numpy(), o_pos) and np.array_equal(st.evict_mask.cpu().numpy(), o_ev)


@pytest.mark.parametrize("steady", [True, False])
@pytest.mark.parametrize("paged,interval,T0", [(False, 1, 600), (True, 1, 600), (False, 8, 600), (True, 8, 600),
                                               (True, 1, 2600), (False, 8, 2600)])
def test_row_index_expiry_keeps_logical_contents(dev, paged, interval, T0, steady):
    """Expiry with a row index (K/V rows stay dense but are not shifted): positions, evict bits and
    compact lengths follow the oracle exactly, and the K/V rows read THROUGH the index are the
    oracle's rows in logical order.  interval 8 drops several tokens per call (holes and movers in
    the same call); spans of 600 tokens are handled from registers, spans of 2600 by the tiled path.
    With interval 1 every call after the first finds the span exact through the previous position and
    inspects one slot only (`steady`); with the record wiped before each call it takes the general path:
    both must give the oracle's state."""
    rng = np.random.default_rng(11 + interval + int(paged) + T0)
    L, Hk, D, W, steps = 1, 3, 64, 8, 40
    C = 1024 if T0 < 1000 else 4096
    m = _mgr(dev, num_layers=L, num_kv_heads=Hk, capacity_tokens=4 * C, max_model_len=C, head_dim=D,
             compact_dtype=torch.float8_e4m3fn, max_active_seqs=2, paged=paged, dms_expiry_interval=interval,
             row_indirection=True)
    seq = _seq(range(T0), steps + 1)
    m.allocate(seq)
    ev0 = rng.random((T0, Hk)) > (0.5 if T0 < 1000 else 0.1)       # long spans keep most tokens
    k = torch.randn((T0, Hk, D), device=dev, dtype=torch.bfloat16)
    v = torch.randn((T0, Hk, D), device=dev, dtype=torch.bfloat16)
    m.streaming_pack_layer(layer_id=0, k=k, v=v, evict_mask=torch.from_numpy(ev0).to(dev),
                           cu_seqlens_q=torch.tensor([0, T0], dtype=torch.int32), seq_ids=[seq.seq_id], window_size=W)
    st = m.seq_states[seq.seq_id]
    ri = m.layer_major_row_index[:, st.active_slot]                        # [L, Hk, C]

    def logical_rows(pool_u8, h, n):
        base = 0 if paged else int(st.base_offsets[0, h])
        bt = m.block_tables[0, st.active_slot, h].cpu().numpy() if paged else None
        phys = O.gather_span(np.arange(m.capacity_tokens), base, n, bt)   # physical row r -> pool row
        idx = ri[0, h, :n].cpu().numpy()
        assert sorted(idx.tolist()) == list(range(n)), "the index of the live slots is a permutation of [0, live)"
        return pool_u8[phys[idx]]

    # oracle state: contiguous spans of its own, contents = the packed rows
    o_pos, o_ev = st.token_positions.cpu().numpy().copy(), st.evict_mask.cpu().numpy().copy()
    o_live = st.live_counts.cpu().numpy().copy()
    o_base = (np.arange(Hk, dtype=np.int32) * C)[None]
    o_k, o_v = np.zeros((Hk * C, D), np.uint8), np.zeros((Hk * C, D), np.uint8)
    ck, cv = n_u8(m.compact_k_per_layer[0]), n_u8(m.compact_v_per_layer[0])
    for h in range(Hk):
        n = int(o_live[0, h])
        o_k[o_base[0, h]:o_base[0, h] + n] = logical_rows(ck, h, n)
        o_v[o_base[0, h]:o_base[0, h] + n] = logical_rows(cv, h, n)
    exact = m.layer_major_exact_through[:, st.active_slot]
    assert (exact == -1).all(), "a pack leaves the record unknown"
    for s in range(steps):
        cur = T0 + s
        if not steady:
            m.layer_major_exact_through.fill_(-1)
        m.apply_dms_evictions([seq], [cur], window_size=W, sync_stats=False)
        if interval == 1 or s == 0 or cur % interval == 0:
            O.expire_layer(o_pos[0][None], o_ev[0][None], o_live[0][None], o_base[0][None], o_k, o_v, [cur], W)
            assert (exact == cur).all(), "an all-slots call records the position it made the span exact for"
        assert np.array_equal(st.live_counts.cpu().numpy(), o_live), f"compact lengths differ at step {s}"
        _, _, slot, _ = m.prepare_decode_metadata([seq])
        _, _, o_slot = O.prepare_decode_metadata(o_base[None], o_live[None])
        newk = rng.integers(0, 120, size=(Hk, D), dtype=np.uint8)
        newv = rng.integers(0, 120, size=(Hk, D), dtype=np.uint8)
        idx = slot[0, 0].long()
        m.compact_k_per_layer[0].view(torch.uint8)[idx] = torch.from_numpy(newk).to(dev)
        m.compact_v_per_layer[0].view(torch.uint8)[idx] = torch.from_numpy(newv).to(dev)
        o_k[o_slot[0, 0]], o_v[o_slot[0, 0]] = newk, newv
        e = rng.random((L, 1, Hk)) > 0.5
        m.record_appended_dms_decisions([seq], [cur], torch.from_numpy(e).to(dev), sync_stats=False)
        O.record_decisions(o_pos[:, None], o_ev[:, None], o_live[:, None], e, [cur])
        if s % 7 == 0 or s == steps - 1:
            ck, cv = n_u8(m.compact_k_per_layer[0]), n_u8(m.compact_v_per_layer[0])
            for h in range(Hk):
                n, b = int(o_live[0, h]), int(o_base[0, h])
                assert np.array_equal(logical_rows(ck, h, n), o_k[b:b + n]), f"K rows differ at step {s}, head {h}"
                assert np.array_equal(logical_rows(cv, h, n), o_v[b:b + n]), f"V rows differ at step {s}, head {h}"
                assert np.array_equal(ri[0, h, n:].cpu().numpy(), np.arange(n, ri.shape[-1])), "index tail is the identity"
    assert np.array_equal(st.token_positions.cpu().numpy(), o_pos) and np.array_equal(st.evict_mask.cpu().numpy(), o_ev)
    from fastdms_b200 import _lib
    assert _lib.read_device_status(dev) == 0
    m.free(seq.seq_id)
    if paged:
        assert m.free_page_counts.tolist() == [m.pages_per_layer] * L


def test_capacity_errors(dev):
    m = _mgr(dev, num_layers=1, num_kv_heads=2, capacity_tokens=64, max_model_len=64, head_dim=16,
             compact_dtype=torch.float32, max_active_seqs=2)
    seq = _seq(range(40), 8)
    m.allocate(seq)
    k = torch.zeros((40, 2, 16), device=dev)
    ev = torch.zeros((40, 2), dtype=torch.bool, device=dev)
    with pytest.raises(RuntimeError, match="capacity exhausted"):
        m.streaming_pack_layer(layer_id=0, k=k, v=k, evict_mask=ev, cu_seqlens_q=torch.tensor([0, 40], dtype=torch.int32),
                               seq_ids=[seq.seq_id], window_size=4)
    assert m.free_ranges_per_layer == [[(0, 64)]]      # the failed reservation was rolled back
    with pytest.raises(RuntimeError, match="no compact KV allocation"):
        m.streaming_pack_layer(layer_id=0, k=k, v=k, evict_mask=ev, cu_seqlens_q=torch.tensor([0, 40], dtype=torch.int32),
                               seq_ids=[12345], window_size=4)
    with pytest.raises(ValueError):
        _mgr(dev, num_layers=1, num_kv_heads=2, capacity_tokens=0, max_model_len=64, head_dim=16, compact_dtype=torch.float32)


@pytest.mark.parametrize("paged,gap", [(False, False), (True, False), (True, True), (False, True)])
def test_hot_path_step_equals_the_manual_kernel_sequence(dev, paged, gap):
    """DecodeHotPath (one graph replay: expiry, metadata, a fused store+attention launch per layer,
    recording with position advance) against the same step issued kernel by kernel with the separate
    store and attention launches on a twin manager: identical outputs and metadata after every step,
    through step_device, step_host and step_host_block.  With `gap` an earlier sequence has been freed,
    so the active slots are not contiguous (0, 2, 3) and the batch's block tables are a gathered copy
    that has to follow the pages the 30 steps add (every span crosses a 16-row page boundary)."""
    from fastdms_b200.engine.hot_path import DecodeHotPath
    from fastdms_b200.layers.compact_attention import compact_decode_attention, fused_dms_rope_store_compact_decode
    L, B, Hk, G, D, W = 2, 3, 2, 4, 64, 16
    Hq = Hk * G
    T0 = [70, 50, 300, 141] if gap else [70, 300, 141]
    rng = np.random.default_rng(5 + int(paged))
    gen = torch.Generator(device=dev).manual_seed(9)
    half = D // 2
    inv = 1.0 / (500000.0 ** (np.arange(half, dtype=np.float32) / half))
    ang = np.arange(1024, dtype=np.float32)[:, None] * inv[None, :]
    cache = torch.from_numpy(np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)).to(dev).unsqueeze(1)
    scales = (torch.tensor([[0.02, 0.03], [0.04, 0.01]], device=dev), torch.tensor([[0.025, 0.015], [0.02, 0.03]], device=dev))

    def build():
        m = _mgr(dev, num_layers=L, num_kv_heads=Hk, capacity_tokens=4096, max_model_len=512, head_dim=D,
                 compact_dtype=torch.float8_e4m3fn, max_active_seqs=4, paged=paged, row_indirection=True,
                 k_scale=scales[0], v_scale=scales[1])
        seqs = [_seq(range(t), 64) for t in T0]
        for s in seqs:
            m.allocate(s)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(T0)]), dtype=torch.int32)
        return m, seqs, cu

    mA, seqsA, cu = build()
    mB, seqsB, _ = build()
    for l in range(L):
        k = torch.randn((sum(T0), Hk, D), device=dev, generator=gen).to(torch.bfloat16)
        v = torch.randn((sum(T0), Hk, D), device=dev, generator=gen).to(torch.bfloat16)
        ev = torch.from_numpy(rng.random((sum(T0), Hk)) < 0.7).to(dev)
        for m, seqs in ((mA, seqsA), (mB, seqsB)):
            m.streaming_pack_layer(layer_id=l, k=k, v=v, evict_mask=ev, cu_seqlens_q=cu, seq_ids=[s.seq_id for s in seqs],
                                   window_size=W)
    if gap:
        for m, seqs in ((mA, seqsA), (mB, seqsB)):
            m.free(seqs.pop(1).seq_id)
        T0 = [T0[0]] + T0[2:]
        assert mA._contiguous_active_slot_start(mA._states(seqsA)) is None
    hp = DecodeHotPath(mA, seqsA, num_q_heads=Hq, window_size=W, alpha_scale=100.0, alpha_offset=5.0, cos_sin_cache=cache)
    assert hp.fuse_store and hp.launches_per_step == 2 + L + 1
    pos0 = torch.tensor(T0, dtype=torch.int64)
    hp.set_positions(pos0)
    slotsB = mB._slots_tensor(mB._states(seqsB))
    posB = pos0.to(dev)
    base, live, slot = (torch.zeros((L, B, Hk), device=dev, dtype=torch.int32) for _ in range(3))
    evB = torch.zeros((L, B, Hk), device=dev, dtype=torch.bool)
    outB = torch.zeros((L, B, Hq, D), device=dev, dtype=torch.bfloat16)
    host_block = None

    def manual_step(q, k, v):
        mB.expire_device(slotsB, posB, window_size=W)
        mB.decode_metadata_device(slotsB, base, live, slot)
        btB = mB.decode_block_tables(seqsB)        # after the metadata launch: it may have added pages
        for l in range(L):
            ks, vs = mB.layer_scales(l)
            ql = q[l].clone()
            fused_dms_rope_store_compact_decode(ql, k[l].clone(), v[l], cache, mB.compact_k_per_layer[l], mB.compact_v_per_layer[l],
                                                slot[l], evB[l], posB, num_kv_heads=Hk, alpha_scale=100.0, alpha_offset=5.0,
                                                store_transient_k=False, k_scale=ks, v_scale=vs)
            compact_decode_attention(ql, mB.compact_k_per_layer[l], mB.compact_v_per_layer[l], base[l], live[l],
                                     block_tables=None if btB is None else btB[l], k_scale=ks, v_scale=vs, out=outB[l])
        mB.record_device(slotsB, posB, evB)
        posB.add_(1)

    def new_inputs():
        q = torch.randn((L, B, Hq, D), device=dev, generator=gen).to(torch.bfloat16)
        q[:, :, 0::G, D - 1] = torch.where(torch.rand((L, B, Hk), device=dev, generator=gen) < 0.7, 1.0, -1.0).to(torch.bfloat16)
        k = torch.randn((L, B, Hk, D), device=dev, generator=gen).to(torch.bfloat16)
        v = torch.randn((L, B, Hk, D), device=dev, generator=gen).to(torch.bfloat16)
        return q, k, v

    q, k, v = new_inputs()
    hp.q.copy_(q); hp.k.copy_(k); hp.v.copy_(v)
    hp.capture()                              # the warm-up inside capture() is a real step
    manual_step(q, k, v)
    for step in range(30):
        q, k, v = new_inputs()
        if step < 20:
            hp.q.copy_(q); hp.k.copy_(k); hp.v.copy_(v)
            hp.step_device()
            got = hp.out
        elif step < 25:
            got = hp.step_host(q.cpu(), k.cpu(), v.cpu(), posB.cpu()).to(dev)
        else:
            if host_block is None:
                host_block = hp.new_host_block()
            blk, bq, bk, bv, bp = host_block
            bq.copy_(q.cpu()); bk.copy_(k.cpu()); bv.copy_(v.cpu()); bp.copy_(posB.cpu())
            got = hp.step_host_block(blk).to(dev)
        manual_step(q, k, v)
        assert torch.equal(got, outB), f"outputs differ at step {step}"
        assert torch.equal(hp.evict_all, evB) and torch.equal(hp.live, live) and torch.equal(hp.positions, posB)
    # pipelined host-driven steps: step n+1 is submitted before step n's outputs are waited for
    blocks = [hp.new_host_block() for _ in range(3)]
    pending = None                                   # (ticket, inputs) of the step not yet checked
    for step in range(30, 41):
        q, k, v = new_inputs()
        blk, bq, bk, bv, bp = blocks[step % 3]
        bq.copy_(q.cpu()); bk.copy_(k.cpu()); bv.copy_(v.cpu()); bp.copy_(posB.cpu() + (0 if pending is None else 1))
        ticket = hp.submit_host_block(blk)
        if pending is not None:
            manual_step(*pending[1])
            assert torch.equal(hp.wait_host_block(pending[0]).to(dev), outB), f"pipelined outputs differ at step {step - 1}"
        pending = (ticket, (q, k, v))
    manual_step(*pending[1])
    assert torch.equal(hp.wait_host_block(pending[0]).to(dev), outB), "pipelined outputs differ at the last step"
    with pytest.raises(ValueError):
        hp.wait_host_block(pending[0] - 2)
    torch.cuda.synchronize(dev)
    assert torch.equal(hp.evict_all, evB) and torch.equal(hp.live, live)
    for a, b in ((mA.layer_major_live_counts, mB.layer_major_live_counts), (mA.layer_major_token_positions, mB.layer_major_token_positions),
                 (mA.layer_major_evict_mask, mB.layer_major_evict_mask), (mA.layer_major_row_index, mB.layer_major_row_index)):
        assert torch.equal(a, b)
    if not paged:                              # identical first-fit spans: the pools are byte-identical too
        assert torch.equal(mA.compact_k.view(torch.uint8), mB.compact_k.view(torch.uint8))
        assert torch.equal(mA.compact_v.view(torch.uint8), mB.compact_v.view(torch.uint8))
    from fastdms_b200 import _lib
    assert _lib.read_device_status(dev) == 0

"""Pins the numpy oracle against vectors produced by the reference's own CPU code paths."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import compact_dms as O
from oracle.dtypes import (bf16_bits_to_f32, decode_e4m3, encode_e4m3, f32_to_bf16_bits, round_to)


def bf(a):
    return bf16_bits_to_f32(a.view(np.uint16))


def test_e4m3_roundtrip_and_rounding():
    codes = np.arange(256, dtype=np.uint8)
    vals = decode_e4m3(codes)
    finite = ~np.isnan(vals)
    back = encode_e4m3(vals[finite])
    # -0 and +0 keep their sign bit; every finite code is a fixed point
    assert np.array_equal(back, codes[finite])
    # ties to even, subnormals, saturation
    x = np.array([0.05, 448.0, 464.0, 465.0, 1e-3, 2.0 ** -10, 2.0 ** -10 * 1.0001, -500.0], np.float32)
    got = decode_e4m3(encode_e4m3(x))
    assert np.allclose(got, [0.05078125, 448, 448, 448, 2.0 ** -9, 0.0, 2.0 ** -9, -448.0])
    assert np.isnan(decode_e4m3(encode_e4m3(np.array([465.0], np.float32), saturate=False)))[0]


def test_e4m3_matches_torch_cpu_cast():
    torch = pytest.importorskip("torch")
    g = torch.Generator().manual_seed(5)
    x = torch.randn(20000, generator=g) * torch.exp(torch.randn(20000, generator=g) * 3)
    x = x.clamp(-448, 448)
    ref = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(encode_e4m3(x.numpy()), ref)
    y = torch.randn(5000, generator=g)
    assert np.array_equal(f32_to_bf16_bits(y.numpy()).view(np.int16), y.to(torch.bfloat16).view(torch.int16).numpy())


def test_extract_decisions(ops_golden):
    z = ops_golden
    q, ev = O.extract_decisions(z["extract_f32_q"], 8, 100.0, 5.0)
    assert np.array_equal(ev, z["extract_f32_evict"])
    assert np.array_equal(q, z["extract_f32_q_out"])
    # known answers around the threshold: exactly 0.05f is NOT evicted, +1 ulp is, -1 ulp is not
    assert not ev[0].any() and ev[1].all() and not ev[2].any()
    q, ev = O.extract_decisions(bf(z["extract_bf16_q"]), 2, 100.0, 5.0)
    assert np.array_equal(ev, z["extract_bf16_evict"])
    assert np.array_equal(q, bf(z["extract_bf16_q_out"]))
    q, ev = O.extract_decisions(z["extract_neg_q"], 4, -50.0, 1.0)
    assert np.array_equal(ev, z["extract_neg_evict"])
    assert np.array_equal(q, z["extract_neg_q_out"])


def test_live_mask(ops_golden):
    z = ops_golden
    ev = z["livemask_evict"]
    assert np.array_equal(O.live_mask(ev, 39, 8), z["livemask_cur39_w8"])
    assert np.array_equal(O.live_mask(ev, 50, 0), z["livemask_cur50_w0"])
    assert np.array_equal(O.live_mask(ev, 60, 16, z["livemask_positions"]), z["livemask_cur60_w16_pos"])


def test_pack_known_answer(ops_golden):
    z = ops_golden
    ck, cv, base, live, pos = O.pack_compact_kv(z["packka_k"], z["packka_v"], z["packka_live_mask"])
    assert base.tolist() == [[0, 3]] and live.tolist() == [[3, 2]] and pos.tolist() == [0, 2, 4, 1, 2]
    assert np.array_equal(ck, z["packka_compact_k"]) and np.array_equal(cv, z["packka_compact_v"])
    out = O.decode_attention(z["packka_q"], ck, cv, base, live, scale=1.0)
    assert np.allclose(out, z["packka_attn_out"], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("tag,pool,qd,scale", [("f32d16", "f32", "f32", None), ("fp8d64", "e4m3", "bf16", None),
                                               ("fp8d128", "e4m3", "bf16", 0.11)])
def test_attention_ref(ops_golden, tag, pool, qd, scale):
    z = ops_golden
    q = z[f"attn_{tag}_q"] if qd == "f32" else bf(z[f"attn_{tag}_q"])
    ref = z[f"attn_{tag}_out"] if qd == "f32" else bf(z[f"attn_{tag}_out"])
    out = O.decode_attention(q, z[f"attn_{tag}_k"], z[f"attn_{tag}_v"], z[f"attn_{tag}_base"],
                             z[f"attn_{tag}_live"], scale, pool_dtype=pool, out_dtype=qd)
    tol = 1e-5 if qd == "f32" else 8e-3   # bf16 output: one ulp at |x|<=1 is 2^-8
    assert np.allclose(out, ref, atol=tol, rtol=tol)


def test_attention_paged_equals_span(ops_golden):
    z = ops_golden
    q = bf(z["attn_fp8d64_q"])
    k, v, base, live = (z[f"attn_fp8d64_{n}"] for n in ("k", "v", "base", "live"))
    span = O.decode_attention(q, k, v, base, live, pool_dtype="e4m3")
    # re-home every span into randomly permuted 16-token pages
    rng = np.random.default_rng(3)
    B, Hk = live.shape
    maxp = int(-(-live.max() // 16))
    npages = int(sum(-(-int(n) // 16) for n in live.ravel()))
    perm = rng.permutation(npages + 7)
    kp = np.zeros(((npages + 7) * 16, k.shape[1]), np.uint8)
    vp = np.zeros_like(kp)
    bt = np.full((B, Hk, maxp), -1, np.int32)
    nxt = 0
    for b in range(B):
        for h in range(Hk):
            n = int(live[b, h])
            for p in range(-(-n // 16)):
                pg = int(perm[nxt]); nxt += 1
                bt[b, h, p] = pg
                rows = min(16, n - p * 16)
                s = int(base[b, h]) + p * 16
                kp[pg * 16: pg * 16 + rows] = k[s:s + rows]
                vp[pg * 16: pg * 16 + rows] = v[s:s + rows]
    paged = O.decode_attention(q, kp, vp, base, live, pool_dtype="e4m3", block_tables=bt)
    assert np.array_equal(span, paged)


@pytest.mark.parametrize("tag,act,pool", [("f32d32", "f32", "f32"), ("bf16d64", "bf16", "e4m3"),
                                          ("bf16d128", "bf16", "e4m3")])
def test_rope_store_decode(ops_golden, tag, act, pool):
    z = ops_golden
    g = lambda n: z[f"ropestore_{tag}_{n}"]
    cv = (lambda a: a) if act == "f32" else bf
    q, k, v = cv(g("q")), cv(g("k")), cv(g("v"))
    B, Hk, D = k.shape
    positions = g("positions")
    cache = np.zeros((int(positions.max()) + 1, D), np.float32)
    cache[positions] = g("cos_sin_rows")
    ck = np.zeros_like(g("compact_k"))
    cvv = np.zeros_like(g("compact_v"))
    q_rot, k_rot, ev = O.rope_store_decode(
        q, k, v, cache, ck, cvv, g("slots"), positions, num_kv_heads=Hk, alpha_scale=100.0,
        alpha_offset=5.0, act_dtype=act, pool_dtype=pool)
    assert np.array_equal(ev, g("evict"))
    assert np.array_equal(q_rot, cv(g("q_out")))
    assert np.array_equal(k_rot, cv(g("k_out")))
    assert np.array_equal(ck, g("compact_k"))
    assert np.array_equal(cvv, g("compact_v"))


def test_manager_known_answers(ops_golden):
    z = ops_golden
    # reference tests/test_compact_kv.py:225-249: two heads, live 2, max_tokens 4 -> spans of 6
    ff = O.FirstFit(32)
    sizes = O.span_sizes([2, 2], 4, 6)
    bases = [ff.alloc(s) for s in sizes]
    assert bases == [0, 6]
    base = np.broadcast_to(np.array(bases, np.int32), (2, 1, 2)).copy()
    live = np.full((2, 1, 2), 2, np.int32)
    _, live, slot = O.prepare_decode_metadata(base, live)
    assert np.array_equal(base, z["meta_base"]) and np.array_equal(slot, z["meta_slot"])
    assert np.array_equal(live, z["meta_live"])
    assert slot.tolist() == [[[2, 8]], [[2, 8]]] and live.tolist() == [[[3, 3]], [[3, 3]]]
    assert [list(r) for r in ff.free] == z["meta_free_after"].tolist()
    for b, s in zip(bases, sizes):
        ff.release(b, s)
    assert [list(r) for r in ff.free] == z["meta_free_end"].tolist() == [[0, 32]]
    # decision recording, reference tests/test_compact_kv.py:252-282
    pos = np.full((2, 2, 2, 16), -1, np.int32)
    evm = np.zeros((2, 2, 2, 16), bool)
    livec = np.ones((2, 2, 2), np.int32)
    t, n = O.record_decisions(pos, evm, livec, z["record_evict_in"], [10, 20])
    assert [t, n] == z["record_stats"].tolist() == [4, 8]
    assert np.array_equal(pos, z["record_positions"]) and np.array_equal(evm, z["record_evict_mask"])


@pytest.mark.parametrize("tag,pool", [("f32", "f32"), ("fp8", "e4m3")])
def test_streaming_pack(ops_golden, tag, pool):
    z = ops_golden
    g = lambda n: z[f"pack_{tag}_{n}"]
    cu = g("cu")
    W = int(g("window")[0])
    headroom = int(g("max_tokens")[0])
    L = 2
    Hk = g("evict_l0").shape[1]
    nseq = len(cu) - 1
    for l in range(L):
        k, v, ev = bf(g(f"k_l{l}")), bf(g(f"v_l{l}")), g(f"evict_l{l}")
        ref_k, ref_v = g(f"compact_k_l{l}"), g(f"compact_v_l{l}")
        ck = np.zeros_like(ref_k)
        cvv = np.zeros_like(ref_v)
        ff = O.FirstFit(4096)
        # allocation pre-scan over the whole batch, then scatter (compact_kv.py:955-985)
        bases = []
        for s in range(nseq):
            T = int(cu[s + 1] - cu[s])
            C = min(1024, T + headroom)
            keep = O.pack_keep(ev[cu[s]:cu[s + 1]], W)
            sizes = O.span_sizes(keep.sum(axis=0), headroom, C)
            bases.append([ff.alloc(x) for x in sizes])
            assert sizes == g(f"cap_s{s}")[l].tolist()
        for s in range(nseq):
            T = int(cu[s + 1] - cu[s])
            C = min(1024, T + headroom)
            pos = np.full((Hk, C), -1, np.int32)
            evm = np.zeros((Hk, C), bool)
            live = O.pack_prefill_seq(k[cu[s]:cu[s + 1]], v[cu[s]:cu[s + 1]], ev[cu[s]:cu[s + 1]], W,
                                      bases[s], ck, cvv, pos, evm, pool)
            assert bases[s] == g(f"base_s{s}")[l].tolist()
            assert np.array_equal(live, g(f"live_s{s}")[l])
            assert np.array_equal(pos, g(f"pos_s{s}")[l])
            assert np.array_equal(evm, g(f"ev_s{s}")[l])
        # the reference pool is torch.empty outside the written spans: compare written rows only
        for s in range(nseq):
            for h in range(Hk):
                b, n = bases[s][h], int(g(f"live_s{s}")[l][h])
                assert np.array_equal(ck[b:b + n], ref_k[b:b + n])
                assert np.array_equal(cvv[b:b + n], ref_v[b:b + n])


@pytest.mark.parametrize("tag", ["f32", "fp8"])
def test_expiry_capacity9_window3(ops_golden, tag):
    """reference tests/test_compact_kv.py:1283-1329 fixture (capacity 9, W=3, positions 8 -> 10)."""
    z = ops_golden
    g = lambda s, n: z[f"expiry_{tag}_s{s}_{n}"].copy()
    live, pos, ev, base = g(0, "live"), g(0, "pos"), g(0, "ev"), g(0, "base")
    ks = [g(0, "k_l0"), g(0, "k_l1")]
    vs = [g(0, "v_l0"), g(0, "v_l1")]
    before = live.copy()

    def step(cur):
        for l in range(2):
            O.expire_layer(pos[l][None], ev[l][None], live[l][None], base[l][None], ks[l], vs[l], [cur], 3)

    def check(s):
        assert np.array_equal(live, g(s, "live")) and np.array_equal(pos, g(s, "pos"))
        assert np.array_equal(ev, g(s, "ev"))
        for l in range(2):
            assert np.array_equal(ks[l], g(s, f"k_l{l}")) and np.array_equal(vs[l], g(s, f"v_l{l}"))

    def append(p):
        for l in range(2):
            for h in range(2):
                i, b = int(live[l, h]), int(base[l, h])
                pos[l, h, i] = p
                ev[l, h, i] = p % 2 == 0
                val = np.full(4, np.float32(l * 10.0 + h + p * 0.01), np.float32)
                if tag == "fp8":
                    kb = encode_e4m3(val)
                    ks[l][b + i] = kb
                    vs[l][b + i] = encode_e4m3((decode_e4m3(kb) + np.float32(0.5)).astype(np.float32))
                else:
                    ks[l][b + i] = val
                    vs[l][b + i] = val + np.float32(0.5)
                live[l, h] += 1

    step(8)
    check(1)
    st = z[f"expiry_{tag}_stats8"].tolist()
    assert st == [int((before - live).sum()), int(before.min()), int(before.max()), int(live.min()), int(live.max())]
    append(8); step(9); check(2)
    append(9); step(10); check(3)


def test_expiry_incremental_equals_full_when_one_token_ages_out(ops_golden):
    z = ops_golden
    g = lambda n: z[f"expiry_f32_s2_{n}"].copy()
    for mr in (None, 1):
        live, pos, ev, base = g("live"), g("pos"), g("ev"), g("base")
        ks, vs = [g("k_l0"), g("k_l1")], [g("v_l0"), g("v_l1")]
        # re-create the state before step 10: append token 9 to the state after step 9
        for l in range(2):
            for h in range(2):
                i = int(live[l, h]); pos[l, h, i] = 9; ev[l, h, i] = False; live[l, h] += 1
        for l in range(2):
            O.expire_layer(pos[l][None], ev[l][None], live[l][None], base[l][None], ks[l], vs[l], [10], 3, mr)
        if mr is None:
            full = (live.copy(), pos.copy(), ev.copy())
        else:
            assert all(np.array_equal(a, b) for a, b in zip(full, (live, pos, ev)))


def test_expiry_random_multistep(ops_golden):
    z = ops_golden
    L, Hk = 2, 3
    W, T0 = int(z["expiryrand_window"][0]), int(z["expiryrand_T0"][0])
    live, pos, ev, base = (z[f"expiryrand_s0_{n}"].copy() for n in ("live", "pos", "ev", "base"))
    ks = [z[f"expiryrand_s0_k_l{l}"].copy() for l in range(L)]
    vs = [z[f"expiryrand_s0_v_l{l}"].copy() for l in range(L)]
    app_k, app_v, app_ev = z["expiryrand_app_k"], z["expiryrand_app_v"], z["expiryrand_app_ev"]
    for s in range(app_k.shape[0]):
        cur = T0 + s
        for l in range(L):
            O.expire_layer(pos[l][None], ev[l][None], live[l][None], base[l][None], ks[l], vs[l], [cur], W)
        b3, l3 = base[:, None, :], live[:, None, :]
        _, _, slot = O.prepare_decode_metadata(b3, l3)   # live is a view: incremented in place
        assert np.array_equal(slot, z[f"expiryrand_slot_{s}"])
        for l in range(L):
            for h in range(Hk):
                ks[l][slot[l, 0, h]] = app_k[s, l, h]
                vs[l][slot[l, 0, h]] = app_v[s, l, h]
        O.record_decisions(pos[:, None], ev[:, None], l3, app_ev[s][:, None, :], [cur])
        assert np.array_equal(live, z[f"expiryrand_live_{s}"])
    assert np.array_equal(pos, z["expiryrand_end_pos"]) and np.array_equal(ev, z["expiryrand_end_ev"])
    for l in range(L):
        for h in range(Hk):
            b, n = int(base[l, h]), int(live[l, h])
            assert np.array_equal(ks[l][b:b + n], z[f"expiryrand_end_k_l{l}"][b:b + n])
            assert np.array_equal(vs[l][b:b + n], z[f"expiryrand_end_v_l{l}"][b:b + n])


def test_kv_quant_roundtrip():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((200, 4, 64)).astype(np.float32) * np.array([0.1, 1, 10, 100], np.float32)[None, :, None]
    s = O.absmax_scale(x)
    raw = O.kv_quant(x, s)
    back = O.kv_dequant(raw, s)
    # e4m3 relative step is 2^-3 at worst -> half-step rounding error <= 2^-4 relative, + subnormal floor
    assert np.all(np.abs(back - x) <= np.abs(x) * 2.0 ** -4 + s[None, :, None] * 2.0 ** -10)
    assert np.array_equal(O.kv_quant(back, s), raw)          # idempotent
    assert np.abs(decode_e4m3(raw)).max() == 448.0
    one = np.ones(4, np.float32)
    assert np.array_equal(O.kv_quant(np.clip(x, -448, 448), one), encode_e4m3(np.clip(x, -448, 448)))

"""CPU checks of the oracle's chunked-prefill restatement (an extension: the reference prefills in
one pass, so these pin it to the reference-derived functions of the same oracle instead of to
reference vectors): the final span contents do not depend on the chunk size, and the chunk attention
reduces to the decode attention / plain causal attention in its two limits."""
from __future__ import annotations

import numpy as np

from oracle import compact_dms as O


def test_chunked_prefill_leaves_the_one_pass_contents():
    rng = np.random.default_rng(0)
    for T in (1, 7, 64, 257, 1000):
        for W in (0, 3, 16, 256):
            evict = rng.random(T) < 0.8
            want = np.nonzero(O.pack_keep(evict[:, None], W)[:, 0])[0]
            for chunk in (1, 5, 16, 100, 256, T, T + 3):
                got = O.chunked_prefill_state(evict, W, chunk)
                assert np.array_equal(got, want), (T, W, chunk)


def test_chunk_attention_limits():
    rng = np.random.default_rng(1)
    T, Hq, Hk, D, n = 9, 4, 2, 16, 21
    q = rng.standard_normal((T, Hq, D)).astype(np.float32)
    k = rng.standard_normal((T, Hk, D)).astype(np.float32)
    v = rng.standard_normal((T, Hk, D)).astype(np.float32)
    pk = [rng.standard_normal((n + h, D)).astype(np.float32) for h in range(Hk)]
    pv = [rng.standard_normal((n + h, D)).astype(np.float32) for h in range(Hk)]
    out, lse_d, lse_t = O.chunk_attention(q, k, v, pk, pv)
    assert np.all(lse_t >= lse_d)
    # every query = decode attention over (prefix rows + chunk tokens up to itself)
    for i in range(T):
        pool_k = np.concatenate([np.concatenate([pk[h], k[:i + 1, h]]) for h in range(Hk)])
        pool_v = np.concatenate([np.concatenate([pv[h], v[:i + 1, h]]) for h in range(Hk)])
        live = np.array([[n + h + i + 1 for h in range(Hk)]], np.int32)
        base = np.array([[0, live[0, 0]]], np.int32)
        want = O.decode_attention(q[i:i + 1], pool_k, pool_v, base, live)
        assert np.abs(out[i] - want[0]).max() < 1e-5
    # no prefix: plain causal attention, the two log-sum-exps coincide
    out0, d0, t0 = O.chunk_attention(q, k, v, [np.zeros((0, D), np.float32)] * Hk, [np.zeros((0, D), np.float32)] * Hk)
    assert np.allclose(d0, t0, atol=1e-6)
    assert np.abs(out0[0, 0] - v[0, 0]).max() < 1e-6          # the first token sees only itself


def test_chunked_state_property_random_chunk_schedules():
    """Hypothesis: for any evict pattern, window and chunk size the chunked state equals the one-pass
    state, and every intermediate state is what the decode-time rule keeps at that position."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=150, deadline=None)
    @given(st.lists(st.booleans(), min_size=1, max_size=300), st.integers(0, 64), st.integers(1, 320))
    def check(evict, window, chunk):
        ev = np.asarray(evict, bool)
        want = np.nonzero(O.pack_keep(ev[:, None], window)[:, 0])[0]
        assert np.array_equal(O.chunked_prefill_state(ev, window, chunk), want)
        # the state after the first chunk alone = live_mask of the decode rule at cur = chunk end - 1
        e = min(len(ev), chunk)
        first = O.chunked_prefill_state(ev[:e], window, chunk)
        keep = O.live_mask(ev[:e][None, :], e - 1, window)[0]
        assert np.array_equal(first, np.nonzero(keep)[0])

    check()

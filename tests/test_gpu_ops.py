"""GPU parity tests: every CUDA entry point (called through the C ABI) against the numpy oracle and
the vectors produced by the reference's CPU code.  Integer / byte results must be bit-exact;
attention outputs must be within 2e-2 max-abs of the float32 oracle (FP8 K/V, bf16 q)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import compact_dms as O
from oracle.dtypes import bf16_bits_to_f32, decode_e4m3, encode_e4m3

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-2      # max-abs, FP8 pools / bf16 activations vs float32 oracle
F32_TOL = 1e-4       # the reference's own tolerance for its float32 fixtures


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from fastdms_b200 import _lib
    _lib.lib()
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _status_clean(dev):
    from fastdms_b200 import _lib
    _lib.read_device_status(dev)
    yield
    assert _lib.read_device_status(dev) == 0, "a kernel raised a device status bit"


@pytest.fixture(params=["direct", "staged"])
def loader(request, monkeypatch):
    """Both page loaders of the FP8 attention kernels: per-lane loads into registers, and bulk copies
    into per-warp shared-memory rings."""
    monkeypatch.setenv("FDMS_ATTN_LOADER", request.param)
    return request.param


def t_bf16(a, dev):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(dev)


def t_fp8(a, dev):
    return torch.from_numpy(a.copy()).view(torch.float8_e4m3fn).to(dev)


def n_bf16(t):
    return bf16_bits_to_f32(t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16))


def n_u8(t):
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


# ------------------------------------------------------------------------------------------------
def test_extract_decisions(ops_golden, dev):
    from fastdms_b200.engine.dms import extract_dms_eviction_decisions
    z = ops_golden
    q = torch.from_numpy(z["extract_f32_q"]).to(dev)
    qc, ev = extract_dms_eviction_decisions(q, num_kv_heads=8, num_qo_heads=32, head_dim=64,
                                            alpha_scale=100.0, alpha_offset=5.0)
    assert torch.equal(q.cpu(), torch.from_numpy(z["extract_f32_q"]))          # not in place
    assert np.array_equal(ev.cpu().numpy(), z["extract_f32_evict"])
    assert np.array_equal(qc.cpu().numpy(), z["extract_f32_q_out"])
    out = torch.empty((11, 8), dtype=torch.bool, device=dev)
    q2, ev2 = extract_dms_eviction_decisions(q.clone(), num_kv_heads=8, num_qo_heads=32, head_dim=64,
                                             alpha_scale=100.0, alpha_offset=5.0, inplace=True, out=out)
    assert ev2.data_ptr() == out.data_ptr() and np.array_equal(out.cpu().numpy(), z["extract_f32_evict"])
    qb = t_bf16(z["extract_bf16_q"], dev)
    qc, ev = extract_dms_eviction_decisions(qb, num_kv_heads=2, num_qo_heads=4, head_dim=64,
                                            alpha_scale=100.0, alpha_offset=5.0)
    assert np.array_equal(ev.cpu().numpy(), z["extract_bf16_evict"])
    assert np.array_equal(n_u8(qc), z["extract_bf16_q_out"].view(np.uint8))
    qn = torch.from_numpy(z["extract_neg_q"]).to(dev).view(9, 8 * 32)          # flat [T, H*D] form
    qc, ev = extract_dms_eviction_decisions(qn, num_kv_heads=4, num_qo_heads=8, head_dim=32,
                                            alpha_scale=-50.0, alpha_offset=1.0)
    assert np.array_equal(ev.cpu().numpy(), z["extract_neg_evict"])
    assert np.array_equal(qc.view(9, 8, 32).cpu().numpy(), z["extract_neg_q_out"])
    with pytest.raises(ValueError):
        extract_dms_eviction_decisions(q, num_kv_heads=5, num_qo_heads=32, head_dim=64, alpha_scale=100.0, alpha_offset=5.0)


@pytest.mark.parametrize("tag,act,pool", [("f32d32", "f32", "f32"), ("bf16d64", "bf16", "e4m3"), ("bf16d128", "bf16", "e4m3")])
def test_fused_rope_store_decode(ops_golden, dev, tag, act, pool):
    from fastdms_b200.layers.compact_attention import fused_dms_rope_store_compact_decode, store_compact_kvcache
    z = ops_golden
    g = lambda n: z[f"ropestore_{tag}_{n}"]
    up = (lambda a: torch.from_numpy(a.copy()).to(dev)) if act == "f32" else (lambda a: t_bf16(a, dev))
    raw = lambda t: n_u8(t)
    q, k, v = up(g("q")), up(g("k")), up(g("v"))
    B, Hk, D = k.shape
    positions = torch.from_numpy(g("positions")).to(dev)
    cache = torch.zeros((int(positions.max()) + 1, 1, D), dtype=torch.float32, device=dev)
    cache[positions, 0] = torch.from_numpy(g("cos_sin_rows")).to(dev)
    pool_dt = torch.float32 if pool == "f32" else torch.float8_e4m3fn
    slots = torch.from_numpy(g("slots")).to(dev)
    ref_ck, ref_cv = g("compact_k"), g("compact_v")

    def run(**kw):
        qq, kk = q.clone(), k.clone()
        ck = torch.zeros(ref_ck.shape, dtype=torch.float32, device=dev).to(pool_dt)
        cv = torch.zeros_like(ck)
        ev = torch.empty((B, Hk), dtype=torch.bool, device=dev)
        fused_dms_rope_store_compact_decode(qq, kk, v, cache, ck, cv, slots, ev, positions, num_kv_heads=Hk,
                                            alpha_scale=100.0, alpha_offset=5.0, **kw)
        return qq, kk, ck, cv, ev

    qq, kk, ck, cv, ev = run()
    assert np.array_equal(ev.cpu().numpy(), g("evict"))
    assert np.array_equal(raw(qq), g("q_out").view(np.uint8).reshape(raw(qq).shape))
    assert np.array_equal(raw(kk), g("k_out").view(np.uint8).reshape(raw(kk).shape))
    assert np.array_equal(raw(ck), ref_ck.view(np.uint8).reshape(raw(ck).shape))
    assert np.array_equal(raw(cv), ref_cv.view(np.uint8).reshape(raw(cv).shape))
    # transient k left alone, pool identical
    qq, kk, ck, cv, ev = run(store_transient_k=False)
    assert torch.equal(kk, k) and np.array_equal(raw(ck), ref_ck.view(np.uint8).reshape(raw(ck).shape))
    assert np.array_equal(raw(qq), g("q_out").view(np.uint8).reshape(raw(qq).shape))
    # q left alone (rotated later inside attention), decisions identical
    qq, kk, ck, cv, ev = run(store_q=False)
    assert torch.equal(qq, q) and np.array_equal(ev.cpu().numpy(), g("evict"))
    assert np.array_equal(raw(ck), ref_ck.view(np.uint8).reshape(raw(ck).shape))
    # plain store of already-rotated k
    ck2 = torch.zeros_like(ck)
    cv2 = torch.zeros_like(cv)
    store_compact_kvcache(up(g("k_out")), v, ck2, cv2, slots)
    assert torch.equal(ck2.view(torch.uint8), ck.view(torch.uint8)) and torch.equal(cv2.view(torch.uint8), cv.view(torch.uint8))
    with pytest.raises(ValueError):
        fused_dms_rope_store_compact_decode(q, k, v, cache, ck, cv, slots[:, :1], ev, positions, num_kv_heads=Hk,
                                            alpha_scale=100.0, alpha_offset=5.0)


def test_store_with_per_head_scale(dev):
    from fastdms_b200.layers.compact_attention import store_compact_kvcache
    rng = np.random.default_rng(11)
    B, Hk, D = 4, 2, 64
    k = rng.standard_normal((B, Hk, D)).astype(np.float32) * 30
    v = rng.standard_normal((B, Hk, D)).astype(np.float32) * 0.01
    ks, vs = O.absmax_scale(k), O.absmax_scale(v)
    kb = torch.from_numpy(k).to(dev).to(torch.bfloat16)
    vb = torch.from_numpy(v).to(dev).to(torch.bfloat16)
    slots = torch.arange(B * Hk, dtype=torch.int32, device=dev).view(B, Hk)
    ck = torch.zeros((B * Hk, D), dtype=torch.float8_e4m3fn, device=dev)
    cv = torch.zeros_like(ck)
    store_compact_kvcache(kb, vb, ck, cv, slots, k_scale=torch.from_numpy(ks).to(dev), v_scale=torch.from_numpy(vs).to(dev))
    exp_k = O.kv_quant(n_bf16(kb), ks).reshape(B * Hk, D)
    exp_v = O.kv_quant(n_bf16(vb), vs).reshape(B * Hk, D)
    assert np.array_equal(n_u8(ck), exp_k) and np.array_equal(n_u8(cv), exp_v)


# ------------------------------------------------------------------------------------------------
def _attn(dev, q, k, v, base, live, **kw):
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    return compact_decode_attention(q, k, v, torch.from_numpy(base).to(dev), torch.from_numpy(live).to(dev), **kw)


def test_attention_reference_f32_fixture(ops_golden, dev):
    """The reference's own split-K test shape (float32, head_dim 16): generic kernel."""
    z = ops_golden
    q, k, v = (torch.from_numpy(z[f"attn_f32d16_{n}"]).to(dev) for n in ("q", "k", "v"))
    out = _attn(dev, q, k, v, z["attn_f32d16_base"], z["attn_f32d16_live"], max_live_count=20, block_n=16)
    assert np.abs(out.cpu().numpy() - z["attn_f32d16_out"]).max() < F32_TOL
    o2 = _attn(dev, torch.ones((1, 4, 4), device=dev), torch.from_numpy(z["packka_compact_k"]).to(dev),
               torch.from_numpy(z["packka_compact_v"]).to(dev), z["packka_base"], z["packka_live"], scale=1.0)
    assert np.abs(o2.cpu().numpy() - z["packka_attn_out"]).max() < F32_TOL


@pytest.mark.parametrize("tag,scale", [("fp8d64", None), ("fp8d128", 0.11)])
@pytest.mark.parametrize("generic", [False, True])
def test_attention_fp8_golden(ops_golden, dev, tag, scale, generic, monkeypatch, loader):
    z = ops_golden
    if generic:
        monkeypatch.setenv("FDMS_ATTN_FORCE_GENERIC", "1")
    q = t_bf16(z[f"attn_{tag}_q"], dev)
    k, v = t_fp8(z[f"attn_{tag}_k"], dev), t_fp8(z[f"attn_{tag}_v"], dev)
    base, live = z[f"attn_{tag}_base"], z[f"attn_{tag}_live"]
    out = _attn(dev, q, k, v, base, live, scale=scale)
    want = O.decode_attention(bf16_bits_to_f32(z[f"attn_{tag}_q"].view(np.uint16)), z[f"attn_{tag}_k"],
                              z[f"attn_{tag}_v"], base, live, scale, pool_dtype="e4m3")
    assert np.abs(n_bf16(out) - want).max() < ATTN_TOL
    # and against the reference's own output (bf16), same tolerance
    assert np.abs(n_bf16(out) - bf16_bits_to_f32(z[f"attn_{tag}_out"].view(np.uint16))).max() < ATTN_TOL


def _config2_case(rng, B, Hk, G, D, mean, jitter, recent, paged, pool_pages_extra=9):
    """Config-2 style inputs: ragged spans, N(0,1) K/V quantised with per-head absmax scales."""
    live = (mean + rng.integers(-jitter, jitter + 1, size=(B, Hk)) + recent).astype(np.int32)
    pages = -(-live // 16)
    total_pages = int(pages.sum()) + pool_pages_extra
    rows = total_pages * 16
    kf = rng.standard_normal((rows, D)).astype(np.float32)
    vf = rng.standard_normal((rows, D)).astype(np.float32)
    q = rng.standard_normal((B, Hk * G, D)).astype(np.float32)
    ks = np.full(Hk, np.abs(kf).max() / 448.0, np.float32) * (1 + 0.1 * np.arange(Hk, dtype=np.float32))
    vs = np.full(Hk, np.abs(vf).max() / 448.0, np.float32) * (1 + 0.05 * np.arange(Hk, dtype=np.float32))
    maxp = int(pages.max())
    bt = np.full((B, Hk, maxp), -1, np.int32)
    base = np.zeros((B, Hk), np.int32)
    kq = np.zeros((rows, D), np.uint8)
    vq = np.zeros((rows, D), np.uint8)
    if paged:
        perm = rng.permutation(total_pages)
        nxt = 0
        for b in range(B):
            for h in range(Hk):
                for p in range(int(pages[b, h])):
                    bt[b, h, p] = perm[nxt]; nxt += 1
                rws = O.gather_span(np.arange(rows), 0, int(live[b, h]), bt[b, h])
                kq[rws] = encode_e4m3(kf[rws] / ks[h]); vq[rws] = encode_e4m3(vf[rws] / vs[h])
    else:
        cur = 0
        for b in range(B):
            for h in range(Hk):
                base[b, h] = cur
                n = int(live[b, h])
                kq[cur:cur + n] = encode_e4m3(kf[cur:cur + n] / ks[h]); vq[cur:cur + n] = encode_e4m3(vf[cur:cur + n] / vs[h])
                cur += n + int(rng.integers(0, 5))
    return q, kq, vq, base, live, (bt if paged else None), ks, vs


@pytest.mark.parametrize("D,G", [(64, 4), (128, 4), (64, 8), (64, 1)])
@pytest.mark.parametrize("paged", [False, True])
def test_attention_ragged_scaled(dev, D, G, paged, loader):
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    rng = np.random.default_rng(100 + D + G + int(paged))
    B, Hk = 3, 2
    q, kq, vq, base, live, bt, ks, vs = _config2_case(rng, B, Hk, G, D, 300, 100, 40, paged)
    qb = torch.from_numpy(q).to(dev).to(torch.bfloat16)
    out = compact_decode_attention(
        qb, t_fp8(kq, dev), t_fp8(vq, dev), torch.from_numpy(base).to(dev), torch.from_numpy(live).to(dev),
        block_tables=None if bt is None else torch.from_numpy(bt).to(dev),
        k_scale=torch.from_numpy(ks).to(dev), v_scale=torch.from_numpy(vs).to(dev))
    want = O.decode_attention(n_bf16(qb), kq, vq, base, live, pool_dtype="e4m3", k_scale=ks, v_scale=vs, block_tables=bt)
    assert np.abs(n_bf16(out) - want).max() < ATTN_TOL


def test_attention_config2_shape(dev, loader):
    """The op-level benchmark shape: 8 sequences, 32 q / 8 KV heads, head_dim 64, live = 1024 +- 128 + 256,
    16-row pages with randomly permuted block tables, per-head absmax scales."""
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    rng = np.random.default_rng(0)
    q, kq, vq, base, live, bt, ks, vs = _config2_case(rng, 8, 8, 4, 64, 1024, 128, 256, True)
    qb = torch.from_numpy(q).to(dev).to(torch.bfloat16)
    args = (qb, t_fp8(kq, dev), t_fp8(vq, dev), torch.from_numpy(base).to(dev), torch.from_numpy(live).to(dev))
    kw = dict(block_tables=torch.from_numpy(bt).to(dev), k_scale=torch.from_numpy(ks).to(dev), v_scale=torch.from_numpy(vs).to(dev))
    out = compact_decode_attention(*args, **kw)
    want = O.decode_attention(n_bf16(qb), kq, vq, base, live, pool_dtype="e4m3", k_scale=ks, v_scale=vs, block_tables=bt)
    assert np.abs(n_bf16(out) - want).max() < ATTN_TOL
    # repeated calls reuse the split-K workspace (counters must come back to zero) and are deterministic
    for _ in range(3):
        again = compact_decode_attention(*args, **kw)
        assert torch.equal(again, out)


@pytest.mark.parametrize("splits,chunks", [(1, 1), (2, 1), (8, 1), (16, 1), (1, 3), (4, 5), (8, 64)])
def test_attention_split_shapes(dev, splits, chunks, monkeypatch, loader):
    """Every split-K shape (cluster size x clusters per span) gives the same answer, including
    shapes with more CTAs than pages; repeated calls leave the workspace counters at zero."""
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    monkeypatch.setenv("FDMS_ATTN_SPLITS", str(splits))
    monkeypatch.setenv("FDMS_ATTN_CHUNKS", str(chunks))
    monkeypatch.setenv("FDMS_ATTN_MAX_SPLITS", "16")
    rng = np.random.default_rng(40 + splits + chunks)
    q, kq, vq, base, live, bt, ks, vs = _config2_case(rng, 2, 2, 4, 64, 500, 300, 3, True)
    live[0, 0] = 5            # fewer pages than CTAs
    qb = torch.from_numpy(q).to(dev).to(torch.bfloat16)
    args = (qb, t_fp8(kq, dev), t_fp8(vq, dev), torch.from_numpy(base).to(dev), torch.from_numpy(live).to(dev))
    kw = dict(block_tables=torch.from_numpy(bt).to(dev), k_scale=torch.from_numpy(ks).to(dev), v_scale=torch.from_numpy(vs).to(dev))
    want = O.decode_attention(n_bf16(qb), kq, vq, base, live, pool_dtype="e4m3", k_scale=ks, v_scale=vs, block_tables=bt)
    for _ in range(3):
        out = compact_decode_attention(*args, **kw)
        assert np.abs(n_bf16(out) - want).max() < ATTN_TOL


def test_attention_edge_lengths(dev, loader):
    """live = 1, exact page multiples, one long span next to tiny ones, and an empty span."""
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    rng = np.random.default_rng(5)
    D, G, Hk = 64, 4, 2
    live = np.array([[1, 16], [17, 5000], [32, 0]], np.int32)
    B = live.shape[0]
    base = np.zeros_like(live)
    cur = 0
    for b in range(B):
        for h in range(Hk):
            base[b, h] = cur; cur += int(live[b, h]) + 3
    kq = encode_e4m3(rng.standard_normal((cur, D)).astype(np.float32))
    vq = encode_e4m3(rng.standard_normal((cur, D)).astype(np.float32))
    q = rng.standard_normal((B, Hk * G, D)).astype(np.float32)
    qb = torch.from_numpy(q).to(dev).to(torch.bfloat16)
    out = compact_decode_attention(qb, t_fp8(kq, dev), t_fp8(vq, dev), torch.from_numpy(base).to(dev), torch.from_numpy(live).to(dev))
    got = n_bf16(out)
    live2 = live.copy(); live2[2, 1] = 1     # the oracle divides by zero on an empty span: compare the rest
    want = O.decode_attention(n_bf16(qb), kq, vq, base, live2, pool_dtype="e4m3")
    mask = np.ones_like(got, bool); mask[2, G:] = False
    assert np.abs(got - want)[mask].max() < ATTN_TOL
    assert np.all(got[2, G:] == 0)            # an empty span yields zeros, not NaN


def test_attention_inline_q_rope(ops_golden, dev, loader):
    """q rotated inside the attention kernel == q rotated by the store kernel first."""
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    z = ops_golden
    g = lambda n: z[f"ropestore_bf16d64_{n}"]
    q = t_bf16(g("q"), dev)
    B, Hq, D = q.shape
    Hk = g("k").shape[1]
    positions = torch.from_numpy(g("positions")).to(dev)
    cache = torch.zeros((int(positions.max()) + 1, 1, D), dtype=torch.float32, device=dev)
    cache[positions, 0] = torch.from_numpy(g("cos_sin_rows")).to(dev)
    rng = np.random.default_rng(2)
    live = rng.integers(20, 90, size=(B, Hk)).astype(np.int32)
    base = (np.arange(B * Hk, dtype=np.int32) * 100).reshape(B, Hk)
    kq = encode_e4m3(rng.standard_normal((B * Hk * 100, D)).astype(np.float32))
    vq = encode_e4m3(rng.standard_normal((B * Hk * 100, D)).astype(np.float32))
    out = compact_decode_attention(q, t_fp8(kq, dev), t_fp8(vq, dev), torch.from_numpy(base).to(dev),
                                   torch.from_numpy(live).to(dev), q_rope_positions=positions, q_rope_cos_sin_cache=cache)
    qf, _ = O.extract_decisions(bf16_bits_to_f32(g("q").view(np.uint16)), Hk, 100.0, 5.0)
    cs = cache[:, 0].cpu().numpy()
    pos = g("positions")
    q_rot = O.rope_neox(qf, cs[pos, : D // 2][:, None, :], cs[pos, D // 2:][:, None, :])
    want = O.decode_attention(q_rot, kq, vq, base, live, pool_dtype="e4m3")
    assert np.abs(n_bf16(out) - want).max() < ATTN_TOL
    with pytest.raises(ValueError):
        compact_decode_attention(q, t_fp8(kq, dev), t_fp8(vq, dev), torch.from_numpy(base).to(dev),
                                 torch.from_numpy(live).to(dev), q_rope_positions=positions)


@pytest.mark.parametrize("D,G,paged,scaled,mean", [(64, 4, True, True, 200), (64, 4, False, False, 200), (128, 4, True, False, 200),
                                                   (64, 8, False, True, 200), (64, 4, True, True, 5000), (128, 2, False, True, 9000)])
def test_fused_store_attention_equals_store_then_attention(dev, D, G, paged, scaled, mean, loader):
    """One launch (decision + RoPE + FP8 store + attention) against the two separate kernels:
    identical decisions, identical pool bytes, identical attention output; spans whose new row
    opens a fresh page (live % 16 == 1) and fills one (live % 16 == 0) are included."""
    from fastdms_b200.layers.compact_attention import (compact_decode_attention, fused_dms_rope_store_compact_decode,
                                                       fused_store_decode_attention)
    rng = np.random.default_rng(70 + D + G)
    B, Hk = 4, 2
    qn, kq, vq, base, live, bt, ks, vs = _config2_case(rng, B, Hk, G, D, mean, 80, 17, paged)
    live[0, 0], live[1, 1], live[2, 0] = 17, 32, 1                           # fresh page, full page, single row
    qb = torch.from_numpy(qn).to(dev).to(torch.bfloat16)
    qb[:, 0::G, -1] = torch.tensor([0.01, 0.06, 0.05, 0.08, 0.10, -0.01, 0.3, -0.2], device=dev).view(B, Hk).to(torch.bfloat16)
    k = torch.from_numpy(rng.standard_normal((B, Hk, D)).astype(np.float32)).to(dev).to(torch.bfloat16)
    v = torch.from_numpy(rng.standard_normal((B, Hk, D)).astype(np.float32)).to(dev).to(torch.bfloat16)
    positions = torch.tensor([5, 100, 0, 777], device=dev)
    half = D // 2
    inv = 1.0 / (500000.0 ** (np.arange(half, dtype=np.float32) / half))
    ang = np.arange(800, dtype=np.float32)[:, None] * inv[None, :]
    cache = torch.from_numpy(np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)).to(dev).unsqueeze(1)
    live_t, base_t = torch.from_numpy(live).to(dev), torch.from_numpy(base).to(dev)
    bt_t = None if bt is None else torch.from_numpy(bt).to(dev)
    kw = dict(k_scale=torch.from_numpy(ks).to(dev), v_scale=torch.from_numpy(vs).to(dev)) if scaled else {}
    rows = kq.shape[0]
    pool_k = torch.zeros((rows, D), dtype=torch.uint8, device=dev)
    pool_k[: kq.shape[0]] = torch.from_numpy(kq).to(dev)
    pool_v = torch.zeros((rows, D), dtype=torch.uint8, device=dev)
    pool_v[: vq.shape[0]] = torch.from_numpy(vq).to(dev)
    # slot of the appended row = logical row live - 1
    idx = live - 1
    slot = (np.take_along_axis(bt, (idx // 16)[..., None], axis=2)[..., 0] * 16 + idx % 16) if paged else base + idx
    slot_t = torch.from_numpy(slot.astype(np.int32)).to(dev)

    ck1, cv1 = pool_k.clone().view(torch.float8_e4m3fn), pool_v.clone().view(torch.float8_e4m3fn)
    q1, k1 = qb.clone(), k.clone()
    ev1 = torch.empty((B, Hk), dtype=torch.bool, device=dev)
    fused_dms_rope_store_compact_decode(q1, k1, v, cache, ck1, cv1, slot_t, ev1, positions, num_kv_heads=Hk,
                                        alpha_scale=100.0, alpha_offset=5.0, store_transient_k=False, **kw)
    want = compact_decode_attention(q1, ck1, cv1, base_t, live_t, block_tables=bt_t, **kw)

    ck2, cv2 = pool_k.clone().view(torch.float8_e4m3fn), pool_v.clone().view(torch.float8_e4m3fn)
    q2 = qb.clone()
    ev2 = torch.empty((B, Hk), dtype=torch.bool, device=dev)
    got = fused_store_decode_attention(q2, k, v, cache, ck2, cv2, base_t, live_t, ev2, positions, num_kv_heads=Hk,
                                       alpha_scale=100.0, alpha_offset=5.0, block_tables=bt_t, **kw)
    assert torch.equal(ev1, ev2)
    assert torch.equal(ck1.view(torch.uint8), ck2.view(torch.uint8)) and torch.equal(cv1.view(torch.uint8), cv2.view(torch.uint8))
    assert torch.equal(q2, qb)                                     # q is left untouched
    assert torch.equal(got, want)
    with pytest.raises(ValueError):
        fused_store_decode_attention(q2, k, v, cache, ck2.view(torch.uint8).float(), cv2.view(torch.uint8).float(), base_t,
                                     live_t, ev2, positions, num_kv_heads=Hk, alpha_scale=100.0, alpha_offset=5.0)


def test_attention_argument_errors(dev):
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    q = torch.zeros((2, 8, 64), dtype=torch.bfloat16, device=dev)
    k = torch.zeros((64, 64), dtype=torch.float8_e4m3fn, device=dev)
    meta = torch.ones((2, 2), dtype=torch.int32, device=dev)
    with pytest.raises(ValueError):
        compact_decode_attention(q[0], k, k, meta, meta)
    with pytest.raises(ValueError):
        compact_decode_attention(q, k, k[:, :32], meta, meta)
    with pytest.raises(ValueError):
        compact_decode_attention(q, k, k, meta[:1], meta[:1])
    with pytest.raises(ValueError):
        compact_decode_attention(q, k, k, torch.ones((2, 3), dtype=torch.int32, device=dev), torch.ones((2, 3), dtype=torch.int32, device=dev))
    with pytest.raises(RuntimeError):
        compact_decode_attention(q.cpu(), k.cpu(), k.cpu(), meta.cpu(), meta.cpu())


# ------------------------------------------------------------------------------------------------
def test_kv_quant_dequant(dev):
    from fastdms_b200.layers.compact_attention import kv_dequantize_fp8, kv_quantize_fp8
    rng = np.random.default_rng(7)
    x = rng.standard_normal((300, 8, 64)).astype(np.float32) * np.logspace(-2, 2, 8, dtype=np.float32)[None, :, None]
    s = O.absmax_scale(x)
    xt, st = torch.from_numpy(x).to(dev), torch.from_numpy(s).to(dev)
    qd = kv_quantize_fp8(xt, st)
    assert np.array_equal(n_u8(qd), O.kv_quant(x, s))
    assert np.array_equal(kv_dequantize_fp8(qd, st).cpu().numpy(), O.kv_dequant(O.kv_quant(x, s), s))
    xb = xt.to(torch.bfloat16)
    assert np.array_equal(n_u8(kv_quantize_fp8(xb, st)), O.kv_quant(n_bf16(xb), s))
    assert np.array_equal(n_bf16(kv_dequantize_fp8(qd, st, torch.bfloat16)), O.kv_dequant(O.kv_quant(x, s), s, "bf16"))
    # scale None is the reference's bare cast; out-of-range saturates to +-448
    big = torch.tensor([[[1000.0, -1000.0] + [0.5] * 14]], device=dev)
    assert decode_e4m3(n_u8(kv_quantize_fp8(big)))[0, 0, :3].tolist() == [448.0, -448.0, 0.5]
    # idempotence at full config-2 volume (round trip is a fixed point)
    y = torch.randn((81920, 8, 64), device=dev, dtype=torch.bfloat16)
    sc = (y.float().abs().amax(dim=(0, 2)) / 448.0).contiguous()
    q1 = kv_quantize_fp8(y, sc)
    q2 = kv_quantize_fp8(kv_dequantize_fp8(q1, sc), sc)
    assert torch.equal(q1.view(torch.uint8), q2.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,n", [(8, 128256), (1, 151936), (3, 1024), (64, 8191), (5, 7), (2, 8193)])
def test_greedy_argmax_kernel_equals_torch_argmax(dev, dtype, rows, n):
    """One-launch row argmax of the greedy head against `logits.argmax(dim=-1)` (reference:
    engine/model_runner.py:1147-1151): exact indices, lowest index on ties, NaN largest, strided
    rows, and a scratch buffer that is left zeroed (shared by consecutive calls)."""
    from fastdms_b200.layers.sampler import argmax_workspace, greedy_argmax
    g = torch.Generator(device=dev).manual_seed(rows * 1000 + n)
    ws = argmax_workspace(rows, dev)
    x = torch.randn((rows, n), device=dev, generator=g).to(dtype)
    assert torch.equal(greedy_argmax(x, ws), x.argmax(dim=-1))
    # 16-bit logits tie often: the first of the equal maxima is the answer
    assert torch.equal(greedy_argmax(x, ws), first_max(x))
    # a planted tie and a planted NaN
    y = x.clone()
    y[:, n // 2] = 60000.0
    y[:, n - 1] = 60000.0
    assert greedy_argmax(y, ws).tolist() == [n // 2] * rows
    y[0, n // 3] = float("nan")
    assert int(greedy_argmax(y, ws)[0]) == n // 3
    # all-negative rows, rows of a wider buffer (row stride != n), no scratch given
    wide = -torch.rand((rows, n + 24), device=dev, generator=g).to(dtype) - 1.0
    view = wide[:, 8:8 + n]
    assert torch.equal(greedy_argmax(view), first_max(view))
    assert int(ws.count_nonzero()) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,hq,hk,d", [(8, 32, 8, 128), (3, 16, 4, 128), (300, 8, 2, 64), (1, 4, 4, 256)])
def test_qk_rmsnorm_equals_two_rmsnorm_calls(dev, dtype, rows, hq, hk, d):
    """The one-launch per-head RMSNorm of q and k (in place in the fused projection output) gives the bits of
    the two RMSNorm modules it replaces (reference: two calls of layers/layernorm.py:16-25 in the Qwen3 block)."""
    from fastdms_b200.layers.layernorm import RMSNorm, qk_rmsnorm_
    g = torch.Generator(device=dev).manual_seed(rows + hq + d)
    qkv = torch.randn((rows, (hq + 2 * hk) * d), device=dev, generator=g).to(dtype)
    qn, kn = RMSNorm(d, eps=1e-6).to(dev).to(dtype), RMSNorm(d, eps=1e-6).to(dev).to(dtype)
    qn.weight.data.copy_((1.0 + 0.1 * torch.randn(d, device=dev, generator=g)).to(dtype))
    kn.weight.data.copy_((1.0 + 0.1 * torch.randn(d, device=dev, generator=g)).to(dtype))
    q, k, v = qkv.split([hq * d, hk * d, hk * d], dim=-1)
    want_q = qn(q.reshape(rows, hq, d).contiguous())
    want_k = kn(k.reshape(rows, hk, d).contiguous())
    want_v = v.clone()
    with torch.inference_mode():
        assert qk_rmsnorm_(q.view(rows, hq, d), k.view(rows, hk, d), qn, kn)
    assert torch.equal(q.reshape(rows, hq, d), want_q)
    assert torch.equal(k.reshape(rows, hk, d), want_k)
    assert torch.equal(v, want_v)                      # the neighbouring v columns are untouched


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,inter,k,bias", [(8, 8192, 2048, False), (3, 6144, 4096, True), (1, 1536, 2048, True), (8, 16, 2048, False)])
def test_gated_decode_linear_equals_linear_then_silu_mul(dev, dtype, rows, inter, k, bias):
    """gate_up projection + SiLU(gate) * up in one launch (`fdms_linear_decode_gated`): the bits of the decode
    linear kernel followed by the SiLU-and-multiply kernel (reference: models/llama.py MLP.forward,
    layers/activation.py SiluAndMul)."""
    from fastdms_b200 import _lib
    from fastdms_b200.layers.activation import SiluAndMul
    from fastdms_b200.layers.linear import linear
    lib = _lib.lib()
    g = torch.Generator(device=dev).manual_seed(rows + inter + k)
    w = (torch.randn((2 * inter, k), device=dev, generator=g) * k ** -0.5).to(dtype)
    b = torch.randn((2 * inter,), device=dev, generator=g).to(dtype) if bias else None
    x = (2.0 * torch.randn((rows, k), device=dev, generator=g)).to(dtype)
    with torch.inference_mode():
        want = SiluAndMul()(linear(x, w, b))
        y = torch.full((rows, inter), float("nan"), device=dev, dtype=dtype)
        _lib.check(lib.fdms_linear_decode_gated(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _lib.ptr(b), y.data_ptr(),
                                                y.stride(0), _lib.dtype_code(dtype), rows, 2 * inter, k, _lib.stream_ptr(dev)))
    assert torch.equal(y, want)
    ref = torch.nn.functional.silu((x.float() @ w[:inter].float().t()) + (b[:inter].float() if bias else 0.0)) * \
        ((x.float() @ w[inter:].float().t()) + (b[inter:].float() if bias else 0.0))
    assert float((y.float() - ref).abs().max()) <= 3 * 2.0 ** (-8 if dtype == torch.bfloat16 else -11) * float(ref.abs().max()) + 1e-3


def first_max(x):
    idx = torch.arange(x.shape[1], device=x.device).expand_as(x)
    return torch.where(x == x.max(dim=-1, keepdim=True).values, idx, x.shape[1]).min(dim=-1).values


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,hidden", [(8, 2048), (3, 4096), (257, 256), (64, 128), (5, 8192)])
def test_rmsnorm_and_silu_kernels_match_torch_ops(dev, dtype, rows, hidden):
    """Single-launch RMSNorm (+ residual) and SiLU*up against the torch op chains they replace
    (reference: layers/layernorm.py:16-48, layers/activation.py); tolerance = two roundings of the
    16-bit type (the float32 sum is taken in a different order)."""
    from fastdms_b200.layers.activation import SiluAndMul
    from fastdms_b200.layers.layernorm import RMSNorm
    g = torch.Generator(device=dev).manual_seed(rows * 131 + hidden)
    x = torch.randn((rows, hidden), device=dev, generator=g).to(dtype)
    res = torch.randn((rows, hidden), device=dev, generator=g).to(dtype)
    norm = RMSNorm(hidden, eps=1e-5).to(dev).to(dtype)
    norm.weight.data.copy_((1.0 + 0.1 * torch.randn(hidden, device=dev, generator=g)).to(dtype))

    def ref(x, residual=None):
        xf = x.float() if residual is None else x.float() + residual.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + 1e-5)).to(dtype) * norm.weight
        return y if residual is None else (y, xf.to(dtype))

    tol = 2.0 ** (-6 if dtype == torch.bfloat16 else -9)       # two roundings, each up to one ulp apart
    y = norm(x)
    want = ref(x)
    assert y.dtype == dtype and y.shape == x.shape
    assert ((y.float() - want.float()).abs() <= tol * want.float().abs() + 1e-6).all()
    y2, r2 = norm(x, res)
    w2, wr2 = ref(x, res)
    assert torch.equal(r2, wr2)
    assert ((y2.float() - w2.float()).abs() <= tol * w2.float().abs() + 1e-6).all()
    # strided rows (a view into a wider buffer) take the same path
    wide = torch.randn((rows, 2 * hidden), device=dev, generator=g).to(dtype)
    yv = norm(wide[:, :hidden])
    wv = ref(wide[:, :hidden])
    assert ((yv.float() - wv.float()).abs() <= tol * wv.float().abs() + 1e-6).all()
    act = SiluAndMul()
    z = act(wide)
    a, b = wide.chunk(2, -1)
    wz = torch.nn.functional.silu(a) * b
    assert z.shape == wz.shape
    assert ((z.float() - wz.float()).abs() <= 2 * tol * wz.float().abs() + 1e-6).all()


def test_positions_outside_the_rotary_table_are_flagged_not_followed(dev):
    """positions index the cos/sin table; a value outside it must raise FDMS_DEV_BAD_INDEX in the
    status word (and be read as position 0), for the store kernel, the inline-RoPE attention and
    the fused launch alike."""
    from fastdms_b200 import _lib
    from fastdms_b200.layers.compact_attention import (compact_decode_attention, fused_dms_rope_store_compact_decode,
                                                       fused_store_decode_attention)
    B, Hk, G, D = 2, 2, 4, 64
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn((B, Hk * G, D), device=dev, generator=g).to(torch.bfloat16)
    k = torch.randn((B, Hk, D), device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn((B, Hk, D), device=dev, generator=g).to(torch.bfloat16)
    cache = torch.randn((32, 1, D), device=dev, generator=g)
    ck = torch.zeros((256, D), device=dev, dtype=torch.float8_e4m3fn)
    cv = torch.zeros_like(ck)
    base = torch.tensor([[0, 64], [128, 192]], device=dev, dtype=torch.int32)
    live = torch.full((B, Hk), 20, device=dev, dtype=torch.int32)
    ev = torch.empty((B, Hk), dtype=torch.bool, device=dev)
    bad = torch.tensor([5, 1 << 40], device=dev)            # far beyond the 32 rows of the table
    ok = torch.tensor([5, 31], device=dev)
    assert _lib.read_device_status(dev) == 0
    for call in (
        lambda pos: fused_dms_rope_store_compact_decode(q.clone(), k.clone(), v, cache, ck, cv, (base + live - 1).contiguous(), ev,
                                                        pos, num_kv_heads=Hk, alpha_scale=100.0, alpha_offset=5.0),
        lambda pos: compact_decode_attention(q, ck, cv, base, live, q_rope_positions=pos, q_rope_cos_sin_cache=cache),
        lambda pos: fused_store_decode_attention(q, k, v, cache, ck, cv, base, live, ev, pos, num_kv_heads=Hk,
                                                 alpha_scale=100.0, alpha_offset=5.0),
    ):
        call(ok)
        assert _lib.read_device_status(dev) == 0
        call(bad)
        assert _lib.read_device_status(dev) & 2, "FDMS_DEV_BAD_INDEX expected"
        _lib.status_word(dev).zero_()
        call(torch.tensor([-1, 3], device=dev))
        assert _lib.read_device_status(dev) & 2
        _lib.status_word(dev).zero_()


def test_peer_allreduce_kernel_with_a_staged_peer_and_with_a_silent_one(dev):
    """The one-shot all-reduce kernel on one GPU.  (1) The peer is staged by the host: its input already sits
    in rank 0's region, every 32-bit word next to the epoch of the call, so the kernel finds it at once and
    must return rank 0's input plus the peer's, for three dtypes and two consecutive calls (the two halves of
    the region); rank 0's own input must have been pushed into the peer's region in the same form.  (2) A
    peer that never pushes: the bounded wait runs out after about a second, the kernel raises
    FDMS_DEV_WAIT_TIMEOUT, leaves that peer out and returns; the context stays usable."""
    import time
    from fastdms_b200 import _lib
    lib = _lib.lib()
    max_bytes = 1 << 16
    nbytes = lib.fdms_allreduce_region_bytes(2, max_bytes)
    half = ((max_bytes + 255) // 256) * 256
    assert nbytes == 2 * 2 * 2 * half + 256
    g = torch.Generator(device=dev).manual_seed(1)
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        regions = [torch.zeros((nbytes,), dtype=torch.uint8, device=dev) for _ in range(2)]
        ptrs = torch.tensor([r.data_ptr() for r in regions], dtype=torch.int64)
        # [half][source rank][word index][word, epoch]
        slots = [r[: 2 * 2 * 2 * half].view(torch.int32).view(2, 2, half // 4, 2) for r in regions]
        n = 8 * 1024
        for call in (1, 2):
            x0 = torch.randn((n,), device=dev, generator=g).to(dtype)
            x1 = torch.randn((n,), device=dev, generator=g).to(dtype)
            words = n * x1.element_size() // 4
            slots[0][call & 1, 1, :words, 0] = x1.view(torch.int32)          # the peer's input, pushed into rank 0's region
            slots[0][call & 1, 1, :words, 1] = call
            out = torch.empty_like(x0)
            _lib.check(lib.fdms_allreduce_oneshot(ptrs.data_ptr(), 0, 2, max_bytes, x0.data_ptr(), out.data_ptr(), n,
                                                  _lib.dtype_code(dtype), _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev)))
            want = (x0.float() + x1.float()).to(dtype)
            assert torch.equal(out, want)
            assert torch.equal(slots[1][call & 1, 0, :words, 0].contiguous(), x0.view(torch.int32)), "rank 0 pushes its input to the peer"
            assert (slots[1][call & 1, 0, :words, 1] == call).all()
        assert _lib.read_device_status(dev) == 0
    # a silent peer
    regions = [torch.zeros((nbytes,), dtype=torch.uint8, device=dev) for _ in range(2)]
    ptrs = torch.tensor([r.data_ptr() for r in regions], dtype=torch.int64)
    x0 = torch.randn((4096,), device=dev, generator=g)
    out = torch.empty_like(x0)
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    _lib.check(lib.fdms_allreduce_oneshot(ptrs.data_ptr(), 0, 2, max_bytes, x0.data_ptr(), out.data_ptr(), 4096, _lib.F32,
                                          _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev)))
    torch.cuda.synchronize(dev)
    waited = time.perf_counter() - t0
    assert _lib.read_device_status(dev) & 1, "FDMS_DEV_WAIT_TIMEOUT expected"
    assert waited < 20.0
    assert torch.equal(out, x0)                      # the silent peer was left out
    assert torch.equal(torch.ones(4, device=dev) + 1, torch.full((4,), 2.0, device=dev))    # context still fine
    with pytest.raises(RuntimeError):
        _lib.check(lib.fdms_allreduce_oneshot(ptrs.data_ptr(), 0, 2, max_bytes, x0.data_ptr(), out.data_ptr(), 1 << 20, _lib.F32,
                                              None, _lib.stream_ptr(dev)))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,n,k,bias", [(8, 3072, 2048, True), (8, 2048, 2048, False), (8, 16384, 2048, False),
                                           (8, 2048, 8192, False), (1, 128256, 2048, False), (5, 6144, 4096, True),
                                           (3, 48, 2048, True), (8, 4096, 12288, True), (2, 1024, 8192, True), (8, 16, 4096, False)])
def test_decode_linear_kernel_matches_float32_reference(dev, dtype, rows, n, k, bias):
    """Weight-streaming linear layer for <= 8 rows against x @ W^T (+ b) in float32 (the reference
    calls F.linear, layers/linear.py:1044-1048): one rounding of the 16-bit output type."""
    from fastdms_b200.layers.linear import linear
    g = torch.Generator(device=dev).manual_seed(rows * 7 + n + k)
    x = torch.randn((rows, k), device=dev, generator=g).to(dtype)
    w = (torch.randn((n, k), device=dev, generator=g) * k ** -0.5).to(dtype)
    b = torch.randn((n,), device=dev, generator=g).to(dtype) if bias else None
    with torch.inference_mode():
        y = linear(x, w, b)
        # rows of a wider buffer (row stride != k)
        wide = torch.randn((rows, k + 64), device=dev, generator=g).to(dtype)
        y2 = linear(wide[:, 8:8 + k], w, b)
    ref = x.float() @ w.float().t() + (b.float() if bias else 0.0)
    ref2 = wide[:, 8:8 + k].float() @ w.float().t() + (b.float() if bias else 0.0)
    eps = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    assert y.shape == (rows, n) and y.dtype == dtype
    assert ((y.float() - ref).abs() <= eps * ref.abs() + 1e-3).all()
    assert ((y2.float() - ref2).abs() <= eps * ref2.abs() + 1e-3).all()
    # the library kernel is what ran: torch's own GEMM rounds an f32 accumulation too, so the two agree to one ulp
    t = torch.nn.functional.linear(x, w, b)
    assert ((y.float() - t.float()).abs() <= 2 * eps * ref.abs() + 2e-3).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,n,k,with_res", [(8, 3072, 2048, True), (8, 16384, 2048, True), (3, 6144, 4096, True),
                                               (8, 3072, 2048, False)])
def test_fused_norm_linear_matches_the_two_modules(dev, dtype, rows, n, k, with_res):
    """RMSNorm (+ residual add) fused in front of the decode linear kernel against the two separate
    launches: the new residual is bit-identical, the projection agrees to one rounding of the 16-bit
    type (the row statistics are summed in a different order)."""
    from fastdms_b200.layers.layernorm import RMSNorm
    from fastdms_b200.layers.linear import ReplicatedLinear, norm_linear
    import fastdms_b200.layers.linear as L
    g = torch.Generator(device=dev).manual_seed(rows + n + k)
    norm = RMSNorm(k, eps=1e-5).to(dev)
    norm.weight.data = (1.0 + 0.1 * torch.randn(k, device=dev, generator=g)).to(dtype)
    lin = ReplicatedLinear(k, n, bias=True).to(dev)
    lin.weight.data = (torch.randn((n, k), device=dev, generator=g) * k ** -0.5).to(dtype)
    lin.bias.data = torch.randn(n, device=dev, generator=g).to(dtype)
    x = torch.randn((rows, k), device=dev, generator=g).to(dtype)
    res = torch.randn((rows, k), device=dev, generator=g).to(dtype) if with_res else None
    saved = L._FUSE_NORM
    with torch.inference_mode():
        try:
            L._FUSE_NORM = True
            y, r = norm_linear(x, res, norm, lin)
            L._FUSE_NORM = False
            y0, r0 = norm_linear(x.clone(), None if res is None else res.clone(), norm, lin)
        finally:
            L._FUSE_NORM = saved
    assert torch.equal(r, r0 if with_res else x)
    xf = x.float() + (res.float() if with_res else 0.0)
    h = ((xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(dtype).float() * norm.weight.float()).to(dtype)
    ref = h.float() @ lin.weight.float().t() + lin.bias.float()
    eps = 2.0 ** -6 if dtype == torch.bfloat16 else 2.0 ** -9
    assert ((y.float() - ref).abs() <= eps * ref.abs() + 2e-2).all()
    assert ((y.float() - y0.float()).abs() <= eps * ref.abs() + 2e-2).all()


def test_page_pops_are_all_or_nothing_when_the_stack_runs_dry(dev):
    """160 spans ask for 1..12 pages each from a stack that holds about half of the total.  A span
    gets all of its pages or none; granted ids are distinct and disjoint from what is left on the
    stack; the counter equals initial - granted; after freeing, the stack is a permutation of every id."""
    from fastdms_b200 import _lib
    lib = _lib.lib()
    rng = np.random.default_rng(77)
    num_seqs, hk, max_pages = 20, 8, 12
    need_pages = rng.integers(1, max_pages + 1, size=(num_seqs, hk)).astype(np.int32)
    total = int(need_pages.sum()) // 2
    rows = torch.from_numpy((need_pages * 16 - rng.integers(0, 16, size=need_pages.shape)).astype(np.int32)).to(dev)
    bt = torch.full((num_seqs, hk, max_pages), -1, dtype=torch.int32, device=dev)
    stack = torch.from_numpy(rng.permutation(total).astype(np.int32)).to(dev)
    count = torch.tensor([total], dtype=torch.int32, device=dev)
    status = _lib.status_word(dev)
    for _ in range(2):                                   # second round: the same pops on the refilled stack
        with torch.cuda.device(dev):
            _lib.check(lib.fdms_alloc_pages(rows.data_ptr(), bt.data_ptr(), bt.stride(0), bt.stride(1), max_pages, None,
                                            stack.data_ptr(), count.data_ptr(), num_seqs, hk, status.data_ptr(),
                                            _lib.stream_ptr(dev)))
        assert _lib.read_device_status(dev) == _lib.DEV_BAD_INDEX      # some spans must have been refused
        got = bt.cpu().numpy()
        left = int(count.item())
        granted = []
        for s in range(num_seqs):
            for h in range(hk):
                n = int(need_pages[s, h])
                ids = got[s, h, :n]
                assert (ids >= 0).all() or (ids == -1).all(), "a span was given part of its pages"
                assert (got[s, h, n:] == -1).all()
                if ids[0] >= 0:
                    granted.extend(ids.tolist())
        assert 0 <= left and left + len(granted) == total, "pages were lost or invented"
        remaining = stack.cpu().numpy()[:left].tolist()
        assert sorted(granted + remaining) == list(range(total)), "a page is owned twice or leaked"
        live = torch.zeros((num_seqs, hk), dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.fdms_free_pages(live.data_ptr(), live.stride(0), bt.data_ptr(), bt.stride(0), bt.stride(1), max_pages,
                                           None, stack.data_ptr(), count.data_ptr(), total, num_seqs, hk, status.data_ptr(),
                                           _lib.stream_ptr(dev)))
        assert int(count.item()) == total and sorted(stack.cpu().numpy().tolist()) == list(range(total))
        assert (bt.cpu().numpy() == -1).all()


def test_split_k_workspace_survives_growth_of_the_batch(dev, monkeypatch):
    """A graph captured for a small batch keeps the raw address of the split-K workspace.  Asking for
    a workspace for a larger problem afterwards must not move or free it: the replay after other
    allocations still equals the eager result."""
    from fastdms_b200 import _lib
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    monkeypatch.setenv("FDMS_ATTN_SPLITS", "2")
    monkeypatch.setenv("FDMS_ATTN_CHUNKS", "3")          # several clusters per span: the workspace is used
    rng = np.random.default_rng(3)
    q, kq, vq, base, live, bt, ks, vs = _config2_case(rng, 2, 2, 4, 64, 700, 100, 9, True)
    qb = torch.from_numpy(q).to(dev).to(torch.bfloat16)
    args = (qb, t_fp8(kq, dev), t_fp8(vq, dev), torch.from_numpy(base).to(dev), torch.from_numpy(live).to(dev))
    kw = dict(block_tables=torch.from_numpy(bt).to(dev), k_scale=torch.from_numpy(ks).to(dev), v_scale=torch.from_numpy(vs).to(dev))
    out = torch.empty_like(qb)
    want = compact_decode_attention(*args, **kw).clone()
    before = _lib.attn_workspace(dev, 2, 2, 64).data_ptr()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        compact_decode_attention(*args, out=out, **kw)
    # a larger batch and a larger head_dim, then unrelated allocations that would reuse a freed block
    assert _lib.attn_workspace(dev, 4096, 8, 128).data_ptr() == before
    assert _lib.attn_workspace(dev, 9, 8, 256).data_ptr() == before
    junk = [torch.full((1 << 20,), 7.0, device=dev) for _ in range(8)]
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize(dev)
        assert torch.equal(out, want)
    del junk


def _lar_layout(n, k):
    """(k-splits, tiles per CTA, CTAs) the fused linear + all-reduce kernel uses for a [n, k] shard."""
    steps, ks = k // 256, 1
    while ks * 2 <= 8 and ks * 2 <= steps:
        ks *= 2
    tpc = 8 // ks
    return ks, tpc, -(-(n // 16) // tpc)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,n,k,bias,world", [(8, 4096, 2048, False, 2), (8, 4096, 512, True, 8), (3, 4096, 1536, True, 4),
                                                  (8, 2064, 256, False, 3), (1, 2048, 6144, True, 2)])
def test_fused_linear_allreduce_with_a_staged_peer(dev, dtype, rows, n, k, bias, world):
    """The row-parallel linear layer fused with its all-reduce, run as rank 0 of `world` on one GPU.  The peers
    are staged by the host: their float32 partial tiles already sit in rank 0's region, every value next to the
    epoch of the call, so the kernel finds them at once.  Result = this rank's x W^T + the staged partials
    (+ bias), compared with a float32 computation; two calls in a row use the two halves of the region; rank
    0's own partial must have been pushed into every peer's region, value by value with the call's epoch."""
    from fastdms_b200 import _lib
    lib = _lib.lib()
    MAXC, SLOT = 512, 1024
    ks, tpc, ctas = _lar_layout(n, k)
    nbytes = lib.fdms_linear_allreduce_region_bytes(world)
    assert nbytes == 2 * world * MAXC * (2 * SLOT) * 4 + MAXC * 4
    regions = [torch.zeros((nbytes,), dtype=torch.uint8, device=dev) for _ in range(world)]
    ptrs = torch.tensor([r.data_ptr() for r in regions], dtype=torch.int64)
    slot_bytes = 2 * world * MAXC * (2 * SLOT) * 4
    # [parity][source][cta][value index][value bits, epoch]
    slots = [r[:slot_bytes].view(torch.int32).view(2, world, MAXC, SLOT, 2) for r in regions]
    g = torch.Generator(device=dev).manual_seed(rows + n + k)
    w = (torch.randn((n, k), device=dev, generator=g) * k ** -0.5).to(dtype)
    b = torch.randn((n,), device=dev, generator=g).to(dtype) if bias else None
    npad = ctas * tpc * 16

    def to_slots(partial):                      # [rows, n] float32 -> [ctas, tpc * 128] in the kernel's tile layout
        full = torch.zeros((8, npad), device=dev)
        full[:rows, :n] = partial
        return full.t().reshape(ctas, tpc * 128)

    for call in (1, 2):
        x = torch.randn((rows, k), device=dev, generator=g).to(dtype)
        peers = [torch.randn((rows, n), device=dev, generator=g) for _ in range(world - 1)]
        for r, peer in enumerate(peers, start=1):
            slots[0][call & 1, r, :ctas, : tpc * 128, 0] = to_slots(peer).contiguous().view(torch.int32)
            slots[0][call & 1, r, :ctas, : tpc * 128, 1] = call
        y = torch.full((rows, n), float("nan"), device=dev, dtype=dtype)
        _lib.check(lib.fdms_linear_decode_allreduce(
            x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _lib.ptr(b), y.data_ptr(), y.stride(0),
            _lib.dtype_code(dtype), rows, n, k, ptrs.data_ptr(), 0, world, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev)))
        own = x.float() @ w.float().t()
        ref = own + sum(peers) + (b.float() if bias else 0.0)
        tol = 2.0 ** -7 * float(ref.abs().max())
        assert torch.isfinite(y.float()).all() and float((y.float() - ref).abs().max()) <= tol
        # this rank's partial went to every peer's region, every value with the epoch of this call
        for r in range(1, world):
            pushed = slots[r][call & 1, 0, :ctas, : tpc * 128, 0].contiguous().view(torch.float32)
            assert float((pushed - to_slots(own)).abs().max()) <= 2e-3 * float(own.abs().max()) + 1e-5
            assert (slots[r][call & 1, 0, :ctas, : tpc * 128, 1] == call).all()
    assert _lib.read_device_status(dev) == 0


def test_fused_linear_allreduce_leaves_a_silent_peer_out(dev):
    """A peer that never pushes its values: the bounded waits run out after about a second, the kernel
    raises FDMS_DEV_WAIT_TIMEOUT, sums what it has (its own partial) and returns; the context stays usable."""
    import time
    from fastdms_b200 import _lib
    lib = _lib.lib()
    rows, n, k = 4, 1024, 2048
    nbytes = lib.fdms_linear_allreduce_region_bytes(2)
    regions = [torch.zeros((nbytes,), dtype=torch.uint8, device=dev) for _ in range(2)]
    ptrs = torch.tensor([r.data_ptr() for r in regions], dtype=torch.int64)
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn((rows, k), device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn((n, k), device=dev, generator=g) * k ** -0.5).to(torch.bfloat16)
    y = torch.empty((rows, n), device=dev, dtype=torch.bfloat16)
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    _lib.check(lib.fdms_linear_decode_allreduce(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), None, y.data_ptr(), y.stride(0), _lib.BF16, rows, n, k,
        ptrs.data_ptr(), 0, 2, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev)))
    torch.cuda.synchronize(dev)
    assert time.perf_counter() - t0 < 30.0
    assert _lib.read_device_status(dev) & _lib.DEV_WAIT_TIMEOUT, "FDMS_DEV_WAIT_TIMEOUT expected"
    ref = x.float() @ w.float().t()
    assert float((y.float() - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max())
    assert torch.equal(torch.ones(4, device=dev) + 1, torch.full((4,), 2.0, device=dev))
    with pytest.raises(ValueError):
        lib_rc = lib.fdms_linear_decode_allreduce(
            x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), None, y.data_ptr(), y.stride(0), _lib.BF16, rows, n, k,
            ptrs.data_ptr(), 2, 2, None, _lib.stream_ptr(dev))
        _lib.check(lib_rc)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,n,k,bias", [(8, 3072, 2048, True), (8, 2048, 8192, False), (3, 16384, 2048, False),
                                            (1, 128256, 2048, False), (8, 4096, 4096, True)])
def test_fp8_weight_decode_linear_matches_float32_reference(dev, dtype, rows, n, k, bias):
    """`fdms_linear_decode_fp8`: e4m3 weights with one scale per output column, 16-bit activations.  The
    kernel's products are exact (FP8 bytes and activations both converted exactly to f16) and it
    accumulates in float32, so the result is the float32 product with the dequantised weights rounded
    once to the activation dtype."""
    from fastdms_b200 import _lib
    lib = _lib.lib()
    g = torch.Generator(device=dev).manual_seed(rows + n + k)
    w = torch.randn((n, k), device=dev, generator=g) * k ** -0.5
    scale = (w.abs().amax(dim=1) / 448.0).float().contiguous()
    w8 = (w / scale[:, None]).to(torch.float8_e4m3fn).contiguous()
    x = torch.randn((rows, k), device=dev, generator=g).to(dtype)
    b = torch.randn((n,), device=dev, generator=g).to(dtype) if bias else None
    y = torch.full((rows, n), float("nan"), device=dev, dtype=dtype)
    _lib.check(lib.fdms_linear_decode_fp8(x.data_ptr(), x.stride(0), w8.data_ptr(), w8.stride(0), scale.data_ptr(), _lib.ptr(b),
                                          y.data_ptr(), y.stride(0), _lib.dtype_code(dtype), rows, n, k, _lib.stream_ptr(dev)))
    ref = (x.float() @ w8.float().t()) * scale[None, :] + (b.float() if bias else 0.0)
    err = (y.float() - ref).abs()
    ulp = ref.abs() * (2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11) + 1e-4
    assert torch.isfinite(y.float()).all() and bool((err <= 1.01 * ulp).all()), float((err / ulp).max())

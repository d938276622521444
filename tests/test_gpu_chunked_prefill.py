"""GPU tests of chunked prefill: the prefill-tail attention kernel (`fdms_prefix_attention`) against
the numpy oracle's `chunk_attention`, the appending prefill pack against `chunked_prefill_state`, and
the engine prefilling a prompt in chunks.  Chunked prefill is an extension (the reference prefills
in one dense pass), so these compare with the restated definition, not with reference vectors."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import compact_dms as O
from oracle.dtypes import bf16_bits_to_f32, decode_e4m3

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-2      # max-abs, FP8 pools / bf16 activations vs float32 oracle


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


def n_bf16(t):
    return bf16_bits_to_f32(t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16))


def dense_causal(q, k, v, cu, scale):
    """The caller's part of a chunk: causal attention of every sequence over its own chunk tokens in
    float32 torch ops; returns (out [T,Hq,D] in q's dtype, natural-log lse [Hq,T] float32)."""
    T, Hq, D = q.shape
    G = Hq // k.shape[1]
    out = torch.empty_like(q)
    lse = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
    for i in range(len(cu) - 1):
        a, b = cu[i], cu[i + 1]
        if a == b:
            continue
        qq = q[a:b].float().transpose(0, 1)                                   # [Hq, t, D]
        kk = k[a:b].float().repeat_interleave(G, dim=1).transpose(0, 1)
        vv = v[a:b].float().repeat_interleave(G, dim=1).transpose(0, 1)
        s = (qq @ kk.transpose(1, 2)) * scale
        s = s.masked_fill(~torch.tril(torch.ones(b - a, b - a, dtype=torch.bool, device=q.device)), float("-inf"))
        lse[:, a:b] = torch.logsumexp(s, dim=-1)
        out[a:b] = (torch.softmax(s, dim=-1) @ vv).transpose(0, 1).to(q.dtype)
    return out, lse


@pytest.mark.parametrize("D,Hq,Hk", [(64, 32, 8), (128, 32, 8), (64, 4, 4), (64, 16, 2), (128, 6, 2)])
@pytest.mark.parametrize("paged", [False, True])
def test_prefix_attention_matches_oracle(dev, D, Hq, Hk, paged):
    """Ragged chunk batch (lengths not multiples of 16, one sequence without any prefix), spans of
    0..~300 rows, FP8 pools with per-head scales: merged result and log-sum-exp against the oracle."""
    from fastdms_b200.layers.compact_attention import compact_prefix_attention
    g = torch.Generator(device=dev).manual_seed(D * 100 + Hq + (7 if paged else 0))
    lens = [37, 130, 1, 64]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T, B = cu[-1], len(lens)
    q = torch.randn((T, Hq, D), device=dev, generator=g).to(torch.bfloat16)
    k = torch.randn((T, Hk, D), device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn((T, Hk, D), device=dev, generator=g).to(torch.bfloat16)
    live = torch.randint(1, 300, (B, Hk), device=dev, generator=g, dtype=torch.int32)
    live[2] = 0                                                                 # a first chunk: nothing stored yet
    live[0, 0] = 64
    live[1, 1] = 1
    pages = (live + 15) // 16
    total_pages = int(pages.sum().item()) + 4
    pool_rows = total_pages * 16
    ck = torch.randint(0, 256, (pool_rows, D), device=dev, generator=g, dtype=torch.uint8)
    cv = torch.randint(0, 256, (pool_rows, D), device=dev, generator=g, dtype=torch.uint8)
    ck[(ck & 0x7f) == 0x7f] = 0x30                                              # no NaN encodings
    cv[(cv & 0x7f) == 0x7f] = 0x30
    k_scale = (torch.rand(Hk, device=dev, generator=g) * 0.01 + 0.002).float()
    v_scale = (torch.rand(Hk, device=dev, generator=g) * 0.01 + 0.002).float()
    perm = torch.randperm(total_pages, device=dev, generator=g).to(torch.int32)
    bt = torch.full((B, Hk, int(pages.max().item())), -1, device=dev, dtype=torch.int32)
    base = torch.zeros((B, Hk), device=dev, dtype=torch.int32)
    off = 0
    for b in range(B):
        for h in range(Hk):
            c = int(pages[b, h])
            bt[b, h, :c] = perm[off:off + c]
            base[b, h] = off * 16
            off += c
    scale = D ** -0.5
    dense, lse_d = dense_causal(q, k, v, cu, scale)
    out = dense.clone()
    lse_out = torch.zeros_like(lse_d)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    compact_prefix_attention(q, ck.view(torch.float8_e4m3fn), cv.view(torch.float8_e4m3fn),
                             None if paged else base, live, cu_t, max(lens), out, lse_d, scale,
                             block_tables=bt if paged else None, k_scale=k_scale, v_scale=v_scale, lse_out=lse_out)
    torch.cuda.synchronize(dev)
    ckn, cvn = decode_e4m3(ck.cpu().numpy()), decode_e4m3(cv.cpu().numpy())
    qn, kn, vn = n_bf16(q), n_bf16(k), n_bf16(v)
    got, got_lse = n_bf16(out), lse_out.cpu().numpy()
    ksn, vsn = k_scale.cpu().numpy(), v_scale.cpu().numpy()
    for b in range(B):
        a, e = cu[b], cu[b + 1]
        pk, pv = [], []
        for h in range(Hk):
            n = int(live[b, h])
            btrow = bt[b, h].cpu().numpy() if paged else None
            pk.append(O.gather_span(ckn, int(base[b, h]), n, btrow) * ksn[h])
            pv.append(O.gather_span(cvn, int(base[b, h]), n, btrow) * vsn[h])
        want, _, want_lse = O.chunk_attention(qn[a:e], kn[a:e], vn[a:e], pk, pv, scale)
        if int(live[b].max()) == 0:
            assert torch.equal(out[a:e], dense[a:e])                            # untouched
            continue
        assert np.abs(got[a:e] - want).max() <= ATTN_TOL
        assert np.abs(got_lse[:, a:e] - want_lse).max() <= ATTN_TOL
    # span rows only (no dense part): equals decode attention of each query over the span
    alone = torch.empty_like(q)
    compact_prefix_attention(q, ck.view(torch.float8_e4m3fn), cv.view(torch.float8_e4m3fn),
                             None if paged else base, live, cu_t, max(lens), alone, None, scale,
                             block_tables=bt if paged else None, k_scale=k_scale, v_scale=v_scale)
    b = 1
    a, e = cu[b], cu[b + 1]
    want = O.decode_attention(qn[a:e], ckn, cvn, np.repeat(base[b:b + 1].cpu().numpy(), e - a, 0),
                              np.repeat(live[b:b + 1].cpu().numpy(), e - a, 0), scale, k_scale=ksn, v_scale=vsn,
                              block_tables=np.repeat(bt[b:b + 1].cpu().numpy(), e - a, 0) if paged else None)
    assert np.abs(n_bf16(alone[a:e]) - want).max() <= ATTN_TOL


def test_prefix_attention_wide_pools_and_f16(dev):
    """bf16 pools (the staging path that converts element-wise) and f16 activations."""
    from fastdms_b200.layers.compact_attention import compact_prefix_attention
    g = torch.Generator(device=dev).manual_seed(5)
    T, Hq, Hk, D = 50, 8, 2, 64
    q = torch.randn((T, Hq, D), device=dev, generator=g).to(torch.float16)
    k = torch.randn((T, Hk, D), device=dev, generator=g).to(torch.float16)
    v = torch.randn((T, Hk, D), device=dev, generator=g).to(torch.float16)
    ck = torch.randn((400, D), device=dev, generator=g).to(torch.bfloat16)
    cv = torch.randn((400, D), device=dev, generator=g).to(torch.bfloat16)
    base = torch.tensor([[0, 200]], device=dev, dtype=torch.int32)
    live = torch.tensor([[150, 77]], device=dev, dtype=torch.int32)
    scale = D ** -0.5
    dense, lse_d = dense_causal(q, k, v, [0, T], scale)
    out = dense.clone()
    compact_prefix_attention(q, ck, cv, base, live, torch.tensor([0, T], dtype=torch.int32), T, out, lse_d, scale)
    ckn, cvn = n_bf16(ck), n_bf16(cv)
    pk = [ckn[0:150], ckn[200:277]]
    pv = [cvn[0:150], cvn[200:277]]
    want, _, _ = O.chunk_attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), pk, pv, scale)
    assert np.abs(out.float().cpu().numpy() - want).max() <= ATTN_TOL


def _mgr(dev, **kw):
    from fastdms_b200.engine.compact_kv import CompactKVManager
    return CompactKVManager(device=dev, **kw)


def _seq(tokens, max_tokens):
    from fastdms_b200.engine.sequence import Sequence
    from fastdms_b200.sampling_params import SamplingParams
    return Sequence(list(tokens), SamplingParams(max_tokens=max_tokens))


def _logical_state(m, seq, paged):
    """(live [Hk], positions, evict bits, K bytes, V bytes in logical order) of layer 0 of one sequence."""
    st = m.seq_states[seq.seq_id]
    live = st.live_counts[0].cpu().numpy()
    ck = m.compact_k_per_layer[0].view(torch.uint8).cpu().numpy()
    cv = m.compact_v_per_layer[0].view(torch.uint8).cpu().numpy()
    ri = None if m.layer_major_row_index is None else m.layer_major_row_index[0, st.active_slot].cpu().numpy()
    out = []
    for h in range(m.num_kv_heads):
        n = int(live[h])
        base = 0 if paged else int(st.base_offsets[0, h])
        bt = m.block_tables[0, st.active_slot, h].cpu().numpy() if paged else None
        phys = O.gather_span(np.arange(m.capacity_tokens), base, n, bt)
        idx = np.arange(n) if ri is None else ri[h, :n]
        out.append((n, st.token_positions[0, h, :n].cpu().numpy(), st.evict_mask[0, h, :n].cpu().numpy(),
                    ck[phys[idx]], cv[phys[idx]]))
    return out


@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("row_index", [False, True])
@pytest.mark.parametrize("chunk", [64, 250, 699])
def test_chunked_pack_leaves_the_one_pass_state(dev, paged, row_index, chunk):
    """Packing a prompt chunk by chunk (expire with the chunk's last position, then append) leaves
    exactly what the one-pass pack leaves: compact lengths, positions, evict bits and the FP8 rows in
    logical order are identical, and equal to the oracle's chunked_prefill_state."""
    rng = np.random.default_rng(chunk + 2 * int(paged) + int(row_index))
    T, Hk, D, W, C = 700, 3, 64, 16, 1024
    ev = rng.random((T, Hk)) < 0.8
    g = torch.Generator(device=dev).manual_seed(chunk)
    k = torch.randn((T, Hk, D), device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn((T, Hk, D), device=dev, generator=g).to(torch.bfloat16)
    evt = torch.from_numpy(ev).to(dev)
    kw = dict(num_layers=1, num_kv_heads=Hk, capacity_tokens=4 * C, max_model_len=C, head_dim=D,
              compact_dtype=torch.float8_e4m3fn, max_active_seqs=2, paged=paged, row_indirection=row_index)
    one, seq1 = _mgr(dev, **kw), _seq(range(T), 4)
    one.allocate(seq1)
    one.streaming_pack_layer(layer_id=0, k=k, v=v, evict_mask=evt, cu_seqlens_q=torch.tensor([0, T], dtype=torch.int32),
                             seq_ids=[seq1.seq_id], window_size=W)
    many, seq2 = _mgr(dev, **kw), _seq(range(T), 4)
    many.allocate(seq2)
    for a in range(0, T, chunk):
        e = min(T, a + chunk)
        many.streaming_pack_layer(layer_id=0, k=k[a:e], v=v[a:e], evict_mask=evt[a:e],
                                  cu_seqlens_q=torch.tensor([0, e - a], dtype=torch.int32), seq_ids=[seq2.seq_id],
                                  window_size=W, chunk_starts=[a], remaining=[T - e])
    want, got = _logical_state(one, seq1, paged), _logical_state(many, seq2, paged)
    for h in range(Hk):
        assert got[h][0] == want[h][0], "compact lengths differ"
        assert np.array_equal(got[h][1], O.chunked_prefill_state(ev[:, h], W, chunk))
        for x, y in zip(got[h][1:], want[h][1:]):
            assert np.array_equal(x, y)
    if paged:
        many.free(seq2.seq_id)
        assert many.free_page_counts.tolist() == [many.pages_per_layer]


def _tiny_engine(dev, chunk, paged, dtype="bfloat16", kv="float8_e4m3fn"):
    from fastdms_b200.utils.shapes import SHAPES
    from fastdms_b200.engine.llm_engine import LLMEngine
    hf = dict(SHAPES["tiny"])
    hf.update(attention_bias=True, torch_dtype=dtype, max_position_embeddings=1024)
    return LLMEngine("synthetic-tiny", hf_config=hf, random_init_seed=3, device=dev, max_model_len=1024,
                     max_num_seqs=4, max_num_batched_tokens=2048, kv_cache_dtype=kv, compact_kv_paged=paged,
                     dms_window_size=16, prefill_chunk_size=chunk)


@pytest.mark.parametrize("paged", [False, True])
def test_engine_chunked_prefill(dev, paged):
    """The engine prefilling in chunks: layer 0 of the pool ends up exactly as after a one-pass
    prefill (its decisions depend on the embeddings only), generation runs to the end and the pool is
    returned clean.  A chunk size that covers every prompt reproduces the one-pass tokens exactly."""
    from fastdms_b200.sampling_params import SamplingParams
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (37, 300, 511)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)

    def run(chunk):
        eng = _tiny_engine(dev, chunk, paged)
        seqs = [eng.add_request(p, sp) for p in prompts]
        while any(s.num_completion_tokens == 0 for s in seqs):
            eng.step()
        m = eng.model_runner.compact_kv_manager
        state = [[(n, p.copy(), e.copy()) for n, p, e, _, _ in _logical_state(m, s, paged)] for s in seqs]
        while not eng.is_finished():
            eng.step()
        clean = (m.free_page_counts.tolist() == [m.pages_per_layer] * m.num_layers if paged
                 else m.free_ranges_per_layer == [[(0, m.capacity_tokens)]] * m.num_layers)
        return state, [s.completion_token_ids for s in seqs], clean

    base_state, base_tokens, clean0 = run(None)
    assert clean0
    same_state, same_tokens, _ = run(1024)                 # chunking on, every prompt fits one chunk
    assert same_tokens == base_tokens
    for chunk in (128, 100):
        state, tokens, clean = run(chunk)
        assert clean and all(len(t) == 8 for t in tokens)
        for s_got, s_want in zip(state, base_state):
            for (n1, p1, e1), (n0, p0, e0) in zip(s_got, s_want):
                # the decode token appended before the snapshot may be in both; compare the prompt part
                k1, k0 = p1 < 10_000, p0 < 10_000
                assert np.array_equal(p1[k1], p0[k0]) and np.array_equal(e1[k1], e0[k0])


def test_chunked_prefill_quality_guard_against_one_pass(dev):
    """Quality guard in the pattern of the reference's benchmarks/check_dms_compact_guard.py:195-249:
    a one-pass prefill run gives the token history, a chunked-prefill run (128-token chunks: later
    chunks see only the rows DMS retained from earlier ones) is forced onto that history, and the two
    runs' next-token distributions are compared step by step.  Chunking must not change what the model
    says: mean KL divergence and the number of greedy disagreements stay under the bounds below, and a
    chunk size that covers the prompt gives zero divergence.  (Measured on a B200: mean KLD 3.5e-3, max
    7.9e-3, 15 of 72 greedy choices differ -- a model with random weights has many near-ties, so the
    divergence is the meaningful figure and the bound on disagreements is loose.)"""
    import torch.nn.functional as F
    from fastdms_b200.sampling_params import SamplingParams
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (300, 511, 640)]
    steps = 24

    def run(chunk, forced=None):
        eng = _tiny_engine(dev, chunk, False, dtype="float32", kv="float32")
        sp = SamplingParams(temperature=0.0, max_tokens=steps + 1, ignore_eos=True)
        seqs = [eng.add_request(p, sp) for p in prompts]
        while any(s.num_completion_tokens == 0 for s in seqs):
            eng.step()
        used, logits = [[s.token_ids[-1] for s in seqs]], []
        if forced is not None:
            for s, t in zip(seqs, forced[0]):
                s.token_ids[-1] = t; s.last_token = t
        for step in range(steps):
            eng.step()
            logits.append(eng.model_runner.graphs[len(seqs)].logits.float().clone())
            used.append([s.token_ids[-1] for s in seqs])
            if forced is not None:
                for s, t in zip(seqs, forced[step + 1]):
                    s.token_ids[-1] = t; s.last_token = t
        while not eng.is_finished():
            eng.step()
        return used, torch.stack(logits)                         # [steps, seqs, vocab]

    ref_used, ref_logits = run(None)
    for chunk, max_kld, max_flips in ((1024, 1e-9, 0), (128, 0.02, 24)):
        used, logits = run(chunk, forced=ref_used)
        lp_ref, lp = F.log_softmax(ref_logits, dim=-1), F.log_softmax(logits, dim=-1)
        kld = (lp_ref.exp() * (lp_ref - lp)).sum(dim=-1)         # per (step, sequence)
        flips = sum(int(a != b) for ra, ca in zip(ref_used[1:], used[1:]) for a, b in zip(ra, ca))
        print(f"chunk {chunk}: mean KLD {float(kld.mean()):.3e}, max KLD {float(kld.max()):.3e}, greedy disagreements {flips}")
        assert torch.isfinite(kld).all()
        assert float(kld.mean()) <= max_kld, f"chunk {chunk}: mean KLD {float(kld.mean())}"
        assert flips <= max_flips, f"chunk {chunk}: {flips} greedy disagreements"

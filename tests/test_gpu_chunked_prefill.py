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

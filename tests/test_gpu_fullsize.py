"""Full-size checks on the benchmark workload (the op-level compact decode on Llama-3.2-1B shapes, as 16 layer pools: c=8, 32 q / 8 KV
heads, head_dim 64, about 1280 live rows per span, FP8 + per-head scales, permuted 16-row pages),
through properties that do not need the CPU oracle at this size:
  * attention against a float32 torch computation on the dequantised, gathered pool;
  * the fused store+attention launch against the two-kernel sequence (bit-identical);
  * after hundreds of decode steps with exact expiry: positions strictly increasing in logical order,
    nothing evict-marked left outside the window, the row index a permutation of the live rows, page
    accounting exact, no device status bit."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def workload():
    import bench
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    m, seqs, hp, g = bench.build_gpu_workload(dev, seed=77)
    bench.fill_activations(hp, g, dev)
    hp.set_positions([bench.CTX] * bench.B)
    return bench, dev, m, seqs, hp


def _torch_attention(q, ck, cv, bt, live, ks, vs, scale):
    """float32 reference on the GPU: q [B,Hq,D]; ck/cv uint8 views of the FP8 pool [rows, D]."""
    B, Hq, D = q.shape
    Hk = live.shape[1]
    G = Hq // Hk
    out = torch.empty((B, Hq, D), dtype=torch.float32, device=q.device)
    for b in range(B):
        for h in range(Hk):
            n = int(live[b, h])
            idx = torch.arange(n, device=q.device)
            rows = bt[b, h, idx // 16].long() * 16 + idx % 16
            k = ck[rows].view(torch.float8_e4m3fn).float() * ks[h]
            v = cv[rows].view(torch.float8_e4m3fn).float() * vs[h]
            s = (q[b, h * G:(h + 1) * G].float() @ k.T) * scale
            out[b, h * G:(h + 1) * G] = torch.softmax(s, dim=-1) @ v
    return out


def test_attention_full_size_against_float32(workload):
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    bench, dev, m, seqs, hp = workload
    slots = hp.slots_t.long()
    for l in (0, 7, 15):
        ks, vs = m.layer_scales(l)
        live = m.layer_major_live_counts[l, slots]
        bt = m.block_tables[l, slots]
        q = hp.q[l]
        got = compact_decode_attention(q, m.compact_k_per_layer[l], m.compact_v_per_layer[l],
                                       torch.zeros_like(live), live, block_tables=bt, k_scale=ks, v_scale=vs)
        want = _torch_attention(q, m.compact_k_per_layer[l].view(torch.uint8), m.compact_v_per_layer[l].view(torch.uint8),
                                bt, live.cpu().numpy(), ks, vs, bench.D ** -0.5)
        err = (got.float() - want).abs().max().item()
        assert err < 2e-2, f"layer {l}: max-abs error {err}"


def test_fused_launch_full_size_is_bit_identical(workload):
    from fastdms_b200.layers.compact_attention import (compact_decode_attention, fused_dms_rope_store_compact_decode,
                                                       fused_store_decode_attention)
    bench, dev, m, seqs, hp = workload
    slots = hp.slots_t.long()
    l = 3
    ks, vs = m.layer_scales(l)
    live = (m.layer_major_live_counts[l, slots] + 1).contiguous()          # the appended token is counted
    bt = m.block_tables[l, slots].clone()
    # the append may open a new page: give spans whose length was a multiple of 16 a spare page
    nfree = int(m.free_page_counts[l].item())
    assert nfree >= bt.shape[0] * bt.shape[1]
    spare = m.free_pages[l][nfree - bt.shape[0] * bt.shape[1]:nfree].view(bt.shape[:2])      # pages nobody uses
    need = ((live - 1) % 16 == 0)
    pg = ((live - 1) // 16).long()
    bt.scatter_(2, pg.unsqueeze(-1), torch.where(need, spare, bt.gather(2, pg.unsqueeze(-1)).squeeze(-1)).unsqueeze(-1))
    idx = live - 1
    slot = (bt.gather(2, (idx // 16).long().unsqueeze(-1)).squeeze(-1) * 16 + idx % 16).to(torch.int32)
    ck1, cv1 = m.compact_k_per_layer[l].clone(), m.compact_v_per_layer[l].clone()
    ck2, cv2 = ck1.clone(), cv1.clone()
    q1 = hp.q[l].clone()
    ev1 = torch.empty((bench.B, bench.HK), dtype=torch.bool, device=dev)
    ev2 = torch.empty_like(ev1)
    pos = torch.full((bench.B,), bench.CTX + 5, device=dev, dtype=torch.int64)
    fused_dms_rope_store_compact_decode(q1, hp.k[l].clone(), hp.v[l], hp.cos_sin_cache, ck1, cv1, slot, ev1, pos,
                                        num_kv_heads=bench.HK, alpha_scale=bench.ALPHA_SCALE, alpha_offset=bench.ALPHA_OFFSET,
                                        store_transient_k=False, k_scale=ks, v_scale=vs)
    want = compact_decode_attention(q1, ck1, cv1, torch.zeros_like(live), live, block_tables=bt, k_scale=ks, v_scale=vs)
    got = fused_store_decode_attention(hp.q[l], hp.k[l], hp.v[l], hp.cos_sin_cache, ck2, cv2, torch.zeros_like(live), live, ev2,
                                       pos, num_kv_heads=bench.HK, alpha_scale=bench.ALPHA_SCALE,
                                       alpha_offset=bench.ALPHA_OFFSET, block_tables=bt, k_scale=ks, v_scale=vs)
    assert torch.equal(ev1, ev2)
    assert torch.equal(ck1.view(torch.uint8), ck2.view(torch.uint8)) and torch.equal(cv1.view(torch.uint8), cv2.view(torch.uint8))
    assert torch.equal(got, want)


def test_invariants_after_many_decode_steps(workload):
    from fastdms_b200 import _lib
    bench, dev, m, seqs, hp = workload
    hp.capture()
    steps = 300
    for _ in range(steps):
        hp.step_device()
    torch.cuda.synchronize(dev)
    assert _lib.read_device_status(dev) == 0
    cur = int(hp.positions[0].item())                 # position the next step will use
    W = hp.window_size
    slots = hp.slots_t.long()
    live = m.layer_major_live_counts[:, slots].cpu().numpy()              # [L, B, Hk]
    pos = m.layer_major_token_positions[:, slots].cpu().numpy()           # [L, B, Hk, C]
    ev = m.layer_major_evict_mask[:, slots].cpu().numpy()
    ri = m.layer_major_row_index[:, slots].cpu().numpy()
    C = pos.shape[-1]
    ar = np.arange(C)
    valid = ar[None, None, None, :] < live[..., None]
    assert ((pos >= 0) == valid).all(), "positions are set exactly on the live prefix"
    d = np.diff(pos, axis=-1)
    assert (d[valid[..., 1:]] > 0).all(), "positions strictly increase in logical order"
    last_expiry_cur = cur - 1                                              # the last step expired with cur - 1
    stale = valid & ev & (pos < last_expiry_cur - W)
    assert not stale.any(), "an evict-marked token outside the window survived expiry"
    assert (pos.max(axis=-1) == cur - 1).all(), "the newest row is the token of the last step"
    # row index: permutation of [0, live) on the live prefix, identity behind it
    srt = np.sort(np.where(valid, ri, C + ar[None, None, None, :]), axis=-1)
    assert (np.where(valid, srt, 0) == np.where(valid, ar[None, None, None, :], 0)).all()
    assert (np.where(valid, 0, ri) == np.where(valid, 0, ar[None, None, None, :])).all()
    # page accounting: every span holds exactly ceil(live / 16) pages and the free stacks hold the rest
    bt = m.block_tables[:, slots].cpu().numpy()
    pages = (bt >= 0).sum(axis=-1)
    assert (pages == -(-live // 16)).all()
    assert (m.free_page_counts.cpu().numpy() == m.pages_per_layer - pages.sum(axis=(1, 2))).all()
    for l in (0, 9):
        used = bt[l][bt[l] >= 0]
        assert len(np.unique(used)) == len(used), "a page is mapped twice"
    # the eviction rate of the synthetic decision lane keeps the spans near their starting length
    assert abs(live.mean() - 1280) < 120

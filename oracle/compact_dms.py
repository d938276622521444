"""numpy restatement of the reference's compact-DMS decode path (test infrastructure only).

Each function cites the reference file:line it follows (paths inside the reference project).
Loops are written for clarity, not speed; the vectorised forms are used where the oracle is
timed as the CPU baseline.
"""
from __future__ import annotations

import numpy as np

from .dtypes import decode_e4m3, encode_e4m3, round_to


# --------------------------------------------------------------------------------------
# DMS decisions
# --------------------------------------------------------------------------------------

def dms_threshold(alpha_scale: float, alpha_offset: float) -> np.float32:
    """fastdms/engine/dms.py:225-226: the comparison constant, rounded once to float32."""
    return np.float32(float(alpha_offset) / float(alpha_scale))


def extract_decisions(q: np.ndarray, num_kv_heads: int, alpha_scale: float, alpha_offset: float):
    """fastdms/engine/dms.py:222-232 (CPU branch of extract_dms_eviction_decisions).

    q: float32 [T, Hq, D] (already rounded to its storage dtype).  Returns (q_clean, evict[T, Hk]).
    The decision value is channel D-1 of the first q head of every GQA group; it is zeroed.
    """
    q = np.array(q, dtype=np.float32, copy=True)
    T, Hq, D = q.shape
    G = Hq // num_kv_heads
    v = q[:, 0::G, D - 1].astype(np.float32)
    if alpha_scale > 0:
        evict = v > dms_threshold(alpha_scale, alpha_offset)
    else:
        evict = (np.float32(v * np.float32(alpha_scale)) - np.float32(alpha_offset)) > 0
    q[:, 0::G, D - 1] = 0.0
    return q, evict


def live_mask(evict: np.ndarray, current_position: int, window_size: int, positions=None) -> np.ndarray:
    """fastdms/engine/dms.py:235-262 build_dms_live_mask: live = ~evict | (cur - pos <= W)."""
    T = evict.shape[-1]
    pos = np.arange(T, dtype=np.int64) if positions is None else np.asarray(positions, dtype=np.int64)
    inside = (int(current_position) - pos) <= int(window_size)
    return (~evict.astype(bool)) | inside.reshape((1,) * (evict.ndim - 1) + (T,))


# --------------------------------------------------------------------------------------
# RoPE + append store (decode)
# --------------------------------------------------------------------------------------

def rope_neox(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """fastdms/layers/rotary_embedding.py:7-15 apply_rotary_emb, float32, no fused multiply-add.

    x [..., D]; cos/sin [..., D/2] broadcastable.  Result is float32 (caller rounds to dtype).
    """
    x = np.asarray(x, dtype=np.float32)
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    y1 = (x1 * cos).astype(np.float32) - (x2 * sin).astype(np.float32)
    y2 = (x2 * cos).astype(np.float32) + (x1 * sin).astype(np.float32)
    return np.concatenate([y1, y2], axis=-1).astype(np.float32)


def to_pool(x: np.ndarray, pool_dtype: str, scale: np.ndarray | float = 1.0) -> np.ndarray:
    """Cast float32 values into the compact pool's storage.  e4m3 -> bytes, else rounded float32.

    `scale` is the per-KV-head dequantisation scale (stored = x / scale); the reference has no
    scale, which is scale == 1 (fastdms/engine/compact_kv.py:1085-1087).
    """
    x = np.asarray(x, dtype=np.float32)
    if np.any(np.asarray(scale) != 1.0):
        x = (x / np.asarray(scale, dtype=np.float32)).astype(np.float32)
    if pool_dtype == "e4m3":
        return encode_e4m3(x)
    return round_to(x, pool_dtype)


def from_pool(raw: np.ndarray, pool_dtype: str, scale: np.ndarray | float = 1.0) -> np.ndarray:
    x = decode_e4m3(raw) if pool_dtype == "e4m3" else np.asarray(raw, dtype=np.float32)
    if np.any(np.asarray(scale) != 1.0):
        x = (x * np.asarray(scale, dtype=np.float32)).astype(np.float32)
    return x


def rope_store_decode(q, k, v, cos_sin_cache, compact_k, compact_v, slot_mapping, positions, *,
                      num_kv_heads, alpha_scale, alpha_offset, act_dtype, pool_dtype,
                      k_scale=None, v_scale=None):
    """Decode-step preprocess of one layer: extraction + RoPE + append store.

    Follows the reference's torch chain extract -> rotary_emb -> store_compact_kvcache
    (fastdms/models/llama.py:157-172, fastdms/layers/attention.py:103-111), which is what its fused
    kernel is tested against (fastdms/layers/compact_attention.py:67-209):
      * decision from q[b, h*G, D-1] BEFORE RoPE, lane zeroed;
      * RoPE in float32 at positions[b], result rounded to the activation dtype;
      * post-RoPE k and raw v cast into the pool at slot_mapping[b, h] (slot < 0 = skip).
    q [B,Hq,D], k/v [B,Hk,D] float32 values; cos_sin_cache [P, D] float32 (cos | sin);
    compact_k/v [slots, D] (uint8 for e4m3 else float32), modified in place.
    Returns (q_rot, k_rot, evict[B,Hk]).
    """
    B, Hq, D = q.shape
    h = D // 2
    q_clean, evict = extract_decisions(q, num_kv_heads, alpha_scale, alpha_offset)
    pos = np.asarray(positions, dtype=np.int64)
    cos = cos_sin_cache[pos, :h][:, None, :]
    sin = cos_sin_cache[pos, h:][:, None, :]
    q_rot = round_to(rope_neox(q_clean, cos, sin), act_dtype)
    k_rot = round_to(rope_neox(k, cos, sin), act_dtype)
    ks = np.ones(num_kv_heads, np.float32) if k_scale is None else np.asarray(k_scale, np.float32)
    vs = np.ones(num_kv_heads, np.float32) if v_scale is None else np.asarray(v_scale, np.float32)
    for b in range(B):
        for hh in range(num_kv_heads):
            s = int(slot_mapping[b, hh])
            if s < 0:
                continue
            compact_k[s] = to_pool(k_rot[b, hh], pool_dtype, ks[hh])
            compact_v[s] = to_pool(np.asarray(v[b, hh], np.float32), pool_dtype, vs[hh])
    return q_rot, k_rot, evict


# --------------------------------------------------------------------------------------
# Span allocator (host logic of the manager)
# --------------------------------------------------------------------------------------

class FirstFit:
    """fastdms/engine/compact_kv.py:705-737 _alloc_range/_free_range: first-fit over a sorted,
    coalesced free list of (start, length)."""

    def __init__(self, capacity: int):
        self.free = [(0, int(capacity))]

    def alloc(self, length: int) -> int:
        for i, (s, n) in enumerate(self.free):
            if n < length:
                continue
            if n == length:
                self.free.pop(i)
            else:
                self.free[i] = (s + length, n - length)
            return s
        raise RuntimeError(f"compact KV capacity exhausted: requested {length}")

    def release(self, start: int, length: int) -> None:
        if length <= 0:
            return
        self.free.append((int(start), int(length)))
        self.free.sort()
        merged: list[tuple[int, int]] = []
        for s, n in self.free:
            if merged and s <= merged[-1][0] + merged[-1][1]:
                ps, pn = merged[-1]
                merged[-1] = (ps, max(ps + pn, s + n) - ps)
            else:
                merged.append((s, n))
        self.free = merged


def span_sizes(live_per_head, decode_headroom: int, max_capacity: int):
    """fastdms/engine/compact_kv.py:836-843: reservation of one (layer, seq): per head
    min(live + headroom, C), at least 1."""
    return [max(min(int(n) + int(decode_headroom), int(max_capacity)), 1) for n in live_per_head]


# --------------------------------------------------------------------------------------
# Prefill pack
# --------------------------------------------------------------------------------------

def pack_keep(evict: np.ndarray, window_size: int) -> np.ndarray:
    """fastdms/engine/compact_kv.py:1011-1014: keep = ~evict | (t >= max(0, T-1-W)); evict [T,Hk]."""
    T = evict.shape[0]
    thr = max(0, T - 1 - int(window_size))
    return (~evict.astype(bool)) | (np.arange(T) >= thr)[:, None]


def pack_prefill_seq(k, v, evict, window_size, base_offsets, compact_k, compact_v,
                     token_positions, evict_mask, pool_dtype, k_scale=None, v_scale=None):
    """fastdms/engine/compact_kv.py:1030-1099 (torch path of streaming_pack_layer, one sequence,
    one layer).  k/v [T,Hk,D] float32 values (post-RoPE k, raw v); evict [T,Hk] bool;
    base_offsets [Hk]; token_positions [Hk,C] int32 and evict_mask [Hk,C] bool are reset and
    refilled; compact_k/v written at base[h] + rank.  Returns live counts [Hk] int32."""
    T, Hk, D = k.shape
    keep = pack_keep(evict, window_size)
    token_positions[...] = -1
    evict_mask[...] = False
    live = keep.sum(axis=0).astype(np.int32)
    ks = np.ones(Hk, np.float32) if k_scale is None else np.asarray(k_scale, np.float32)
    vs = np.ones(Hk, np.float32) if v_scale is None else np.asarray(v_scale, np.float32)
    for h in range(Hk):
        idx = np.nonzero(keep[:, h])[0]
        n = idx.size
        if n == 0:
            continue
        b = int(base_offsets[h])
        compact_k[b:b + n] = to_pool(k[idx, h], pool_dtype, ks[h])
        compact_v[b:b + n] = to_pool(v[idx, h], pool_dtype, vs[h])
        token_positions[h, :n] = idx.astype(np.int32)
        evict_mask[h, :n] = evict[idx, h]
    return live


def pack_compact_kv(k, v, keep):
    """fastdms/engine/compact_kv.py:1798-1850 pack_compact_kv (known-answer packer).
    k/v [B,T,Hk,D], keep [B,Hk,T] -> (compact_k, compact_v, base[B,Hk], live[B,Hk], positions)."""
    B, T, Hk, D = k.shape
    live = keep.sum(axis=-1).astype(np.int32)
    total = int(live.sum())
    ck = np.empty((total, D), k.dtype)
    cv = np.empty((total, D), v.dtype)
    base = np.empty((B, Hk), np.int32)
    pos = np.empty((total,), np.int32)
    cur = 0
    for b in range(B):
        for h in range(Hk):
            idx = np.nonzero(keep[b, h])[0]
            base[b, h] = cur
            n = idx.size
            ck[cur:cur + n] = k[b, idx, h]
            cv[cur:cur + n] = v[b, idx, h]
            pos[cur:cur + n] = idx
            cur += n
    return ck, cv, base, live, pos


# --------------------------------------------------------------------------------------
# Expiry (eviction + in-place compaction)
# --------------------------------------------------------------------------------------

def expire_span(pos_row, ev_row, live, cur, window, k_span, v_span, max_remove=None):
    """One (layer, seq, head) span.  Exact expiry, fastdms/engine/compact_kv.py:1270-1337
    (python path of apply_dms_evictions; the Triton twin is layers/compact_attention.py:690-773):
    keep slot i iff i < live and (not evict[i] or cur - pos[i] <= W); stable compaction of
    K/V rows, positions and evict bits to the front; tail reset to -1 / False.
    With max_remove=1 it is the steady-state variant (layers/compact_attention.py:776-858): only
    the FIRST slot with evict and pos < cur - W is dropped.
    Arrays are modified in place; returns the new live count."""
    n = int(live)
    idx = np.arange(n)
    p = pos_row[:n].astype(np.int64)
    e = ev_row[:n].astype(bool)
    if max_remove == 1:
        expired = e & (p < int(cur) - int(window))
        keep = np.ones(n, bool)
        hit = np.nonzero(expired)[0]
        if hit.size:
            keep[hit[0]] = False
    else:
        keep = (~e) | ((int(cur) - p) <= int(window))
    src = idx[keep]
    m = src.size
    k_span[:m] = k_span[src].copy()
    v_span[:m] = v_span[src].copy()
    newp = pos_row[src].copy()
    newe = ev_row[src].copy()
    pos_row[:m] = newp
    ev_row[:m] = newe
    pos_row[m:n] = -1
    ev_row[m:n] = False
    return m


def expire_layer(token_positions, evict_mask, live_counts, base_offsets, compact_k, compact_v,
                 current_positions, window, max_remove=None):
    """All spans of one layer: token_positions/evict_mask [B,Hk,C], live/base [B,Hk] (live updated
    in place), compact_k/v [slots,D], current_positions [B]."""
    B, Hk = live_counts.shape
    for b in range(B):
        for h in range(Hk):
            base = int(base_offsets[b, h])
            n = int(live_counts[b, h])
            if base < 0 or n <= 0:
                continue
            live_counts[b, h] = expire_span(
                token_positions[b, h], evict_mask[b, h], n, int(current_positions[b]), window,
                compact_k[base:base + n], compact_v[base:base + n], max_remove)


# --------------------------------------------------------------------------------------
# Decode metadata + decision recording
# --------------------------------------------------------------------------------------

def prepare_decode_metadata(base_offsets, live_counts):
    """fastdms/engine/compact_kv.py:1753-1760: slot = base + live, then live += 1 IN PLACE (the
    forward sees the incremented count).  base/live [L,B,Hk] int32.  Returns (base, live, slot)."""
    slot = (base_offsets + live_counts).astype(np.int32)
    live_counts += 1
    return base_offsets, live_counts, slot


def record_decisions(token_positions, evict_mask, live_counts, evict_all, positions):
    """fastdms/engine/compact_kv.py:1657-1690 / kernel :426-484: after the forward,
    token_positions[l,b,h,live-1] = positions[b]; evict_mask[l,b,h,live-1] = evict_all[l,b,h]."""
    L, B, Hk = live_counts.shape
    for l in range(L):
        for b in range(B):
            for h in range(Hk):
                i = int(live_counts[l, b, h]) - 1
                token_positions[l, b, h, i] = int(positions[b])
                evict_mask[l, b, h, i] = bool(evict_all[l, b, h])
    return int(np.asarray(evict_all).sum()), L * B * Hk


# --------------------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------------------

def gather_span(pool, base, live, block_table=None, page_size=16):
    """Logical rows [0, live) of a span.  block_table None: contiguous rows base..base+live
    (the reference layout, fastdms/engine/compact_kv.py:503-517); else logical row i lives at
    block_table[i // P] * P + i % P."""
    if block_table is None:
        return pool[base:base + live]
    i = np.arange(live)
    rows = np.asarray(block_table, dtype=np.int64)[i // page_size] * page_size + i % page_size
    return pool[rows]


def decode_attention(q, compact_k, compact_v, base_offsets, live_counts, scale=None, *,
                     pool_dtype="f32", out_dtype="f32", k_scale=None, v_scale=None,
                     block_tables=None, page_size=16):
    """fastdms/layers/compact_attention.py:1339-1364 compact_decode_attention_ref: for every
    (seq, q head): softmax(scale * K q) V over the span of its KV head, float32 math.
    q [B,Hq,D] float32 values; pools [slots,D]; base/live [B,Hk]; block_tables [B,Hk,maxpages]
    or None.  Returns float32 values rounded to out_dtype."""
    B, Hq, D = q.shape
    Hk = base_offsets.shape[1]
    G = Hq // Hk
    if scale is None:
        scale = D ** -0.5
    out = np.zeros((B, Hq, D), np.float32)
    for b in range(B):
        for h in range(Hk):
            n = int(live_counts[b, h])
            bt = None if block_tables is None else block_tables[b, h]
            kk = from_pool(gather_span(compact_k, int(base_offsets[b, h]), n, bt, page_size), pool_dtype,
                           1.0 if k_scale is None else k_scale[h])
            vv = from_pool(gather_span(compact_v, int(base_offsets[b, h]), n, bt, page_size), pool_dtype,
                           1.0 if v_scale is None else v_scale[h])
            for g in range(G):
                qh = h * G + g
                s = (kk @ q[b, qh].astype(np.float32)) * np.float32(scale)
                s = s - s.max()
                p = np.exp(s)
                p = p / p.sum()
                out[b, qh] = p @ vv
    return round_to(out, out_dtype)


def chunk_attention(q, k_chunk, v_chunk, prefix_k, prefix_v, scale=None):
    """Attention of one prefill chunk of one sequence under chunked prefill (an extension: the
    reference prefills densely in one pass, fastdms/layers/attention.py:85-92; parity unpinned).
    A query at chunk index i sees every prefix row (the rows its KV head's span held when the chunk
    started, already dequantised: prefix_k/v[h] float32 [n_h, D]) and chunk tokens 0..i.
    q [T,Hq,D], k_chunk/v_chunk [T,Hk,D] float32 values.  Returns (out [T,Hq,D],
    lse_dense [Hq,T], lse_total [Hq,T]) in float32; the log-sum-exps are natural-log, of the scaled scores."""
    T, Hq, D = q.shape
    Hk = k_chunk.shape[1]
    G = Hq // Hk
    if scale is None:
        scale = D ** -0.5
    out = np.zeros((T, Hq, D), np.float32)
    lse_d = np.zeros((Hq, T), np.float32)
    lse_t = np.zeros((Hq, T), np.float32)
    causal = np.tril(np.ones((T, T), bool))
    for h in range(Hk):
        pk, pv = np.asarray(prefix_k[h], np.float32), np.asarray(prefix_v[h], np.float32)
        n = pk.shape[0]
        for g in range(G):
            qh = h * G + g
            qq = q[:, qh].astype(np.float32)
            sd = (qq @ k_chunk[:, h].astype(np.float32).T) * np.float32(scale)
            sd = np.where(causal, sd, -np.inf)
            sp = (qq @ pk.T) * np.float32(scale) if n else np.zeros((T, 0), np.float32)
            s = np.concatenate([sp, sd], axis=1).astype(np.float64)
            m = s.max(axis=1, keepdims=True)
            e = np.exp(s - m)
            z = e.sum(axis=1, keepdims=True)
            vv = np.concatenate([pv, v_chunk[:, h].astype(np.float32)], axis=0).astype(np.float64)
            out[:, qh] = ((e / z) @ vv).astype(np.float32)
            lse_t[qh] = (m[:, 0] + np.log(z[:, 0])).astype(np.float32)
            md = sd.max(axis=1)
            lse_d[qh] = (md + np.log(np.exp(sd.astype(np.float64) - md[:, None]).sum(axis=1))).astype(np.float32)
    return out, lse_d, lse_t


def chunked_prefill_state(evict, window_size, chunk):
    """Logical contents (prompt positions, ascending) of one (layer, seq, head) span after the prompt
    was prefilled in chunks of `chunk` tokens: after every chunk ending at position e-1 the span is
    expired with cur = e-1 (rule of expire_span) and the chunk's tokens that pass pack_keep (chunk-
    local rule = the global rule at cur = e-1) are appended.  evict bool [T].  The final contents
    equal those of the one-pass pack, pack_keep(evict, window_size), for every chunk size."""
    T = len(evict)
    kept: list[int] = []
    for s0 in range(0, T, chunk):
        e = min(T, s0 + chunk)
        cur = e - 1
        kept = [t for t in kept if (not evict[t]) or cur - t <= window_size]
        kept += [t for t in range(s0, e) if (not evict[t]) or cur - t <= window_size]
    return np.asarray(kept, np.int64)


# --------------------------------------------------------------------------------------
# FP8 KV quantise / dequantise with a per-head scale
# --------------------------------------------------------------------------------------

def kv_quant(x, scale):
    """x [N,Hk,D] float32 values, scale [Hk] -> e4m3 bytes of x / scale[h] (scale 1 = the
    reference's bare cast, fastdms/engine/compact_kv.py:1085-1087)."""
    s = np.asarray(scale, np.float32)[None, :, None]
    return encode_e4m3((np.asarray(x, np.float32) / s).astype(np.float32))


def kv_dequant(raw, scale, out_dtype="f32"):
    s = np.asarray(scale, np.float32)[None, :, None]
    return round_to((decode_e4m3(raw) * s).astype(np.float32), out_dtype)


def absmax_scale(x):
    """Per-KV-head scale amax / 448 over a [N,Hk,D] tensor (1.0 for an all-zero head)."""
    a = np.abs(np.asarray(x, np.float32)).max(axis=(0, 2))
    return np.where(a > 0, a / np.float32(448.0), np.float32(1.0)).astype(np.float32)

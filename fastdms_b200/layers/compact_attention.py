"""Compact-DMS decode operators: same names, argument order and error behaviour as the reference's
`fastdms/layers/compact_attention.py`, bodies are calls into the sm_100a CUDA library.

Extensions over the reference (all optional keyword arguments, default = reference behaviour):
`block_tables` (16-row pages instead of contiguous spans), `k_scale` / `v_scale` (per-KV-head FP8
scales).  There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

import torch

from fastdms_b200 import _lib

PAGE_SIZE = 16


def compact_attention_splitk_enabled() -> bool:
    """The work-balanced split over the compact length is always on."""
    return True


def compact_attention_splitk_block_n() -> int:
    """Granularity of the split, in rows (one page)."""
    return PAGE_SIZE


def dms_fused_decode_preprocess_enabled() -> bool:
    return True


def dms_decode_store_transient_k_enabled() -> bool:
    """Whether the decode preprocess writes the rotated k back to the transient activation
    (reference: fastdms/layers/compact_attention.py:54-60, default off)."""
    import os

    return os.environ.get("FASTDMS_DMS_DECODE_STORE_TRANSIENT_K", "0").strip().lower() in {"1", "true", "yes", "on"}


def fused_store_attention_enabled() -> bool:
    """Whether decode layers with FP8 pools run decision + RoPE + store + attention as one launch
    (`FDMS_FUSED_STORE_ATTENTION`, default on; off gives the reference's two-kernel sequence)."""
    import os

    return os.environ.get("FDMS_FUSED_STORE_ATTENTION", "1").strip().lower() in {"1", "true", "yes", "on"}


def compact_attention_inline_q_rope_enabled() -> bool:
    return True


def _inner_contiguous(t: torch.Tensor, name: str) -> None:
    if t.stride(-1) != 1:
        raise ValueError(f"{name} must be contiguous in its last dimension")


def _scales(k_scale, v_scale, num_kv_heads, device):
    out = []
    for s in (k_scale, v_scale):
        if s is None:
            out.append(None)
            continue
        if s.shape != (num_kv_heads,) or s.dtype != torch.float32:
            raise ValueError(f"expected float32 scale of shape {(num_kv_heads,)}, got {tuple(s.shape)} {s.dtype}")
        out.append(s.to(device).contiguous())
    return out


def compact_decode_attention(
    q: torch.Tensor,
    compact_k: torch.Tensor,
    compact_v: torch.Tensor,
    base_offsets: torch.Tensor,
    live_counts: torch.Tensor,
    scale: float | None = None,
    max_live_count: int | None = None,
    block_n: int = 128,
    grouped: bool = True,
    q_rope_positions: torch.Tensor | None = None,
    q_rope_cos_sin_cache: torch.Tensor | None = None,
    *,
    block_tables: torch.Tensor | None = None,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    overlap_previous_kernel: bool = False,
) -> torch.Tensor:
    """Decode attention over compact K/V spans (reference: compact_attention.py:1116-1336).

    q [batch, q_heads, head_dim]; compact_k/compact_v [slots, head_dim]; base_offsets/live_counts
    [batch, kv_heads]; q head hq reads the span of KV head hq // group.  `max_live_count`,
    `block_n` and `grouped` are accepted for signature compatibility and do not change the result.
    `overlap_previous_kernel=True` lets the launch start while the preceding kernel of the stream
    still runs; only valid when that kernel writes nothing this call reads except q and the last
    live row of each span (the decode step's store kernel), see FDMS_ATTN_OVERLAP_PREVIOUS.
    """
    if q.ndim != 3:
        raise ValueError(f"expected q as [batch, q_heads, head_dim], got {q.shape}")
    if compact_k.shape != compact_v.shape:
        raise ValueError(f"compact k/v shape mismatch: {compact_k.shape} != {compact_v.shape}")
    if compact_k.ndim != 2:
        raise ValueError(f"expected compact K/V as [total_live, head_dim], got {compact_k.shape}")
    batch, num_q_heads, head_dim = q.shape
    if compact_k.shape[1] != head_dim:
        raise ValueError(f"K/V head_dim {compact_k.shape[1]} does not match q head_dim {head_dim}")
    if base_offsets.shape != live_counts.shape or base_offsets.ndim != 2:
        raise ValueError("base_offsets and live_counts must both be [batch, kv_heads]")
    if base_offsets.shape[0] != batch:
        raise ValueError(f"metadata batch {base_offsets.shape[0]} does not match q batch {batch}")
    num_kv_heads = base_offsets.shape[1]
    if num_q_heads % num_kv_heads != 0:
        raise ValueError(f"q_heads={num_q_heads} must be divisible by kv_heads={num_kv_heads}")
    if max_live_count is not None and max_live_count <= 0:
        raise ValueError("compact decode requires at least one live token per active KV head")
    if compact_k.dtype != compact_v.dtype:
        raise ValueError(f"compact k/v dtype mismatch: {compact_k.dtype} != {compact_v.dtype}")
    inline_q_rope = q_rope_positions is not None or q_rope_cos_sin_cache is not None
    if inline_q_rope:
        if q_rope_positions is None or q_rope_cos_sin_cache is None:
            raise ValueError("inline q RoPE requires both positions and cos_sin_cache")
        if head_dim % 2 != 0:
            raise ValueError(f"inline q RoPE requires even head_dim, got {head_dim}")
        if q_rope_positions.shape != (batch,):
            raise ValueError(f"expected q_rope_positions {(batch,)}, got {tuple(q_rope_positions.shape)}")
        if q_rope_cos_sin_cache.ndim != 3 or q_rope_cos_sin_cache.shape[2] != head_dim:
            raise ValueError(
                f"expected q_rope_cos_sin_cache [positions, 1, {head_dim}], got {tuple(q_rope_cos_sin_cache.shape)}")
    _lib.require_cuda(q, compact_k, compact_v)
    dev = q.device
    _inner_contiguous(q, "q")
    compact_k = compact_k.contiguous()
    compact_v = compact_v.contiguous()
    base_offsets = base_offsets.to(device=dev, dtype=torch.int32)
    live_counts = live_counts.to(device=dev, dtype=torch.int32)
    if base_offsets.stride(1) != 1 or live_counts.stride(1) != 1 or base_offsets.stride(0) != live_counts.stride(0):
        base_offsets = base_offsets.contiguous()
        live_counts = live_counts.contiguous()
    bt_sb = bt_sh = bt_pages = 0
    if block_tables is not None:
        if block_tables.ndim != 3 or block_tables.shape[:2] != (batch, num_kv_heads):
            raise ValueError(f"expected block_tables [batch, kv_heads, pages], got {tuple(block_tables.shape)}")
        block_tables = block_tables.to(device=dev, dtype=torch.int32)
        if block_tables.stride(2) != 1:
            block_tables = block_tables.contiguous()
        bt_sb, bt_sh, bt_pages = block_tables.stride(0), block_tables.stride(1), block_tables.shape[2]
    k_scale, v_scale = _scales(k_scale, v_scale, num_kv_heads, dev)
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.stride(-1) != 1:
        raise ValueError("out must have q's shape and a contiguous last dimension")
    if scale is None:
        scale = head_dim ** -0.5
    rope_pos = rope_cs = None
    cs_stride = 0
    if inline_q_rope:
        rope_pos = q_rope_positions.to(device=dev, dtype=torch.int64).contiguous()
        rope_cs = q_rope_cos_sin_cache.to(device=dev, dtype=torch.float32)
        if rope_cs.stride(2) != 1:
            rope_cs = rope_cs.contiguous()
        cs_stride = rope_cs.stride(0)
    ws = _lib.attn_workspace(dev, batch, num_kv_heads, head_dim)
    status = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().fdms_attn_decode(
            q.data_ptr(), _lib.dtype_code(q.dtype), q.stride(0), q.stride(1),
            compact_k.data_ptr(), compact_v.data_ptr(), _lib.dtype_code(compact_k.dtype), compact_k.shape[0],
            base_offsets.data_ptr(), live_counts.data_ptr(), live_counts.stride(0),
            _lib.ptr(block_tables), bt_sb, bt_sh, bt_pages,
            _lib.ptr(k_scale), _lib.ptr(v_scale),
            out.data_ptr(), _lib.dtype_code(out.dtype), out.stride(0), out.stride(1),
            batch, num_q_heads, num_kv_heads, head_dim, float(scale),
            _lib.ptr(rope_pos), _lib.ptr(rope_cs), cs_stride, rope_cs.shape[0] if rope_cs is not None else 0,
            ws.data_ptr(), ws.numel(), _lib.ATTN_OVERLAP_PREVIOUS if overlap_previous_kernel else 0,
            status.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc)
    return out


def compact_prefix_attention(
    q: torch.Tensor,
    compact_k: torch.Tensor,
    compact_v: torch.Tensor,
    base_offsets: torch.Tensor | None,
    live_counts: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    max_q_len: int,
    out: torch.Tensor,
    dense_lse: torch.Tensor | None = None,
    scale: float | None = None,
    *,
    seq_slots: torch.Tensor | None = None,
    block_tables: torch.Tensor | None = None,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    lse_out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Prefill-tail attention of a chunked prefill (no counterpart in the reference, whose prefill is
    one dense pass, `layers/attention.py:85-92`): the chunk's queries `q [tokens, q_heads, head_dim]`
    (post-RoPE, sequences delimited by `cu_seqlens_q`) attend to the rows their (sequence, KV head)
    span already holds -- `base_offsets` / `live_counts` `[rows, kv_heads]` addressed through
    `seq_slots` (or row i = sequence i), `block_tables [rows, kv_heads, pages]` for the paged layout --
    and the result is merged IN PLACE into `out`, which on entry holds the chunk's own causal
    attention with `dense_lse [q_heads, tokens]` its natural-log log-sum-exp.  `dense_lse=None`
    overwrites `out` with the attention over the span rows alone.  Spans with no rows leave `out`
    untouched.  One launch of `fdms_prefix_attention`."""
    if q.ndim != 3 or out.shape != q.shape or out.dtype != q.dtype:
        raise ValueError(f"expected q and out as [tokens, q_heads, head_dim] of one dtype, got {tuple(q.shape)} / {tuple(out.shape)}")
    tokens, num_q_heads, head_dim = q.shape
    if live_counts.ndim != 2:
        raise ValueError(f"expected live_counts [rows, kv_heads], got {tuple(live_counts.shape)}")
    num_kv_heads = live_counts.shape[1]
    if num_q_heads % num_kv_heads != 0:
        raise ValueError(f"q heads {num_q_heads} not divisible by kv heads {num_kv_heads}")
    if base_offsets is None and block_tables is None:
        raise ValueError("base_offsets or block_tables required")
    if compact_k.shape != compact_v.shape or compact_k.ndim != 2 or compact_k.shape[1] != head_dim:
        raise ValueError(f"expected compact_k/v as [slots, {head_dim}], got {tuple(compact_k.shape)} / {tuple(compact_v.shape)}")
    _lib.require_cuda(q, compact_k, compact_v, out)
    dev = q.device
    _inner_contiguous(q, "q")
    _inner_contiguous(out, "out")
    num_seqs = cu_seqlens_q.numel() - 1
    cu = cu_seqlens_q.to(device=dev, dtype=torch.int32).contiguous()
    live_counts = live_counts.to(device=dev, dtype=torch.int32)
    if live_counts.stride(1) != 1:
        live_counts = live_counts.contiguous()
    if base_offsets is not None:
        base_offsets = base_offsets.to(device=dev, dtype=torch.int32)
        if base_offsets.stride() != live_counts.stride():
            base_offsets, live_counts = base_offsets.contiguous(), live_counts.contiguous()
    bt_ss = bt_sh = bt_pages = 0
    if block_tables is not None:
        if block_tables.ndim != 3 or block_tables.shape[1] != num_kv_heads or block_tables.stride(2) != 1:
            raise ValueError(f"expected block_tables [rows, kv_heads, pages] (last dim contiguous), got {tuple(block_tables.shape)}")
        if block_tables.dtype != torch.int32:
            raise ValueError("block_tables must be int32")
        bt_ss, bt_sh, bt_pages = block_tables.stride(0), block_tables.stride(1), block_tables.shape[2]
    if seq_slots is not None:
        seq_slots = seq_slots.to(device=dev, dtype=torch.int32).contiguous()
    elif live_counts.shape[0] < num_seqs:
        raise ValueError("live_counts has fewer rows than sequences and no seq_slots were given")
    k_scale, v_scale = _scales(k_scale, v_scale, num_kv_heads, dev)
    lse_sh = lse_st = lo_sh = lo_st = 0
    if dense_lse is not None:
        if dense_lse.shape != (num_q_heads, tokens) or dense_lse.dtype != torch.float32:
            raise ValueError(f"expected float32 dense_lse {(num_q_heads, tokens)}, got {tuple(dense_lse.shape)} {dense_lse.dtype}")
        lse_sh, lse_st = dense_lse.stride()
    if lse_out is not None:
        if lse_out.shape != (num_q_heads, tokens) or lse_out.dtype != torch.float32:
            raise ValueError(f"expected float32 lse_out {(num_q_heads, tokens)}")
        lo_sh, lo_st = lse_out.stride()
    if scale is None:
        scale = head_dim ** -0.5
    status = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().fdms_prefix_attention(
            q.data_ptr(), _lib.dtype_code(q.dtype), q.stride(0), q.stride(1), cu.data_ptr(), int(max_q_len),
            compact_k.data_ptr(), compact_v.data_ptr(), _lib.dtype_code(compact_k.dtype), compact_k.shape[0],
            _lib.ptr(base_offsets), live_counts.data_ptr(), live_counts.stride(0),
            _lib.ptr(block_tables), bt_ss, bt_sh, bt_pages, _lib.ptr(seq_slots),
            _lib.ptr(k_scale), _lib.ptr(v_scale),
            out.data_ptr(), out.stride(0), out.stride(1),
            _lib.ptr(dense_lse), lse_sh, lse_st, _lib.ptr(lse_out), lo_sh, lo_st,
            num_seqs, num_q_heads, num_kv_heads, head_dim, float(scale), status.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc)
    return out


def fused_store_decode_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cos_sin_cache: torch.Tensor,
    compact_k: torch.Tensor,
    compact_v: torch.Tensor,
    base_offsets: torch.Tensor,
    live_counts: torch.Tensor,
    evict_out: torch.Tensor | None,
    positions: torch.Tensor,
    *,
    num_kv_heads: int,
    alpha_scale: float,
    alpha_offset: float,
    scale: float | None = None,
    block_tables: torch.Tensor | None = None,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    overlap_previous_kernel: bool = False,
) -> torch.Tensor:
    """`fused_dms_rope_store_compact_decode(store_q=False, store_transient_k=False)` followed by
    `compact_decode_attention(q_rope_positions=..., q_rope_cos_sin_cache=...)` in ONE launch.

    `live_counts` already counts the token being appended; its row is the last logical row of every
    span (row base + live - 1, or through the block table).  The new K/V rows land in the pool with
    the same bytes the separate store kernel writes, `evict_out` gets the same decisions, q/k/v are
    left untouched, and the attention output is returned.  FP8 pools, head_dim 64 or 128 only."""
    if q.ndim != 3 or k.ndim != 3 or v.ndim != 3:
        raise ValueError("expected q/k/v as [batch, heads, head_dim]")
    if k.shape != v.shape:
        raise ValueError(f"k/value shape mismatch: {k.shape} != {v.shape}")
    batch, num_q_heads, head_dim = q.shape
    if k.shape != (batch, num_kv_heads, head_dim):
        raise ValueError(f"q/k shape mismatch: q={q.shape}, k={k.shape}, num_kv_heads={num_kv_heads}")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError(f"q_heads={num_q_heads} must be divisible by kv_heads={num_kv_heads}")
    if compact_k.shape != compact_v.shape or compact_k.ndim != 2 or compact_k.shape[1] != head_dim:
        raise ValueError(f"expected compact cache [slots, {head_dim}], got {compact_k.shape}/{compact_v.shape}")
    if base_offsets.shape != (batch, num_kv_heads) or live_counts.shape != (batch, num_kv_heads):
        raise ValueError("base_offsets and live_counts must both be [batch, kv_heads]")
    if evict_out is not None and (evict_out.shape != (batch, num_kv_heads) or evict_out.dtype != torch.bool):
        raise ValueError(f"expected evict_out bool {(batch, num_kv_heads)}, got {tuple(evict_out.shape)} {evict_out.dtype}")
    if positions.shape != (batch,):
        raise ValueError(f"expected positions {(batch,)}, got {tuple(positions.shape)}")
    if cos_sin_cache.ndim != 3 or cos_sin_cache.shape[2] != head_dim:
        raise ValueError(f"expected cos_sin_cache [positions, 1, {head_dim}], got {tuple(cos_sin_cache.shape)}")
    if q.dtype != k.dtype or k.dtype != v.dtype:
        raise ValueError("q, k and v must share a dtype")
    _lib.require_cuda(q, k, v, compact_k, compact_v)
    dev = q.device
    for name, t in (("q", q), ("k", k), ("v", v)):
        _inner_contiguous(t, name)
    if not compact_k.is_contiguous() or not compact_v.is_contiguous():
        raise ValueError("compact caches must be contiguous")
    base_offsets = base_offsets.to(device=dev, dtype=torch.int32)
    live_counts = live_counts.to(device=dev, dtype=torch.int32)
    if base_offsets.stride(1) != 1 or live_counts.stride(1) != 1 or base_offsets.stride(0) != live_counts.stride(0):
        base_offsets, live_counts = base_offsets.contiguous(), live_counts.contiguous()
    bt_sb = bt_sh = bt_pages = 0
    if block_tables is not None:
        if block_tables.ndim != 3 or block_tables.shape[:2] != (batch, num_kv_heads):
            raise ValueError(f"expected block_tables [batch, kv_heads, pages], got {tuple(block_tables.shape)}")
        block_tables = block_tables.to(device=dev, dtype=torch.int32)
        if block_tables.stride(2) != 1:
            block_tables = block_tables.contiguous()
        bt_sb, bt_sh, bt_pages = block_tables.stride(0), block_tables.stride(1), block_tables.shape[2]
    k_scale, v_scale = _scales(k_scale, v_scale, num_kv_heads, dev)
    positions = positions.to(device=dev, dtype=torch.int64).contiguous()
    cos_sin_cache = cos_sin_cache.to(device=dev, dtype=torch.float32)
    if cos_sin_cache.stride(2) != 1:
        cos_sin_cache = cos_sin_cache.contiguous()
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.stride(-1) != 1:
        raise ValueError("out must have q's shape and a contiguous last dimension")
    if scale is None:
        scale = head_dim ** -0.5
    ev_u8 = None if evict_out is None else evict_out.view(torch.uint8)
    if ev_u8 is not None and ev_u8.stride(1) != 1:
        raise ValueError("evict_out must be contiguous in its last dimension")
    ws = _lib.attn_workspace(dev, batch, num_kv_heads, head_dim)
    status = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().fdms_attn_decode_append(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.dtype_code(q.dtype),
            q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
            compact_k.data_ptr(), compact_v.data_ptr(), _lib.dtype_code(compact_k.dtype), compact_k.shape[0],
            base_offsets.data_ptr(), live_counts.data_ptr(), live_counts.stride(0),
            _lib.ptr(block_tables), bt_sb, bt_sh, bt_pages, _lib.ptr(k_scale), _lib.ptr(v_scale),
            cos_sin_cache.data_ptr(), cos_sin_cache.stride(0), cos_sin_cache.shape[0], positions.data_ptr(),
            _lib.ptr(ev_u8), ev_u8.stride(0) if ev_u8 is not None else 0, float(alpha_scale), float(alpha_offset),
            out.data_ptr(), _lib.dtype_code(out.dtype), out.stride(0), out.stride(1),
            batch, num_q_heads, num_kv_heads, head_dim, float(scale),
            ws.data_ptr(), ws.numel(), _lib.ATTN_OVERLAP_PREVIOUS if overlap_previous_kernel else 0,
            status.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc)
    return out


def _store_common(q, k, v, cos_sin_cache, compact_k, compact_v, slot_mapping, evict_out, positions, *,
                  num_kv_heads, alpha_scale, alpha_offset, do_decision, do_rope, store_q, store_k,
                  k_scale=None, v_scale=None):
    dev = k.device
    batch, _, head_dim = k.shape
    num_q_heads = q.shape[1] if q is not None else num_kv_heads
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t is not None:
            _inner_contiguous(t, name)
    if compact_k is not None and (not compact_k.is_contiguous() or not compact_v.is_contiguous()):
        raise ValueError("compact caches must be contiguous")
    if slot_mapping is not None:
        slot_mapping = slot_mapping.to(device=dev, dtype=torch.int32)
        if slot_mapping.stride(1) != 1:
            slot_mapping = slot_mapping.contiguous()
    cs_stride = 0
    if do_rope:
        if positions.dtype != torch.int64:
            positions = positions.to(dtype=torch.int64)
        positions = positions.to(dev).contiguous()
        cos_sin_cache = cos_sin_cache.to(device=dev, dtype=torch.float32)
        if cos_sin_cache.stride(-1) != 1:
            cos_sin_cache = cos_sin_cache.contiguous()
        cs_stride = cos_sin_cache.stride(0)
    k_scale, v_scale = _scales(k_scale, v_scale, num_kv_heads, dev)
    ev_u8 = None if evict_out is None else evict_out.view(torch.uint8)
    status = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().fdms_store_decode(
            _lib.ptr(q), q.stride(0) if q is not None else 0, q.stride(1) if q is not None else 0,
            k.data_ptr(), k.stride(0), k.stride(1),
            v.data_ptr(), v.stride(0), v.stride(1), _lib.dtype_code(k.dtype),
            _lib.ptr(cos_sin_cache) if do_rope else None, cs_stride, cos_sin_cache.shape[0] if do_rope else 0,
            _lib.ptr(positions) if do_rope else None,
            _lib.ptr(compact_k), _lib.ptr(compact_v),
            _lib.dtype_code(compact_k.dtype) if compact_k is not None else 0,
            compact_k.shape[0] if compact_k is not None else 0,
            _lib.ptr(slot_mapping), slot_mapping.stride(0) if slot_mapping is not None else 0,
            _lib.ptr(ev_u8), ev_u8.stride(0) if ev_u8 is not None else 0,
            _lib.ptr(k_scale), _lib.ptr(v_scale),
            batch, num_q_heads, num_kv_heads, head_dim,
            float(alpha_scale), float(alpha_offset),
            int(do_decision), int(do_rope), int(store_q), int(store_k),
            status.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc)


def store_compact_kvcache(
    key: torch.Tensor,
    value: torch.Tensor,
    compact_k: torch.Tensor,
    compact_v: torch.Tensor,
    slot_mapping: torch.Tensor,
    *,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
) -> None:
    """Plain append of k, v rows at slot_mapping (reference: compact_attention.py:968-1007)."""
    if key.shape != value.shape:
        raise ValueError(f"key/value shape mismatch: {key.shape} != {value.shape}")
    if key.ndim != 3:
        raise ValueError(f"expected key/value as [batch, kv_heads, head_dim], got {key.shape}")
    batch, num_kv_heads, head_dim = key.shape
    if compact_k.shape != compact_v.shape:
        raise ValueError(f"compact cache shape mismatch: {compact_k.shape} != {compact_v.shape}")
    if compact_k.ndim != 2 or compact_k.shape[1] != head_dim:
        raise ValueError(f"expected compact cache [slots, {head_dim}], got {compact_k.shape}")
    if slot_mapping.shape != (batch, num_kv_heads):
        raise ValueError(f"expected slot_mapping {(batch, num_kv_heads)}, got {tuple(slot_mapping.shape)}")
    _lib.require_cuda(key, value, compact_k, compact_v)
    if head_dim % 2 != 0:
        raise ValueError(f"head_dim must be even, got {head_dim}")
    _store_common(None, key, value, None, compact_k, compact_v, slot_mapping, None, None,
                  num_kv_heads=num_kv_heads, alpha_scale=1.0, alpha_offset=0.0, do_decision=False,
                  do_rope=False, store_q=False, store_k=False, k_scale=k_scale, v_scale=v_scale)


def fused_dms_rope_store_compact_decode(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cos_sin_cache: torch.Tensor,
    compact_k: torch.Tensor,
    compact_v: torch.Tensor,
    slot_mapping: torch.Tensor,
    evict_out: torch.Tensor,
    positions: torch.Tensor,
    *,
    num_kv_heads: int,
    alpha_scale: float,
    alpha_offset: float,
    store_q: bool = True,
    store_transient_k: bool = True,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
) -> None:
    """Decode-only DMS extraction + RoPE + compact append-store (reference:
    compact_attention.py:1010-1113).  q (when store_q) and k (when store_transient_k) are rotated
    in place; post-RoPE k and raw v are cast into compact_k/compact_v at slot_mapping; evict_out
    receives the per-(sequence, KV head) decision."""
    if q.ndim != 3 or k.ndim != 3 or v.ndim != 3:
        raise ValueError("expected q/k/v as [batch, heads, head_dim]")
    if k.shape != v.shape:
        raise ValueError(f"k/value shape mismatch: {k.shape} != {v.shape}")
    batch, num_q_heads, head_dim = q.shape
    if k.shape[0] != batch or k.shape[1] != num_kv_heads or k.shape[2] != head_dim:
        raise ValueError(f"q/k shape mismatch: q={q.shape}, k={k.shape}, num_kv_heads={num_kv_heads}")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError(f"q_heads={num_q_heads} must be divisible by kv_heads={num_kv_heads}")
    if head_dim % 2 != 0:
        raise ValueError(f"RoPE head_dim must be even, got {head_dim}")
    if compact_k.shape != compact_v.shape or compact_k.ndim != 2 or compact_k.shape[1] != head_dim:
        raise ValueError(f"expected compact cache [slots, {head_dim}], got {compact_k.shape}/{compact_v.shape}")
    if slot_mapping.shape != (batch, num_kv_heads):
        raise ValueError(f"expected slot_mapping {(batch, num_kv_heads)}, got {tuple(slot_mapping.shape)}")
    if evict_out.shape != (batch, num_kv_heads) or evict_out.dtype != torch.bool:
        raise ValueError(f"expected evict_out bool {(batch, num_kv_heads)}, got {tuple(evict_out.shape)} {evict_out.dtype}")
    if positions.shape != (batch,):
        raise ValueError(f"expected positions {(batch,)}, got {tuple(positions.shape)}")
    if head_dim > 256:
        raise ValueError(f"head_dim={head_dim} is above the fused decode preprocess kernel limit")
    if not (q.is_cuda and k.is_cuda and v.is_cuda and compact_k.is_cuda):
        raise RuntimeError("fused decode preprocess requires CUDA tensors")
    if evict_out.device != q.device:
        raise ValueError(f"expected evict_out on {q.device}, got {evict_out.device}")
    if q.dtype != k.dtype or k.dtype != v.dtype:
        raise ValueError("q, k and v must share a dtype")
    if evict_out.stride(1) != 1:
        raise ValueError("evict_out must be contiguous in its last dimension")
    if cos_sin_cache.ndim != 3 or cos_sin_cache.shape[2] != head_dim:
        raise ValueError(f"expected cos_sin_cache [positions, 1, {head_dim}], got {tuple(cos_sin_cache.shape)}")
    _store_common(q, k, v, cos_sin_cache, compact_k, compact_v, slot_mapping, evict_out, positions,
                  num_kv_heads=num_kv_heads, alpha_scale=alpha_scale, alpha_offset=alpha_offset,
                  do_decision=True, do_rope=True, store_q=store_q, store_k=store_transient_k,
                  k_scale=k_scale, v_scale=v_scale)


def _expiry_one_layer(mode, positions_per_lh, evict_per_lh, live_counts, base_offsets, compact_k, compact_v,
                      current_positions, window_size):
    if positions_per_lh.ndim != 3 or evict_per_lh.shape != positions_per_lh.shape:
        raise ValueError("expected positions/evict as [num_seqs, num_kv_heads, max_capacity]")
    num_seqs, num_kv_heads, capacity = positions_per_lh.shape
    if live_counts.shape != (num_seqs, num_kv_heads) or base_offsets.shape != (num_seqs, num_kv_heads):
        raise ValueError("expected live_counts/base_offsets as [num_seqs, num_kv_heads]")
    if positions_per_lh.dtype != torch.int32 or evict_per_lh.dtype != torch.bool or live_counts.dtype != torch.int32:
        raise ValueError("expected int32 positions / live counts and bool evict mask")
    _lib.require_cuda(positions_per_lh, evict_per_lh, live_counts, base_offsets, compact_k, compact_v)
    if positions_per_lh.stride(2) != 1 or evict_per_lh.stride(2) != 1:
        raise ValueError("metadata rows must be contiguous")
    if live_counts.stride(1) != 1 or base_offsets.stride() != live_counts.stride() or base_offsets.dtype != torch.int32:
        raise ValueError("live_counts and base_offsets must be int32 with identical, head-contiguous strides")
    if not compact_k.is_contiguous() or not compact_v.is_contiguous():
        raise ValueError("compact caches must be contiguous")
    dev = compact_k.device
    cur = current_positions.to(device=dev, dtype=torch.int64).contiguous()
    ev = evict_per_lh.view(torch.uint8)
    row_bytes = compact_k.shape[-1] * compact_k.element_size()
    status = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().fdms_expire_compact(
            positions_per_lh.data_ptr(), 0, positions_per_lh.stride(0), positions_per_lh.stride(1),
            ev.data_ptr(), 0, ev.stride(0), ev.stride(1), None,
            live_counts.data_ptr(), base_offsets.data_ptr(), 0, live_counts.stride(0),
            compact_k.data_ptr(), compact_v.data_ptr(), 0, row_bytes, compact_k.shape[0],
            None, 0, 0, 0, None, None, 0,
            None, cur.data_ptr(),
            1, num_seqs, num_kv_heads, capacity, int(window_size), mode, None, None,
            status.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc)


def dms_expiry_one_layer(*, positions_per_lh, evict_per_lh, live_counts, base_offsets, compact_k, compact_v,
                         current_positions, window_size) -> None:
    """Full expiry of one layer, in place (reference: compact_attention.py:861-911)."""
    _expiry_one_layer(0, positions_per_lh, evict_per_lh, live_counts, base_offsets, compact_k, compact_v,
                      current_positions, window_size)


def dms_expiry_incremental_one_layer(*, positions_per_lh, evict_per_lh, live_counts, base_offsets, compact_k,
                                     compact_v, current_positions, window_size) -> None:
    """Steady-state expiry: drops the first window-expired slot only (reference:
    compact_attention.py:914-965)."""
    _expiry_one_layer(1, positions_per_lh, evict_per_lh, live_counts, base_offsets, compact_k, compact_v,
                      current_positions, window_size)


def kv_quantize_fp8(x: torch.Tensor, scale: torch.Tensor | None = None) -> torch.Tensor:
    """x [n, kv_heads, head_dim] (f32/bf16/f16) -> float8_e4m3fn of x / scale[h]."""
    if x.ndim != 3:
        raise ValueError(f"expected x as [n, kv_heads, head_dim], got {tuple(x.shape)}")
    _lib.require_cuda(x)
    x = x.contiguous()
    n, hk, d = x.shape
    (scale,) = _scales(scale, None, hk, x.device)[:1]
    out = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().fdms_kv_quant(x.data_ptr(), _lib.dtype_code(x.dtype), out.data_ptr(), _lib.ptr(scale),
                                      n, hk, d, _lib.stream_ptr(x.device))
    _lib.check(rc)
    return out


def kv_dequantize_fp8(x: torch.Tensor, scale: torch.Tensor | None = None,
                      dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """float8_e4m3fn [n, kv_heads, head_dim] -> `dtype` of x * scale[h]."""
    if x.ndim != 3 or x.dtype != torch.float8_e4m3fn:
        raise ValueError("expected float8_e4m3fn x as [n, kv_heads, head_dim]")
    _lib.require_cuda(x)
    x = x.contiguous()
    n, hk, d = x.shape
    (scale,) = _scales(scale, None, hk, x.device)[:1]
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().fdms_kv_dequant(x.data_ptr(), out.data_ptr(), _lib.dtype_code(dtype), _lib.ptr(scale),
                                        n, hk, d, _lib.stream_ptr(x.device))
    _lib.check(rc)
    return out

"""CompactKVManager: owner of the compact FP8 KV pools and of the per-(layer, sequence, KV head)
DMS metadata.  Public names follow the reference's `fastdms/engine/compact_kv.py`.

B200-first layout (differences from the reference are storage only, results are identical):
  * One pool allocation per manager, `[layers, capacity_tokens, head_dim]` for K and for V, made
    up front (180 GB of HBM makes the reference's lazy 256-slot growth, and the CUDA-graph
    re-capture it forces, unnecessary).  `compact_k_per_layer[l]` are views into it.
  * Metadata is always layer-major on the device: `[layers, active_slots, kv_heads(, capacity)]`.
    A sequence's state object holds views of its slot, like the reference's layer-major mode.
  * Two span layouts: contiguous ranges handed out by a host first-fit list (the reference's
    scheme, so base offsets and slot indices are bit-identical), or 16-row pages with block tables
    and a per-layer free stack that lives on the GPU (`paged=True`; no host round trip at all).
  * Expiry, decode metadata and decision recording each take ONE launch for all layers.
"""
from __future__ import annotations

import bisect
import os
from dataclasses import dataclass

import torch

from fastdms_b200 import _lib
from fastdms_b200.engine.sequence import Sequence

PAGE = 16
PACK_CHUNK = 256
_I64_MAX = (1 << 63) - 1


@dataclass(slots=True)
class CompactKVMetadata:
    base_offsets: torch.Tensor
    live_counts: torch.Tensor
    token_positions: torch.Tensor | None = None

    @property
    def max_live_count(self) -> int:
        if self.live_counts.numel() == 0:
            return 0
        return int(self.live_counts.max().item())


@dataclass(slots=True)
class CompactKVSequenceState:
    """Views of one sequence's rows in the manager's layer-major arrays (reference:
    compact_kv.py:500-520)."""
    seq_id: int
    base_offsets: torch.Tensor      # [layers, kv_heads] int32, -1 = not allocated
    range_capacity: torch.Tensor    # [layers, kv_heads] int32 reserved rows
    live_counts: torch.Tensor       # [layers, kv_heads] int32
    token_positions: torch.Tensor   # [layers, kv_heads, capacity] int32, -1 padded
    evict_mask: torch.Tensor        # [layers, kv_heads, capacity] bool
    max_capacity_per_lh: int
    decode_headroom: int
    active_slot: int | None = None
    dms_initial_expiry_done: bool = False
    last_dms_expiry_position: int = -1
    # host mirror of the reserved ranges: (base, size) per [layer][head]; avoids device reads on free
    host_ranges: list | None = None


def expiry_interval_from_env(default: int) -> int:
    """FASTDMS_DMS_EXPIRY_INTERVAL: 1 = expire every step (exact), N = only when position % N == 0."""
    raw = os.environ.get("FASTDMS_DMS_EXPIRY_INTERVAL")
    return max(1, int(raw)) if raw not in (None, "") else max(1, int(default))


class CompactKVManager:
    def __init__(
        self,
        *,
        num_layers: int,
        num_kv_heads: int,
        capacity_tokens: int,
        max_model_len: int,
        device: torch.device | str,
        target_live_tokens_per_seq: int | None = None,
        head_dim: int | None = None,
        compact_dtype: torch.dtype | None = None,
        per_layer_storage: bool = True,
        layer_major_metadata: bool = True,
        max_active_seqs: int | None = None,
        paged: bool = False,
        k_scale: torch.Tensor | None = None,
        v_scale: torch.Tensor | None = None,
        dms_expiry_interval: int = 1,
        row_indirection: bool = False,
        admission: str = "reserve",
        admission_keep_estimate: float = 0.25,
        admission_window: int = 256,
    ):
        if capacity_tokens <= 0:
            raise ValueError(f"capacity_tokens must be positive, got {capacity_tokens}")
        self.num_layers = int(num_layers)
        self.num_kv_heads = int(num_kv_heads)
        self.capacity_tokens = int(capacity_tokens)
        self.max_model_len = int(max_model_len)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("CompactKVManager requires a CUDA device (there is no CPU fallback)")
        if head_dim is None or compact_dtype is None:
            raise RuntimeError("CompactKVManager requires head_dim and compact_dtype")
        self.head_dim = int(head_dim)
        self.compact_dtype = compact_dtype
        self.per_layer_storage = True
        self.layer_major_metadata = True
        self.max_active_seqs = int(max_active_seqs or 64)
        self.target_live_tokens_per_seq = target_live_tokens_per_seq
        self.paged = bool(paged)
        self.dms_expiry_interval = int(dms_expiry_interval)
        self.row_indirection = bool(row_indirection)
        if admission not in ("reserve", "optimistic"):
            raise ValueError(f"admission must be 'reserve' or 'optimistic', got {admission!r}")
        self.admission = admission
        # paged layout: host-side lower bound of the free pages of the fullest layer (None = unknown)
        self._free_pages_lb: int | None = None
        self.preemption_guard_refreshes = 0
        self.admission_keep_estimate = float(admission_keep_estimate)
        self.admission_window = int(admission_window)
        self.debug_checks = os.environ.get("FASTDMS_COMPACT_DEBUG_CHECKS") == "1"
        self.admission_denied_count = 0
        L, S, Hk, C = self.num_layers, self.max_active_seqs, self.num_kv_heads, self.max_model_len
        dev = self.device
        if self.paged:
            self.capacity_tokens = ((self.capacity_tokens + PAGE - 1) // PAGE) * PAGE
        # pools: one allocation each, [layers, rows, head_dim]
        self.compact_k = torch.zeros((L, self.capacity_tokens, self.head_dim), device=dev, dtype=compact_dtype)
        self.compact_v = torch.zeros_like(self.compact_k)
        self.compact_k_per_layer = [self.compact_k[l] for l in range(L)]
        self.compact_v_per_layer = [self.compact_v[l] for l in range(L)]
        # layer-major metadata
        self.layer_major_base_offsets = torch.full((L, S, Hk), -1, device=dev, dtype=torch.int32)
        self.layer_major_range_capacity = torch.zeros((L, S, Hk), device=dev, dtype=torch.int32)
        self.layer_major_live_counts = torch.zeros((L, S, Hk), device=dev, dtype=torch.int32)
        self.layer_major_token_positions = torch.full((L, S, Hk, C), -1, device=dev, dtype=torch.int32)
        self.layer_major_evict_mask = torch.zeros((L, S, Hk, C), device=dev, dtype=torch.bool)
        # Optional logical slot -> physical row map of every span.  With it, expiry compacts only the
        # metadata in order and keeps the span's K/V rows dense by refilling freed rows (one row copy
        # per dropped token); without it K/V rows are shifted like the reference's.  Logical row i of
        # a span is physical row layer_major_row_index[l, slot, h, i]; entries >= live equal i.
        self.layer_major_row_index = None
        if self.row_indirection:
            self.layer_major_row_index = torch.arange(C, device=dev, dtype=torch.int32).expand(L, S, Hk, C).contiguous()
        # Position up to which a span is known to hold no expired slot (-1: unknown): lets the per-step expiry of a
        # decode loop inspect one slot per span instead of the whole span (`fdms_expire_compact: exact_through`).
        # Written by the expiry launch; reset here whenever slots are written by other means (pack, release).
        self.layer_major_exact_through = None
        if self.layer_major_row_index is not None:
            self.layer_major_exact_through = torch.full((L, S, Hk), -1, device=dev, dtype=torch.int64)
        self.free_active_slots: list[int] = list(range(S))
        self.active_slot_by_seq: dict[int, int] = {}
        self.seq_states: dict[int, CompactKVSequenceState] = {}
        # span allocator (host) or page allocator (device)
        self.free_ranges_per_layer: list[list[tuple[int, int]]] = [[(0, self.capacity_tokens)] for _ in range(L)]
        self.block_tables = None
        self.free_pages = None
        self.free_page_counts = None
        self.max_pages = 0
        self.pages_per_layer = 0
        if self.paged:
            self.pages_per_layer = self.capacity_tokens // PAGE
            self.max_pages = (C + PAGE - 1) // PAGE
            self.block_tables = torch.full((L, S, Hk, self.max_pages), -1, device=dev, dtype=torch.int32)
            # stack of free page ids; popped from the top, so page 0 is handed out first
            ids = torch.arange(self.pages_per_layer - 1, -1, -1, device=dev, dtype=torch.int32)
            self.free_pages = ids.unsqueeze(0).repeat(L, 1).contiguous()
            self.free_page_counts = torch.full((L,), self.pages_per_layer, device=dev, dtype=torch.int32)
        self.k_scale = self._check_scale(k_scale)
        self.v_scale = self._check_scale(v_scale)
        self._attn_modules: list = []
        self._slot_cache: dict[tuple, torch.Tensor] = {}
        self._decode_buffers: dict[int, tuple] = {}
        self._stats_init = torch.tensor([0, _I64_MAX, 0, _I64_MAX, 0], device=dev, dtype=torch.int64)

    # ------------------------------------------------------------------ helpers
    def _check_scale(self, s):
        if s is None:
            return None
        if tuple(s.shape) != (self.num_layers, self.num_kv_heads):
            raise ValueError(f"expected per-(layer, kv head) scale {(self.num_layers, self.num_kv_heads)}, got {tuple(s.shape)}")
        return s.to(device=self.device, dtype=torch.float32).contiguous()

    def layer_scales(self, layer_id: int):
        ks = None if self.k_scale is None else self.k_scale[layer_id]
        vs = None if self.v_scale is None else self.v_scale[layer_id]
        return ks, vs

    def attach_attention_modules(self, attn_modules: list) -> None:
        """Binds every attention module (ordered by layer) to its layer's pool views."""
        self._attn_modules = attn_modules
        for l, module in enumerate(attn_modules[: self.num_layers]):
            module.compact_k_cache = self.compact_k_per_layer[l]
            module.compact_v_cache = self.compact_v_per_layer[l]
            module.compact_k_scale, module.compact_v_scale = self.layer_scales(l)

    def _ensure_layer_storage(self, layer_id: int, min_tokens: int):
        """Pools are allocated up front; only checks the request against the layer capacity."""
        if min_tokens > self.capacity_tokens:
            raise RuntimeError(
                f"compact KV capacity exhausted in layer {layer_id}: requested {min_tokens}, capacity {self.capacity_tokens}")
        return self.compact_k_per_layer[layer_id], self.compact_v_per_layer[layer_id]

    def _slots_tensor(self, states) -> torch.Tensor:
        key = tuple(int(s.active_slot) for s in states)
        t = self._slot_cache.get(key)
        if t is None:
            if len(self._slot_cache) > 256:
                self._slot_cache.clear()
            t = torch.tensor(key, device=self.device, dtype=torch.int32)
            self._slot_cache[key] = t
        return t

    def _states(self, seqs) -> list[CompactKVSequenceState]:
        states = [self.seq_states.get(seq.seq_id) for seq in seqs]
        if any(s is None for s in states):
            missing = [seq.seq_id for seq, s in zip(seqs, states) if s is None]
            raise RuntimeError(f"sequence(s) {missing} have no compact KV allocation")
        return states

    def _contiguous_active_slot_start(self, states) -> int | None:
        if not states:
            return None
        slots = [s.active_slot for s in states]
        if any(s is None for s in slots):
            return None
        start = int(slots[0])
        return start if [int(s) for s in slots] == list(range(start, start + len(slots))) else None

    # ------------------------------------------------------------------ span allocator (host)
    def free_tokens_in_layer(self, layer_id: int) -> int:
        if self.paged:
            return int(self.free_page_counts[layer_id].item()) * PAGE
        return sum(n for _, n in self.free_ranges_per_layer[layer_id])

    @property
    def free_tokens(self) -> int:
        if self.paged:
            return int(self.free_page_counts.sum().item()) * PAGE
        return sum(self.free_tokens_in_layer(l) for l in range(self.num_layers))

    def _alloc_range(self, layer_id: int, length: int) -> int:
        """Takes `length` rows from the lowest free range of the layer that can hold them and
        returns the first row.  The list is kept sorted by start and coalesced, so this first-fit
        rule hands out the same bases as the reference's allocator (compact_kv.py:705-718) for the
        same sequence of requests, which the slot-index parity tests rely on."""
        ranges = self.free_ranges_per_layer[layer_id]
        hit = next((i for i, (_, size) in enumerate(ranges) if size >= length), None)
        if hit is None:
            raise RuntimeError(f"compact KV capacity exhausted in layer {layer_id}: {length} rows requested, "
                               f"{self.free_tokens_in_layer(layer_id)} free in {len(ranges)} ranges")
        first, size = ranges[hit]
        if size > length:
            ranges[hit] = (first + length, size - length)
        else:
            del ranges[hit]
        return first

    def _free_range(self, layer_id: int, start: int, length: int) -> None:
        """Gives rows [start, start + length) back: inserted at its sorted place and fused with the
        free neighbour on either side (reference: compact_kv.py:720-737)."""
        if length <= 0:
            return
        ranges = self.free_ranges_per_layer[layer_id]
        at = bisect.bisect_left(ranges, (start, 0))
        lo, hi = start, start + length
        if at > 0 and ranges[at - 1][0] + ranges[at - 1][1] >= lo:          # touches the range below
            at -= 1
            lo = ranges[at][0]
            hi = max(hi, ranges[at][0] + ranges[at][1])
            del ranges[at]
        while at < len(ranges) and ranges[at][0] <= hi:                      # swallows ranges above
            hi = max(hi, ranges[at][0] + ranges[at][1])
            del ranges[at]
        ranges.insert(at, (lo, hi - lo))

    def _reservation_tokens(self, seq: Sequence) -> int:
        worst = min(self.max_model_len, seq.num_prompt_tokens + seq.max_tokens)
        if self.target_live_tokens_per_seq is not None:
            return min(worst, max(1, int(self.target_live_tokens_per_seq)))
        return worst

    def admission_need(self, seq: Sequence) -> int:
        """Pool rows per layer a new sequence is charged at admission.  `reserve`: its worst case
        (every token kept).  `optimistic`: an estimate of what the DMS
        prefill keeps, `prompt * admission_keep_estimate + window`, plus the decode headroom; the
        engine retries a prefill that turns out not to fit."""
        rows = self._reservation_tokens(seq)
        if self.admission == "optimistic":
            est = int(seq.num_tokens * self.admission_keep_estimate) + self.admission_window + \
                max(int(seq.max_tokens) - seq.num_completion_tokens, 0) + 1
            rows = min(rows, max(est, 1))
        if self.paged:
            rows = ((rows + PAGE - 1) // PAGE) * PAGE
        return rows * self.num_kv_heads

    def decode_pages_guaranteed(self, batch: int) -> bool:
        """Paged layout: True when every span of a decode batch of `batch` sequences can take a new
        page in this step (the worst case: all of them cross a page boundary at once) in every layer.
        Works on a host-side lower bound of the free pages that is decremented by that worst case per
        step and refreshed from the device only when it runs low, so a roomy pool costs no
        synchronisation.  Contiguous spans own their decode headroom: always True."""
        if not self.paged:
            return True
        need = batch * self.num_kv_heads
        if self._free_pages_lb is None or self._free_pages_lb < need:
            self._free_pages_lb = int(self.free_page_counts.min().item())
            self.preemption_guard_refreshes += 1
        if self._free_pages_lb < need:
            return False
        self._free_pages_lb -= need
        return True

    def prefill_pages_guaranteed(self, tokens: int, num_seqs: int) -> bool:
        """Paged layout, chunked prefill: True when a prefill step of `tokens` tokens over `num_seqs`
        sequences finds its pages in every layer even if every token is kept (one partly filled page
        per span on top).  Same host-side bound as `decode_pages_guaranteed`; a check only -- the pack
        marks the bound stale, so it is read again before the next step."""
        if not self.paged:
            return True
        need = ((int(tokens) + PAGE - 1) // PAGE + int(num_seqs)) * self.num_kv_heads
        if self._free_pages_lb is None or self._free_pages_lb < need:
            self._free_pages_lb = int(self.free_page_counts.min().item())
            self.preemption_guard_refreshes += 1
        return self._free_pages_lb >= need

    def admission_free(self) -> int:
        """Free pool rows in the fullest layer."""
        if self.paged:
            self._free_pages_lb = int(self.free_page_counts.min().item())
            return self._free_pages_lb * PAGE
        return min(self.free_tokens_in_layer(l) for l in range(self.num_layers))

    def can_allocate(self, seq: Sequence, pending_rows: int = 0) -> bool:
        """Admission check (the reference defines it, compact_kv.py:739-745, and never calls it):
        an active slot is free and the charged rows, on top of `pending_rows` already promised to
        requests admitted in the same scheduling pass, fit in every layer."""
        ok = bool(self.free_active_slots or seq.seq_id in self.seq_states) and \
            self.admission_need(seq) + pending_rows <= self.admission_free()
        if not ok:
            self.admission_denied_count += 1
        return ok

    # ------------------------------------------------------------------ registration
    def allocate(self, seq: Sequence) -> CompactKVSequenceState:
        """Registers a sequence: takes an active slot and resets its metadata rows; the spans are
        reserved later, per layer, from the observed live counts (reference: compact_kv.py:753-828)."""
        existing = self.seq_states.get(seq.seq_id)
        if existing is not None:
            return existing
        cap = self._reservation_tokens(seq)
        if cap <= 0:
            raise ValueError(f"invalid reservation {cap} for seq {seq.seq_id}")
        if not self.free_active_slots:
            raise RuntimeError(f"compact KV active-slot capacity exhausted: max_active_seqs={self.max_active_seqs}")
        slot = self.free_active_slots.pop(0)
        self.active_slot_by_seq[seq.seq_id] = slot
        base = self.layer_major_base_offsets[:, slot, :]
        rcap = self.layer_major_range_capacity[:, slot, :]
        live = self.layer_major_live_counts[:, slot, :]
        pos = self.layer_major_token_positions[:, slot, :, :cap]
        ev = self.layer_major_evict_mask[:, slot, :, :cap]
        base.fill_(-1)
        rcap.zero_()
        live.zero_()
        pos.fill_(-1)
        ev.zero_()
        if self.layer_major_row_index is not None:
            self.layer_major_row_index[:, slot, :, :] = torch.arange(self.max_model_len, device=self.device, dtype=torch.int32)
            self.layer_major_exact_through[:, slot, :].fill_(-1)
        state = CompactKVSequenceState(
            seq_id=seq.seq_id, base_offsets=base, range_capacity=rcap, live_counts=live,
            token_positions=pos, evict_mask=ev, max_capacity_per_lh=cap,
            decode_headroom=int(seq.max_tokens), active_slot=slot,
            host_ranges=[[None] * self.num_kv_heads for _ in range(self.num_layers)])
        self.seq_states[seq.seq_id] = state
        return state

    def _reserve_layer(self, state: CompactKVSequenceState, layer_id: int, live_per_head: list[int]):
        """Host part of the per-layer reservation: first-fit ranges of min(live + headroom, C) rows
        per head (reference: compact_kv.py:830-857).  Returns (bases, sizes)."""
        sizes = [max(min(int(n) + int(state.decode_headroom), state.max_capacity_per_lh), 1) for n in live_per_head]
        bases: list[int] = []
        try:
            for size in sizes:
                bases.append(self._alloc_range(layer_id, size))
        except Exception:
            for b, sz in zip(bases, sizes):
                self._free_range(layer_id, b, sz)
            raise
        for h, (b, sz) in enumerate(zip(bases, sizes)):
            state.host_ranges[layer_id][h] = (b, sz)
        return bases, sizes

    def _allocate_layer_ranges_for_seq(self, state, layer_id: int, live_count_per_head: torch.Tensor) -> torch.Tensor:
        bases, sizes = self._reserve_layer(state, layer_id, live_count_per_head.tolist())
        bases_t = torch.tensor(bases, device=self.device, dtype=torch.int32)
        state.base_offsets[layer_id].copy_(bases_t)
        state.range_capacity[layer_id].copy_(torch.tensor(sizes, device=self.device, dtype=torch.int32))
        return bases_t

    def mark_all_heads_live(self, seq_id: int, live_count: int) -> None:
        self.mark_live_counts(seq_id, torch.full((self.num_layers, self.num_kv_heads), live_count,
                                                 device=self.device, dtype=torch.int32))

    def mark_live_counts(self, seq_id: int, live_counts: torch.Tensor) -> None:
        state = self.seq_states[seq_id]
        if live_counts.shape != (self.num_layers, self.num_kv_heads):
            raise ValueError(f"expected live_counts {(self.num_layers, self.num_kv_heads)}, got {tuple(live_counts.shape)}")
        live_counts = live_counts.to(device=self.device, dtype=torch.int32)
        if not self.paged and bool(torch.any(live_counts > state.range_capacity).item()):
            raise RuntimeError(
                f"compact KV live count {int(live_counts.max().item())} exceeds per-(layer,head) range capacity")
        state.live_counts.copy_(live_counts)

    # ------------------------------------------------------------------ prefill pack
    def streaming_pack_layer(self, *, layer_id: int, k: torch.Tensor, v: torch.Tensor, evict_mask: torch.Tensor,
                             cu_seqlens_q: torch.Tensor, seq_ids: list[int], window_size: int,
                             chunk_starts: list[int] | None = None, remaining: list[int] | None = None) -> None:
        """Packs one layer's post-RoPE K / raw V of a prefill batch into compact spans
        (reference: compact_kv.py:915-1099).  k, v [total_tokens, kv_heads, head_dim];
        evict_mask bool [total_tokens, kv_heads]; cu_seqlens_q int32 [num_seqs + 1].

        Chunked prefill (an extension): `chunk_starts[i]` is the prompt position of sequence i's first
        token in this batch and `remaining[i]` the prompt tokens still to come after it.  The layer's
        spans are first expired with the chunk's last position, then the chunk's kept tokens are
        appended behind the rows the span already holds.  Contiguous spans are reserved at the first
        chunk for the worst case of the rest of the prompt; paged spans grow page by page."""
        _lib.require_cuda(k, v, evict_mask)
        states = []
        for sid in seq_ids:
            st = self.seq_states.get(sid)
            if st is None:
                raise RuntimeError(f"sequence {sid} has no compact KV allocation")
            states.append(st)
        n = len(states)
        if n == 0:
            return
        dev = self.device
        Hk, D = self.num_kv_heads, self.head_dim
        if k.shape != v.shape or k.ndim != 3 or k.shape[1] != Hk or k.shape[2] != D:
            raise ValueError(f"expected k/v as [tokens, {Hk}, {D}], got {tuple(k.shape)} / {tuple(v.shape)}")
        if k.stride(2) != 1 or v.stride() != k.stride():
            k, v = k.contiguous(), v.contiguous()
        if evict_mask.dtype != torch.bool or evict_mask.shape != (k.shape[0], Hk):
            raise ValueError(f"expected bool evict_mask {(k.shape[0], Hk)}, got {tuple(evict_mask.shape)} {evict_mask.dtype}")
        evict_mask = evict_mask.contiguous()
        cu = cu_seqlens_q.to(device=dev, dtype=torch.int32).contiguous()
        cu_host = cu_seqlens_q.tolist() if not cu_seqlens_q.is_cuda else None
        if cu_host is None:
            cu_host = cu.tolist()                                   # one small device read per layer
        max_len = max(cu_host[i + 1] - cu_host[i] for i in range(n))
        max_chunks = max(1, (max_len + PACK_CHUNK - 1) // PACK_CHUNK)
        live = torch.empty((n, Hk), device=dev, dtype=torch.int32)
        chunk_offsets = torch.empty((n, Hk, max_chunks), device=dev, dtype=torch.int32)
        ev_u8 = evict_mask.view(torch.uint8)
        stream = _lib.stream_ptr(dev)
        status = _lib.status_word(dev)
        lib = _lib.lib()
        slots_t = self._slots_tensor(states)
        chunked = chunk_starts is not None
        prior = starts_t = None
        self._free_pages_lb = None                       # a prefill takes pages: the host bound is stale
        if chunked:
            if len(chunk_starts) != n or remaining is None or len(remaining) != n:
                raise ValueError("chunk_starts / remaining need one entry per sequence")
            if any(int(c) > 0 for c in chunk_starts):
                cur = torch.tensor([int(c) + cu_host[i + 1] - cu_host[i] - 1 for i, c in enumerate(chunk_starts)],
                                   dtype=torch.int64).to(dev, non_blocking=True)
                self.expire_device(slots_t, cur, window_size=window_size, layer_id=layer_id)
            starts_t = torch.tensor([int(c) for c in chunk_starts], dtype=torch.int32).to(dev, non_blocking=True)
            prior = self.layer_major_live_counts[layer_id].index_select(0, slots_t.long()).contiguous()
        if self.layer_major_exact_through is not None:
            self.layer_major_exact_through[layer_id].index_fill_(0, slots_t.long(), -1)      # the pack writes slots
        with torch.cuda.device(dev):
            _lib.check(lib.fdms_pack_count(ev_u8.data_ptr(), ev_u8.stride(0), cu.data_ptr(), live.data_ptr(),
                                           chunk_offsets.data_ptr(), max_chunks, n, Hk, int(window_size), stream))
            capacity = self.max_model_len
            if self.paged:
                bt = self.block_tables[layer_id]
                if chunked:
                    after = prior + live
                    _lib.check(lib.fdms_grow_pages(
                        prior.data_ptr(), after.data_ptr(), bt.data_ptr(), bt.stride(0), bt.stride(1), self.max_pages,
                        slots_t.data_ptr(), self.free_pages[layer_id].data_ptr(),
                        self.free_page_counts[layer_id:].data_ptr(), n, Hk, status.data_ptr(), stream))
                else:
                    _lib.check(lib.fdms_alloc_pages(
                        live.data_ptr(), bt.data_ptr(), bt.stride(0), bt.stride(1), self.max_pages,
                        slots_t.data_ptr(), self.free_pages[layer_id].data_ptr(),
                        self.free_page_counts[layer_id:].data_ptr(), n, Hk, status.data_ptr(), stream))
                base_ptr, base_ss = None, 0
                bt_args = (bt.data_ptr(), bt.stride(0), bt.stride(1))
            else:
                live_host = live.tolist()        # the host first-fit allocator needs the counts
                all_bases, all_sizes = [], []
                for i, (st, row) in enumerate(zip(states, live_host)):
                    if chunked and st.host_ranges[layer_id][0] is not None:
                        # a later chunk: the span was reserved for the whole prompt at the first one
                        all_bases.append([r[0] for r in st.host_ranges[layer_id]])
                        all_sizes.append([r[1] for r in st.host_ranges[layer_id]])
                        continue
                    extra = int(remaining[i]) if chunked else 0
                    if max(row) + extra > st.max_capacity_per_lh:
                        raise RuntimeError(
                            f"streaming pack live count {max(row) + extra} exceeds metadata capacity "
                            f"{st.max_capacity_per_lh} (layer {layer_id}, seq {st.seq_id})")
                    b, s = self._reserve_layer(st, layer_id, [r + extra for r in row])
                    all_bases.append(b)
                    all_sizes.append(s)
                hi = max(b + s for bs, ss in zip(all_bases, all_sizes) for b, s in zip(bs, ss))
                self._ensure_layer_storage(layer_id, hi)
                both = torch.tensor([all_bases, all_sizes], dtype=torch.int32).to(dev, non_blocking=True)
                idx = slots_t.long()
                self.layer_major_base_offsets[layer_id].index_copy_(0, idx, both[0])
                self.layer_major_range_capacity[layer_id].index_copy_(0, idx, both[1])
                base_l = self.layer_major_base_offsets[layer_id]
                base_ptr, base_ss = base_l.data_ptr(), base_l.stride(0)
                bt_args = (None, 0, 0)
            pos = self.layer_major_token_positions[layer_id]
            evm = self.layer_major_evict_mask[layer_id].view(torch.uint8)
            lc = self.layer_major_live_counts[layer_id]
            ks, vs = self.layer_scales(layer_id)
            ck, cv = self.compact_k_per_layer[layer_id], self.compact_v_per_layer[layer_id]
            _lib.check(lib.fdms_pack_scatter_append(
                k.data_ptr(), v.data_ptr(), _lib.dtype_code(k.dtype), k.stride(0), k.stride(1),
                ev_u8.data_ptr(), ev_u8.stride(0), cu.data_ptr(),
                chunk_offsets.data_ptr(), max_chunks, live.data_ptr(), _lib.ptr(prior), _lib.ptr(starts_t),
                ck.data_ptr(), cv.data_ptr(), _lib.dtype_code(ck.dtype), ck.shape[0],
                base_ptr, base_ss, *bt_args,
                slots_t.data_ptr(),
                pos.data_ptr(), pos.stride(0), pos.stride(1),
                evm.data_ptr(), evm.stride(0), evm.stride(1),
                lc.data_ptr(), lc.stride(0), capacity,
                _lib.ptr(ks), _lib.ptr(vs),
                n, Hk, D, int(window_size), status.data_ptr(), stream))

    def trim_spans(self, seq_ids: list[int]) -> None:
        """Contiguous spans only: gives back the part of every span that a chunked prefill reserved for
        the worst case and did not fill -- each span shrinks to min(live + decode headroom, C) rows, the
        size a one-pass prefill reserves (reference sizing: compact_kv.py:830-857).  One device read."""
        if self.paged or not seq_ids:
            return
        states = [self.seq_states[sid] for sid in seq_ids if sid in self.seq_states]
        if not states:
            return
        slots = self._slots_tensor(states).long()
        live = self.layer_major_live_counts.index_select(1, slots).cpu()          # [L, n, Hk]
        for i, st in enumerate(states):
            new_cap = torch.zeros((self.num_layers, self.num_kv_heads), dtype=torch.int32)
            for l in range(self.num_layers):
                for h in range(self.num_kv_heads):
                    r = st.host_ranges[l][h]
                    if r is None:
                        continue
                    b, size = r
                    want = max(min(int(live[l, i, h]) + int(st.decode_headroom), st.max_capacity_per_lh), 1)
                    if want < size:
                        self._free_range(l, b + want, size - want)
                        st.host_ranges[l][h] = (b, want)
                        size = want
                    new_cap[l, h] = size
            st.range_capacity.copy_(new_cap.to(self.device, non_blocking=True))

    # ------------------------------------------------------------------ expiry
    def apply_dms_evictions(self, seqs: list[Sequence], current_positions: list[int], *, window_size: int,
                            compact_k=None, compact_v=None, sync_stats: bool = True,
                            expiry_interval: int | None = None, incremental: bool = False) -> dict:
        """Drops evict-marked tokens that left the window and compacts every span in place, all
        layers in one launch (reference: compact_kv.py:1174-1361).  `expiry_interval` > 1 skips
        the launch unless some position is a multiple of it (the reference's windowed cadence,
        :1214-1235); the default comes from the constructor / FASTDMS_DMS_EXPIRY_INTERVAL."""
        if len(seqs) != len(current_positions):
            raise ValueError("seq/current_positions length mismatch")
        zero_stats = {"evicted_tokens": 0, "live_tokens_before_min": 0, "live_tokens_before_max": 0,
                      "live_tokens_after_min": 0, "live_tokens_after_max": 0}
        if not seqs:
            return zero_stats
        states = self._states(seqs)
        interval = expiry_interval if expiry_interval is not None else expiry_interval_from_env(self.dms_expiry_interval)
        sequential = all(st.dms_initial_expiry_done and int(p) == st.last_dms_expiry_position + 1
                         for st, p in zip(states, current_positions))
        for st, p in zip(states, current_positions):
            st.last_dms_expiry_position = int(p)
        if interval > 1 and sequential and not any(int(p) % interval == 0 for p in current_positions):
            if not sync_stats:
                return zero_stats
            lc = self.layer_major_live_counts[:, self._slots_tensor(states).long(), :].to(torch.int64)
            lo, hi = int(lc.min().item()), int(lc.max().item())
            return {"evicted_tokens": 0, "live_tokens_before_min": lo, "live_tokens_before_max": hi,
                    "live_tokens_after_min": lo, "live_tokens_after_max": hi}
        dev = self.device
        cur = torch.tensor([int(p) for p in current_positions], dtype=torch.int64).to(dev, non_blocking=True)
        slots_t = self._slots_tensor(states)
        stats = self._stats_init.clone()
        self.expire_device(slots_t, cur, window_size=window_size, incremental=incremental, stats=stats)
        for st in states:
            st.dms_initial_expiry_done = True
        keys = ("evicted_tokens", "live_tokens_before_min", "live_tokens_before_max",
                "live_tokens_after_min", "live_tokens_after_max")
        if sync_stats:
            return dict(zip(keys, stats.tolist()))
        return {k: stats[i] for i, k in enumerate(keys)}

    def expire_device(self, slots_t: torch.Tensor, cur_positions_t: torch.Tensor, *, window_size: int,
                      incremental: bool = False, stats: torch.Tensor | None = None,
                      layer_id: int | None = None) -> None:
        """The expiry launch itself, on device-resident arguments only (no allocation, no host
        synchronisation; safe inside CUDA-graph capture).  slots_t int32 [n] active slots,
        cur_positions_t int64 [n]; stats optional int64[5] initialised by the caller.  `layer_id`
        restricts the launch to one layer (chunked prefill expires a layer right before it appends
        the chunk to it)."""
        dev = self.device
        ls = slice(None) if layer_id is None else slice(layer_id, layer_id + 1)
        pos, ev = self.layer_major_token_positions[ls], self.layer_major_evict_mask.view(torch.uint8)[ls]
        lc, base = self.layer_major_live_counts[ls], self.layer_major_base_offsets[ls]
        ck, cv = self.compact_k[ls], self.compact_v[ls]
        row_index = None if self.layer_major_row_index is None else self.layer_major_row_index[ls]
        row_bytes = self.head_dim * self.compact_k.element_size()
        if self.paged:
            bt = self.block_tables[ls]
            bt_args = (bt.data_ptr(), bt.stride(0), bt.stride(1), bt.stride(2),
                       self.free_pages[ls].data_ptr(), self.free_page_counts[ls].data_ptr(), self.pages_per_layer)
            base_ptr = None
        else:
            bt_args = (None, 0, 0, 0, None, None, 0)
            base_ptr = base.data_ptr()
        with torch.cuda.device(dev):
            rc = _lib.lib().fdms_expire_compact(
                pos.data_ptr(), pos.stride(0), pos.stride(1), pos.stride(2),
                ev.data_ptr(), ev.stride(0), ev.stride(1), ev.stride(2), _lib.ptr(row_index),
                lc.data_ptr(), base_ptr, lc.stride(0), lc.stride(1),
                ck.data_ptr(), cv.data_ptr(),
                self.compact_k.stride(0) * self.compact_k.element_size(), row_bytes, self.capacity_tokens,
                *bt_args,
                slots_t.data_ptr(), cur_positions_t.data_ptr(),
                pos.shape[0], slots_t.numel(), self.num_kv_heads, self.max_model_len,
                int(window_size), 1 if incremental else 0, _lib.ptr(stats),
                _lib.ptr(None if self.layer_major_exact_through is None else self.layer_major_exact_through[ls]),
                _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc)

    def decode_metadata_device(self, slots_t: torch.Tensor, base_out: torch.Tensor, live_out: torch.Tensor,
                               slot_out: torch.Tensor, cu_out: torch.Tensor | None = None) -> None:
        """The decode-metadata launch on device-resident arguments (capture-safe).  Outputs are
        int32 [layers, batch, kv_heads]; cu_out int32 [layers, batch*kv_heads + 1]."""
        dev = self.device
        lc, base = self.layer_major_live_counts, self.layer_major_base_offsets
        if self.paged:
            bt = self.block_tables
            bt_args = (bt.data_ptr(), bt.stride(0), bt.stride(1), bt.stride(2), self.max_pages,
                       self.free_pages.data_ptr(), self.free_page_counts.data_ptr(), self.pages_per_layer)
            base_ptr = None
        else:
            bt_args = (None, 0, 0, 0, 0, None, None, 0)
            base_ptr = base.data_ptr()
        with torch.cuda.device(dev):
            rc = _lib.lib().fdms_build_decode_metadata(
                lc.data_ptr(), base_ptr, lc.stride(0), lc.stride(1), *bt_args,
                slots_t.data_ptr(), base_out.data_ptr(), live_out.data_ptr(), slot_out.data_ptr(), _lib.ptr(cu_out),
                self.num_layers, slots_t.numel(), self.num_kv_heads,
                _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc)

    def record_device(self, slots_t: torch.Tensor, positions_t: torch.Tensor, evict_all: torch.Tensor,
                      true_count: torch.Tensor | None = None, advance_positions: bool = False) -> None:
        """The decision-recording launch on device-resident arguments (capture-safe).
        positions_t int64 [batch]; evict_all bool [layers, batch, kv_heads], head-contiguous.
        `advance_positions` adds one to every position once all spans are recorded (same launch)."""
        dev = self.device
        pos, ev = self.layer_major_token_positions, self.layer_major_evict_mask.view(torch.uint8)
        lc = self.layer_major_live_counts
        ea = evict_all.view(torch.uint8)
        with torch.cuda.device(dev):
            rc = _lib.lib().fdms_record_decisions(
                pos.data_ptr(), pos.stride(0), pos.stride(1), pos.stride(2),
                ev.data_ptr(), ev.stride(0), ev.stride(1), ev.stride(2),
                lc.data_ptr(), lc.stride(0), lc.stride(1),
                ea.data_ptr(), ea.stride(0), ea.stride(1),
                positions_t.data_ptr(), slots_t.data_ptr(), self.num_layers, slots_t.numel(), self.num_kv_heads,
                self.max_model_len, _lib.ptr(true_count), 1 if advance_positions else 0, _lib.stream_ptr(dev))
        _lib.check(rc)

    # ------------------------------------------------------------------ decode metadata
    def prepare_decode_metadata(self, seqs: list[Sequence]):
        """slot = row of logical index `live` of every (layer, seq, head); live += 1 in place, so
        the forward sees the count that includes the token being appended.  Returns
        (base_offsets, live_counts, slot_mapping, max_capacity), each [layers, batch, kv_heads]
        int32 (reference: compact_kv.py:1727-1770).  No host synchronisation."""
        states = self._states(seqs)
        B = len(states)
        dev = self.device
        L, Hk = self.num_layers, self.num_kv_heads
        bufs = self._decode_buffers.get(B)
        if bufs is None:
            bufs = tuple(torch.empty((L, B, Hk), device=dev, dtype=torch.int32) for _ in range(3)) + (
                torch.empty((L, B * Hk + 1), device=dev, dtype=torch.int32),)
            self._decode_buffers[B] = bufs
        base_out, live_out, slot_out, cu_out = bufs
        self.decode_metadata_device(self._slots_tensor(states), base_out, live_out, slot_out, cu_out)
        self.last_cu_live = cu_out
        return base_out, live_out, slot_out, max(st.max_capacity_per_lh for st in states)

    def decode_block_tables(self, seqs: list[Sequence]) -> torch.Tensor | None:
        """[layers, batch, kv_heads, max_pages] block tables of the batch (paged layout only)."""
        if not self.paged:
            return None
        states = self._states(seqs)
        start = self._contiguous_active_slot_start(states)
        if start is not None:
            return self.block_tables[:, start:start + len(states)]
        return self.block_tables.index_select(1, self._slots_tensor(states).long())

    def record_appended_dms_decisions(self, seqs: list[Sequence], current_positions, layer_evictions,
                                      *, sync_stats: bool = True) -> dict:
        """After the forward: token_positions[l, seq, h, live-1] = position, evict_mask[...] = the
        decision the layer made for the appended token (reference: compact_kv.py:1562-1725)."""
        if len(seqs) != len(current_positions):
            raise ValueError("seq/current_positions length mismatch")
        B = len(seqs)
        if B == 0:
            return {"eviction_decisions_true": 0, "eviction_decisions_total": 0}
        dev = self.device
        L, Hk = self.num_layers, self.num_kv_heads
        if isinstance(layer_evictions, torch.Tensor):
            if tuple(layer_evictions.shape) != (L, B, Hk):
                raise RuntimeError(f"expected DMS decode decisions {(L, B, Hk)}, got {tuple(layer_evictions.shape)}")
            evict_all = layer_evictions
        else:
            rows = []
            for l in range(L):
                e = layer_evictions.get(l)
                if e is None:
                    raise RuntimeError(f"missing DMS decode eviction decisions for layer {l}")
                if tuple(e.shape) != (B, Hk):
                    raise RuntimeError(f"expected DMS decode decisions {(B, Hk)}, got {tuple(e.shape)}")
                rows.append(e)
            evict_all = torch.stack(rows, dim=0)
        evict_all = evict_all.to(device=dev, dtype=torch.bool)
        if evict_all.stride(2) != 1:
            evict_all = evict_all.contiguous()
        if isinstance(current_positions, torch.Tensor):
            if current_positions.numel() != B:
                raise ValueError("current_positions tensor length mismatch")
            pos_t = current_positions.to(device=dev, dtype=torch.int64).contiguous()
        else:
            pos_t = torch.tensor([int(p) for p in current_positions], dtype=torch.int64).to(dev, non_blocking=True)
        states = self._states(seqs)
        slots_t = self._slots_tensor(states)
        true_count = torch.zeros(1, device=dev, dtype=torch.int64)
        self.record_device(slots_t, pos_t, evict_all, true_count)
        total_true = true_count[0]
        return {"eviction_decisions_true": int(total_true.item()) if sync_stats else total_true,
                "eviction_decisions_total": L * B * Hk}

    # ------------------------------------------------------------------ release
    def free(self, seq_id: int) -> None:
        """Returns a sequence's spans / pages and its active slot (reference: compact_kv.py:1772-1795)."""
        state = self.seq_states.pop(seq_id, None)
        if state is None:
            return
        slot = int(state.active_slot)
        if self.paged:
            slot_t = torch.tensor([slot], device=self.device, dtype=torch.int32)
            status = _lib.status_word(self.device)
            with torch.cuda.device(self.device):
                for l in range(self.num_layers):
                    bt = self.block_tables[l]
                    lc = self.layer_major_live_counts[l]
                    _lib.check(_lib.lib().fdms_free_pages(
                        lc.data_ptr(), lc.stride(0), bt.data_ptr(), bt.stride(0), bt.stride(1), self.max_pages,
                        slot_t.data_ptr(), self.free_pages[l].data_ptr(), self.free_page_counts[l:].data_ptr(),
                        self.pages_per_layer, 1, self.num_kv_heads, status.data_ptr(), _lib.stream_ptr(self.device)))
        else:
            for l in range(self.num_layers):
                for h in range(self.num_kv_heads):
                    r = state.host_ranges[l][h]
                    if r is not None and r[0] >= 0 and r[1] > 0:
                        self._free_range(l, r[0], r[1])
        self.active_slot_by_seq.pop(seq_id, None)
        self.layer_major_base_offsets[:, slot, :].fill_(-1)
        self.layer_major_range_capacity[:, slot, :].zero_()
        self.layer_major_live_counts[:, slot, :].zero_()
        if self.layer_major_exact_through is not None:
            self.layer_major_exact_through[:, slot, :].fill_(-1)
        self.layer_major_token_positions[:, slot, :, :state.max_capacity_per_lh].fill_(-1)
        self.layer_major_evict_mask[:, slot, :, :state.max_capacity_per_lh].zero_()
        self.free_active_slots.append(slot)
        self.free_active_slots.sort()

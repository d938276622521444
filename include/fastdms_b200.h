/*
 * fastdms_b200 -- C ABI of the B200-native compact-DMS decode path.
 *
 * One shared library (libfastdms_b200.so) exports every entry point below.  All functions are
 * `extern "C"`, take raw device pointers plus explicit sizes/strides, return an int32 status
 * (0 = ok, < 0 = FDMS_E_*), never throw, never exit and never trap on the device.  The library
 * owns no memory: every buffer (pools, metadata, outputs, workspaces) belongs to the caller.
 * Kernels are enqueued on the CUDA stream passed as `stream` (a cudaStream_t; NULL = default
 * stream) and do not synchronise, allocate or copy to the host, so a sequence of calls can be
 * captured into a CUDA graph as long as the pointers stay stable.
 *
 * The reference project (shisa-ai/FastDMS) has no FFI; the interface each entry point replaces is
 * the Python function / Triton kernel named in its comment (paths inside the reference project).
 *
 * Layouts
 *   pools        K and V pools are row arrays [slots, head_dim] with contiguous rows.  A span of a
 *                (sequence, KV head) is either `live` consecutive rows starting at `base`
 *                (block_tables == NULL, the reference layout) or 16-row pages listed in a block
 *                table: logical row i lives at block_table[i / 16] * 16 + i % 16.
 *   metadata     int32 [batch, kv_heads] (one layer) or [layers, batch, kv_heads]; strides are in
 *                elements.
 *   FP8          e4m3 ("fn": no infinities, max 448) with an optional per-KV-head float scale:
 *                stored = value / scale, value = stored * scale.  scale == NULL means 1.0, which
 *                is the reference's bare cast.
 */
#ifndef FASTDMS_B200_H
#define FASTDMS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FDMS_ABI_VERSION 1

/* status codes */
#define FDMS_OK 0
#define FDMS_E_ARG (-1)         /* bad shape / stride / null pointer: the reference raises ValueError */
#define FDMS_E_DTYPE (-2)       /* unsupported dtype combination: ValueError */
#define FDMS_E_WORKSPACE (-3)   /* workspace missing or too small: ValueError */
#define FDMS_E_CUDA (-4)        /* a CUDA runtime call failed: RuntimeError */
#define FDMS_E_CAPACITY (-5)    /* a size exceeds a documented limit: RuntimeError */

/* dtype codes */
#define FDMS_F32 0
#define FDMS_BF16 1
#define FDMS_F16 2
#define FDMS_E4M3 3

/* bits of the optional device status word (int32, OR-ed by kernels, never cleared by them) */
#define FDMS_DEV_WAIT_TIMEOUT 1   /* a bounded wait on an async copy ran out; results are invalid */
#define FDMS_DEV_BAD_INDEX 2      /* a slot / page index was out of range and the access was skipped */

int32_t fdms_abi_version(void);
/* Message of the last failing call on this host thread (empty string if none). */
const char* fdms_last_error(void);

/* ---------------------------------------------------------------------------------------------
 * (a) compact decode attention.
 * Replaces fastdms/layers/compact_attention.py:1116-1336 compact_decode_attention (split-K partial
 * + reduce kernels :334-603, inline-RoPE variant :418-534).
 *   out[b, hq, :] = softmax(scale * K_span q[b, hq]) V_span   over the span of KV head hq / group.
 * q/out [batch, q_heads, head_dim] with the given element strides (inner stride 1).
 * Optional inline neox RoPE of q at q_rope_positions[b] (int64) with the decision lane
 * (first head of each group, channel head_dim-1) zeroed first; cos_sin rows are
 * [cos(head_dim/2) | sin(head_dim/2)] float32 with row stride cos_sin_stride and cos_sin_rows rows;
 * a position outside [0, cos_sin_rows) raises FDMS_DEV_BAD_INDEX in the status word and is read as 0.
 * block_tables: optional int32 [batch, kv_heads, bt_max_pages] (element strides given).
 * workspace: fdms_attn_decode_workspace_bytes(...) bytes, 256-byte aligned.  Its first
 * `batch*kv_heads` int32 must be zero before the FIRST call; every call leaves them zero again.
 * Calls that share a workspace must not overlap on the GPU.
 * flags: FDMS_ATTN_OVERLAP_PREVIOUS lets the launch begin while the preceding kernel of the stream
 * is still running (programmatic dependent launch).  The caller then promises that the preceding
 * kernel writes none of: live_counts, base_offsets, block_tables, scales, and pool rows other than
 * the LAST live row of each span.  q, that last row and every output are only touched after the
 * preceding kernel has completed.  This is the situation of a decode step, where the preceding
 * kernel is fdms_store_decode of the same layer.
 * --------------------------------------------------------------------------------------------- */
#define FDMS_ATTN_OVERLAP_PREVIOUS 1
int64_t fdms_attn_decode_workspace_bytes(int32_t batch, int32_t num_kv_heads, int32_t head_dim);

int32_t fdms_attn_decode(
    const void* q, int32_t q_dtype, int64_t q_stride_b, int64_t q_stride_h,
    const void* k_pool, const void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, const int32_t* live_counts, int64_t meta_stride_b,
    const int32_t* block_tables, int64_t bt_stride_b, int64_t bt_stride_h, int32_t bt_max_pages,
    const float* k_scale, const float* v_scale,
    void* out, int32_t out_dtype, int64_t out_stride_b, int64_t out_stride_h,
    int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
    const int64_t* q_rope_positions, const float* q_rope_cos_sin, int64_t cos_sin_stride, int64_t cos_sin_rows,
    void* workspace, int64_t workspace_bytes, int32_t flags, int32_t* dev_status, void* stream);

/* Fused decode step of one layer: fdms_store_decode and fdms_attn_decode in ONE launch (the
 * reference keeps them as two kernels, layers/compact_attention.py:1010-1113 and :1116-1336).
 * live_counts must already count the new token (fdms_build_decode_metadata); its row is the last
 * logical row of each span.  Per span, the CTA that owns the last page reads the DMS decision
 * (evict_out, optional), rotates k, quantises k and v exactly like fdms_store_decode, writes the row to
 * the pool and attends to it; every CTA rotates q on the fly (q itself is left untouched, as with
 * store_q = 0).  FP8 e4m3 pools, head_dim 64 or 128, group size <= 8.
 * With FDMS_ATTN_OVERLAP_PREVIOUS the preceding kernel may still be producing q, k and v: they are
 * read after it has completed, pool pages are prefetched before. */
int32_t fdms_attn_decode_append(
    const void* q, const void* k, const void* v, int32_t act_dtype,
    int64_t q_stride_b, int64_t q_stride_h, int64_t k_stride_b, int64_t k_stride_h, int64_t v_stride_b, int64_t v_stride_h,
    void* k_pool, void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, const int32_t* live_counts, int64_t meta_stride_b,
    const int32_t* block_tables, int64_t bt_stride_b, int64_t bt_stride_h, int32_t bt_max_pages,
    const float* k_scale, const float* v_scale,
    const float* cos_sin, int64_t cos_sin_stride, int64_t cos_sin_rows, const int64_t* positions,
    uint8_t* evict_out, int64_t evict_stride_b, double alpha_scale, double alpha_offset,
    void* out, int32_t out_dtype, int64_t out_stride_b, int64_t out_stride_h,
    int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
    void* workspace, int64_t workspace_bytes, int32_t flags, int32_t* dev_status, void* stream);

/* Decode attention with the split-K scratch built into the library, for callers that cannot
 * allocate device memory (no counterpart in the reference, which allocates its partial buffers with
 * torch.empty on every call).  Same arguments and results as fdms_attn_decode without workspace and
 * flags.  Meant for hosts whose device memory was fully handed out at start-up and that forbid later
 * cudaMalloc calls, and for foreign-language runtimes that load this library as a plugin and own no
 * device allocator.  The scratch is a fixed 4,276,224-byte array in the library image, held by every
 * GPU that loads the library until the process exits; limits: batch * kv_heads <= 4096 and
 * head_dim <= 128, beyond which the call fails with FDMS_E_CAPACITY.  Nothing is allocated or freed.
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress): make it
 * outside any stream capture.  All calls share the array and it keeps the previous call's contents;
 * each call clears the counters it needs on its stream, but calls whose kernels overlap on the GPU
 * race on it and must be serialised by the caller. */
int32_t fdms_attn_decode_noalloc(
    const void* q, int32_t q_dtype, int64_t q_stride_b, int64_t q_stride_h,
    const void* k_pool, const void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, const int32_t* live_counts, int64_t meta_stride_b,
    const int32_t* block_tables, int64_t bt_stride_b, int64_t bt_stride_h, int32_t bt_max_pages,
    const float* k_scale, const float* v_scale,
    void* out, int32_t out_dtype, int64_t out_stride_b, int64_t out_stride_h,
    int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
    const int64_t* q_rope_positions, const float* q_rope_cos_sin, int64_t cos_sin_stride, int64_t cos_sin_rows,
    int32_t* dev_status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (b)+(d) fused decode preprocess: DMS decision + RoPE + FP8 quantise + append store.
 * Replaces fastdms/layers/compact_attention.py:1010-1113 fused_dms_rope_store_compact_decode
 * (kernel :67-209); with rope == 0 and evict_out == NULL it is store_compact_kvcache (:968-1007).
 * Per (b, kv head h): v = q[b, h*group, D-1]; evict_out[b,h] = v > offset/scale (scale > 0) else
 * (v*scale - offset) > 0; that lane is zeroed; neox RoPE (float32, no fused multiply-add, result
 * rounded to the activation dtype) of the group's q heads (store_q) and of k (written back when
 * store_k); k (post-RoPE) and v are divided by the head's scale, cast to the pool dtype and
 * written to row slot_mapping[b,h] (negative = skip).  positions: int64 [batch].
 * --------------------------------------------------------------------------------------------- */
int32_t fdms_store_decode(
    void* q, int64_t q_stride_b, int64_t q_stride_h,
    void* k, int64_t k_stride_b, int64_t k_stride_h,
    const void* v, int64_t v_stride_b, int64_t v_stride_h, int32_t act_dtype,
    const float* cos_sin, int64_t cos_sin_stride, int64_t cos_sin_rows, const int64_t* positions,
    void* k_pool, void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* slot_mapping, int64_t slot_stride_b,
    uint8_t* evict_out, int64_t evict_stride_b,
    const float* k_scale, const float* v_scale,
    int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
    double alpha_scale, double alpha_offset,
    int32_t do_decision, int32_t do_rope, int32_t store_q, int32_t store_k,
    int32_t* dev_status, void* stream);

/* Prefill-side decision extraction.  Replaces fastdms/engine/dms.py:152-232
 * extract_dms_eviction_decisions (kernel :12-42): evict[t,h] from q[t, h*group, D-1], lane zeroed. */
int32_t fdms_extract_decisions(
    void* q, int32_t q_dtype, int64_t q_stride_t, int64_t q_stride_h,
    uint8_t* evict_out, int64_t evict_stride_t,
    int64_t tokens, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
    double alpha_scale, double alpha_offset, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (b) expiry: DMS eviction + in-place stable compaction of every (layer, seq, head) span.
 * Replaces fastdms/engine/compact_kv.py:1174-1361 apply_dms_evictions (python path) and
 * fastdms/layers/compact_attention.py:861-965 dms_expiry_one_layer / _incremental_one_layer
 * (kernels :690-858), for all layers in one launch and without the 32768-slot span limit.
 * A slot i < live is kept iff !evict[i] || cur - pos[i] <= window; kept K/V rows, positions and
 * evict bits move to the front in order; [new_live, old_live) of the metadata rows becomes -1 / 0;
 * live_counts is updated.  mode 1 (incremental): only the first slot with evict && pos < cur-window
 * is dropped.  Layer l uses pools k_pool + l*pool_layer_stride_bytes (rows of row_bytes bytes, a
 * multiple of 4) and metadata [layers, seqs, kv_heads(, capacity)] arrays with the given element
 * strides.  With block tables, pages that end up beyond the live prefix are pushed onto the
 * layer's free stack (free_pages int32 [layers, pages_per_layer], free_counts int32 [layers]).
 * seq_slots: optional int32 [num_seqs] rows of the metadata arrays to process (NULL = 0..num_seqs-1);
 * current_positions: int64 [num_seqs].  stats: optional int64[5] {evicted, live_before_min,
 * live_before_max, live_after_min, live_after_max}; the caller initialises it to
 * {0, INT64_MAX, 0, INT64_MAX, 0}.
 * row_index (optional, no counterpart in the reference; int32 with the shape and strides of
 * token_positions): logical slot -> physical row of the span.  When given, positions, evict bits and
 * the index are compacted in order as above, but K/V rows are not shifted: physical rows only stay
 * dense in [0, live) -- a dropped slot's row below the new length is refilled with a row from at or
 * above it, one row copy per dropped slot -- which attention, being independent of row order, reads
 * as before.  Logical row i of the span is then physical row row_index[i]; entries at or beyond
 * live equal their own position (the caller initialises the index to 0, 1, 2, ...), so appending at
 * logical slot live needs no index write.
 * exact_through (optional, with row_index only; int64 with the shape and strides of live_counts, -1 = unknown): the
 * position up to which a span is known to hold no expired slot.  An all-slots call (mode 0) sets it to the call's
 * current position, an incremental call to -1.  A mode-0 call that finds `current position - 1` there inspects only
 * the one slot that can have expired since (decode steps append one token in position order) instead of the whole
 * span; the result is the same.  The caller sets it to -1 whenever it writes slots of a span by other means (pack,
 * release).
 * --------------------------------------------------------------------------------------------- */
int32_t fdms_expire_compact(
    int32_t* token_positions, int64_t pos_stride_l, int64_t pos_stride_s, int64_t pos_stride_h,
    uint8_t* evict_mask, int64_t ev_stride_l, int64_t ev_stride_s, int64_t ev_stride_h,
    int32_t* row_index,
    int32_t* live_counts, const int32_t* base_offsets,
    int64_t meta_stride_l, int64_t meta_stride_s,
    void* k_pool, void* v_pool, int64_t pool_layer_stride_bytes, int32_t row_bytes, int64_t pool_rows,
    int32_t* block_tables, int64_t bt_stride_l, int64_t bt_stride_s, int64_t bt_stride_h,
    int32_t* free_pages, int32_t* free_counts, int64_t pages_per_layer,
    const int32_t* seq_slots, const int64_t* current_positions,
    int32_t num_layers, int32_t num_seqs, int32_t num_kv_heads, int32_t capacity,
    int32_t window, int32_t mode, int64_t* stats, int64_t* exact_through, int32_t* dev_status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (b) prefill pack of one layer, two launches around the span / page allocation.
 * Replaces fastdms/engine/compact_kv.py:915-1099 streaming_pack_layer (kernels :140-262).
 * keep[t,h] = !evict[t,h] || t_in_seq >= max(0, T-1-window).
 * fdms_pack_count : live_out[s,h] = number of kept tokens; chunk_offsets[s,h,c] = exclusive prefix
 *                   of kept tokens before 256-token chunk c (int32 [num_seqs, kv_heads, max_chunks],
 *                   max_chunks >= ceil(longest prompt / 256)).
 * fdms_pack_scatter: kept tokens go to logical row `rank` of their span (row base[s,h]+rank or the
 *                   paged address), divided by the head's scale and cast to the pool dtype;
 *                   positions (index within the prompt) and evict bits are written at [s,h,rank];
 *                   the metadata rows are reset to -1 / 0 beyond live; live_counts[s,h] = live_in.
 * cu_seqlens int32 [num_seqs+1]; k/v [total_tokens, kv_heads, head_dim] activation dtype; metadata
 * arrays are the layer's [seqs, kv_heads(, capacity)] slices; seq_slots maps batch rows to them.
 * --------------------------------------------------------------------------------------------- */
int32_t fdms_pack_count(
    const uint8_t* evict, int64_t evict_stride_t, const int32_t* cu_seqlens,
    int32_t* live_out, int32_t* chunk_offsets, int32_t max_chunks,
    int32_t num_seqs, int32_t num_kv_heads, int32_t window, void* stream);

int32_t fdms_pack_scatter(
    const void* k, const void* v, int32_t act_dtype, int64_t kv_stride_t, int64_t kv_stride_h,
    const uint8_t* evict, int64_t evict_stride_t, const int32_t* cu_seqlens,
    const int32_t* chunk_offsets, int32_t max_chunks, const int32_t* live_in,
    void* k_pool, void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, int64_t base_stride_s,
    const int32_t* block_tables, int64_t bt_stride_s, int64_t bt_stride_h,
    const int32_t* seq_slots,
    int32_t* token_positions, int64_t pos_stride_s, int64_t pos_stride_h,
    uint8_t* evict_mask, int64_t ev_stride_s, int64_t ev_stride_h,
    int32_t* live_counts, int64_t meta_stride_s, int32_t capacity,
    const float* k_scale, const float* v_scale,
    int32_t num_seqs, int32_t num_kv_heads, int32_t head_dim, int32_t window,
    int32_t* dev_status, void* stream);

/* Chunked prefill: the same scatter for a chunk [pos_offsets[s], pos_offsets[s] + T) of a prompt whose
 * earlier chunks already sit in the span (no counterpart in the reference, which packs a prompt in one
 * pass).  prior_live int32 [num_seqs, kv_heads] = rows the span holds before this chunk (after the
 * expiry run with the chunk's last position): kept tokens go to logical rows prior_live + rank, their
 * recorded position is pos_offsets[s] + index within the chunk, live_counts = prior_live + live_in and
 * the metadata rows are reset beyond that.  The keep rule is the chunk-local one of fdms_pack_scatter,
 * which equals the global rule evaluated at the chunk's last position.  NULL prior_live / pos_offsets
 * read as zeros (then the call is fdms_pack_scatter). */
int32_t fdms_pack_scatter_append(
    const void* k, const void* v, int32_t act_dtype, int64_t kv_stride_t, int64_t kv_stride_h,
    const uint8_t* evict, int64_t evict_stride_t, const int32_t* cu_seqlens,
    const int32_t* chunk_offsets, int32_t max_chunks, const int32_t* live_in,
    const int32_t* prior_live, const int32_t* pos_offsets,
    void* k_pool, void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, int64_t base_stride_s,
    const int32_t* block_tables, int64_t bt_stride_s, int64_t bt_stride_h,
    const int32_t* seq_slots,
    int32_t* token_positions, int64_t pos_stride_s, int64_t pos_stride_h,
    uint8_t* evict_mask, int64_t ev_stride_s, int64_t ev_stride_h,
    int32_t* live_counts, int64_t meta_stride_s, int32_t capacity,
    const float* k_scale, const float* v_scale,
    int32_t num_seqs, int32_t num_kv_heads, int32_t head_dim, int32_t window,
    int32_t* dev_status, void* stream);

/* Prefill-tail attention (no counterpart in the reference, whose prefill is one dense pass,
 * fastdms/layers/attention.py:85-92): the queries of a prefill chunk against the rows their span
 * already holds, merged in place with the chunk's own causal attention.
 *   q [total_q, q_heads, head_dim] post-RoPE, cu_seqlens_q int32 [num_seqs+1], max_q_len = longest chunk;
 *   pools / base_offsets / live_counts / block tables / seq_slots / scales as in fdms_attn_decode, the
 *   metadata being the layer's [seqs, kv_heads] slices addressed through seq_slots (live = rows in the
 *   span BEFORE the chunk is packed);
 *   out [total_q, q_heads, head_dim] activation dtype: on entry the normalised causal attention of the
 *   chunk over its own K/V, with dense_lse[h * lse_stride_h + token * lse_stride_t] its natural-log
 *   log-sum-exp of the scaled scores; on return softmax over (span rows + chunk tokens <= query).
 *   dense_lse NULL: out is overwritten with the attention over the span rows alone.  Spans with
 *   live = 0 leave out untouched.  lse_out (optional, same indexing with its own strides) receives
 *   the merged log-sum-exp.  head_dim 64 or 128, at most 8 q heads per KV head. */
int32_t fdms_prefix_attention(
    const void* q, int32_t act_dtype, int64_t q_stride_t, int64_t q_stride_h, const int32_t* cu_seqlens_q,
    int32_t max_q_len, const void* k_pool, const void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, const int32_t* live_counts, int64_t meta_stride_s,
    const int32_t* block_tables, int64_t bt_stride_s, int64_t bt_stride_h, int32_t bt_max_pages,
    const int32_t* seq_slots, const float* k_scale, const float* v_scale,
    void* out, int64_t out_stride_t, int64_t out_stride_h,
    const float* dense_lse, int64_t lse_stride_h, int64_t lse_stride_t,
    float* lse_out, int64_t lse_out_stride_h, int64_t lse_out_stride_t,
    int32_t num_seqs, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
    int32_t* dev_status, void* stream);

/* Page allocator of the paged layout (no counterpart in the reference, whose spans are contiguous
 * ranges handed out by a host first-fit list, fastdms/engine/compact_kv.py:705-737).
 * fdms_alloc_pages pops ceil(rows_needed[s,h] / 16) pages per span from one layer's free stack into
 * its block-table row; fdms_free_pages pushes every page of the listed spans back and clears the
 * rows.  block_tables is the layer's [seqs, kv_heads, max_pages] slice. */
int32_t fdms_alloc_pages(
    const int32_t* rows_needed, int32_t* block_tables, int64_t bt_stride_s, int64_t bt_stride_h,
    int32_t max_pages, const int32_t* seq_slots, int32_t* free_pages, int32_t* free_count,
    int32_t num_seqs, int32_t num_kv_heads, int32_t* dev_status, void* stream);
/* fdms_grow_pages: pops the pages with indices [ceil(rows_before/16), ceil(rows_after/16)) of every
 * listed span (chunked prefill appends to spans that already hold rows). */
int32_t fdms_grow_pages(
    const int32_t* rows_before, const int32_t* rows_after, int32_t* block_tables, int64_t bt_stride_s,
    int64_t bt_stride_h, int32_t max_pages, const int32_t* seq_slots, int32_t* free_pages, int32_t* free_count,
    int32_t num_seqs, int32_t num_kv_heads, int32_t* dev_status, void* stream);
int32_t fdms_free_pages(
    const int32_t* live_counts, int64_t meta_stride_s, int32_t* block_tables, int64_t bt_stride_s,
    int64_t bt_stride_h, int32_t max_pages, const int32_t* seq_slots, int32_t* free_pages,
    int32_t* free_count, int64_t pages_per_layer, int32_t num_seqs, int32_t num_kv_heads,
    int32_t* dev_status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (c) ragged-batch decode metadata for all layers in one launch.
 * Replaces fastdms/engine/compact_kv.py:1727-1770 prepare_decode_metadata.  For every
 * (layer, batch row b -> metadata row seq_slots[b], head): base_out = base; slot_out = physical
 * row of logical index `live` (base+live, or through the block table; when live is a multiple of
 * 16 and block tables are used a page is popped from the layer's free stack first);
 * live += 1 in the manager's array and live_out = the incremented value.  cu_live_out (optional,
 * int32 [layers, batch*kv_heads + 1]) receives the exclusive prefix sum of live_out per layer.
 * free_pages int32 [layers, pages_per_layer], free_counts int32 [layers]: per-layer stacks of
 * free page ids (only with block tables).
 * --------------------------------------------------------------------------------------------- */
int32_t fdms_build_decode_metadata(
    int32_t* live_counts, const int32_t* base_offsets, int64_t meta_stride_l, int64_t meta_stride_s,
    int32_t* block_tables, int64_t bt_stride_l, int64_t bt_stride_s, int64_t bt_stride_h, int32_t max_pages,
    int32_t* free_pages, int32_t* free_counts, int64_t pages_per_layer,
    const int32_t* seq_slots,
    int32_t* base_out, int32_t* live_out, int32_t* slot_out, int32_t* cu_live_out,
    int32_t num_layers, int32_t batch, int32_t num_kv_heads, int32_t* dev_status, void* stream);

/* Replaces fastdms/engine/compact_kv.py:1562-1725 record_appended_dms_decisions (kernel :426-484):
 * token_positions[l, slot, h, live-1] = positions[b]; evict_mask[...] = evict_all[l,b,h];
 * true_count (optional int64, caller-zeroed) accumulates the number of true decisions.
 * advance_positions != 0 (no counterpart in the reference): after every span has been recorded,
 * positions[b] += 1 for the whole batch, in the same launch -- for callers that keep the step's
 * positions on the device across steps. */
int32_t fdms_record_decisions(
    int32_t* token_positions, int64_t pos_stride_l, int64_t pos_stride_s, int64_t pos_stride_h,
    uint8_t* evict_mask, int64_t ev_stride_l, int64_t ev_stride_s, int64_t ev_stride_h,
    const int32_t* live_counts, int64_t meta_stride_l, int64_t meta_stride_s,
    const uint8_t* evict_all, int64_t ea_stride_l, int64_t ea_stride_b,
    int64_t* positions, const int32_t* seq_slots,
    int32_t num_layers, int32_t batch, int32_t num_kv_heads, int32_t capacity,
    int64_t* true_count, int32_t advance_positions, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (d) FP8 e4m3 KV quantise / dequantise with a per-KV-head scale, x [n, kv_heads, head_dim].
 * The reference's equivalent is the bare cast `.to(float8_e4m3fn)` (fastdms/engine/compact_kv.py:
 * 1085-1087), i.e. scale == NULL.  Round to nearest even, saturating at +-448.
 * --------------------------------------------------------------------------------------------- */
int32_t fdms_kv_quant(const void* x, int32_t x_dtype, uint8_t* out, const float* scale,
                      int64_t n, int32_t num_kv_heads, int32_t head_dim, void* stream);
int32_t fdms_kv_dequant(const uint8_t* x, void* out, int32_t out_dtype, const float* scale,
                        int64_t n, int32_t num_kv_heads, int32_t head_dim, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Callers either side of the path inside a decoder block (decode steps are launch-bound, so these
 * are single launches instead of the reference's chains of torch ops under torch.compile).
 * 16-bit activations (FDMS_BF16 / FDMS_F16) only; pointers and row strides 16-byte aligned.
 *
 * fdms_rmsnorm: RMSNorm.rms_forward / add_rms_forward (fastdms/layers/layernorm.py:16-48).
 *   xf = float(x) (+ float(residual));  residual_out = round(xf) (optional);
 *   out = round(round(xf * rsqrt(mean(xf^2) + eps)) * weight).   hidden % 8 == 0, hidden <= 8192.
 *   out may alias x, residual_out may alias residual.
 * fdms_silu_and_mul: SiluAndMul (fastdms/layers/activation.py): out[r, c] = silu(x[r, c]) * x[r, n + c].
 * --------------------------------------------------------------------------------------------- */
int32_t fdms_rmsnorm(
    const void* x, int64_t x_row_stride, const void* residual, int64_t residual_row_stride, const void* weight,
    void* out, int64_t out_row_stride, void* residual_out, int64_t residual_out_row_stride,
    int32_t dtype, int64_t rows, int32_t hidden, float eps, void* stream);
int32_t fdms_silu_and_mul(const void* x, int64_t x_row_stride, void* out, int64_t out_row_stride,
                          int32_t dtype, int64_t rows, int32_t n, void* stream);
/* Per-head RMSNorm of q and k before RoPE (the Qwen3 attention block: fastdms/models/qwen3.py applies
 * RMSNorm(head_dim) to q.view(-1, heads, head_dim) and k.view(-1, kv_heads, head_dim), two calls of
 * layernorm.py:16-25), both in ONE launch and in place: q [rows, q_heads, head_dim] and k [rows, k_heads, head_dim]
 * with the given row and head strides in elements (views into the fused qkv projection output), inner stride 1.
 * Same arithmetic as fdms_rmsnorm.  head_dim % 8 == 0, head_dim <= 256, 16-byte aligned pointers and strides. */
int32_t fdms_qk_rmsnorm(
    void* q, int64_t q_stride_row, int64_t q_stride_head, int32_t q_heads, const void* q_weight,
    void* k, int64_t k_stride_row, int64_t k_stride_head, int32_t k_heads, const void* k_weight,
    int32_t dtype, int64_t rows, int32_t head_dim, float eps, void* stream);

/* Decode-sized linear layer: y[rows, out] = x[rows, in] * weight[out, in]^T (+ bias), rows <= 8, the
 * weight streamed once from HBM (the reference calls F.linear -> cuBLAS for qkv_proj, o_proj,
 * gate_up_proj, down_proj and the LM head, fastdms/layers/linear.py:635-662, 1044-1048,
 * fastdms/layers/embed_head.py).  dtype FDMS_BF16 / FDMS_F16 for x, weight, bias and y; f32
 * accumulation, one rounding at the end; row strides in elements; out % 16 == 0, in % 2048 == 0,
 * x and weight rows 16-byte aligned.  bias may be NULL. */
int32_t fdms_linear_decode(const void* x, int64_t x_row_stride, const void* weight, int64_t w_row_stride,
                           const void* bias, void* y, int64_t y_row_stride, int32_t dtype, int32_t rows,
                           int32_t out_features, int32_t in_features, void* stream);
/* The gate_up projection of a gated MLP with its activation in one launch (the reference runs F.linear and then
 * SiluAndMul, fastdms/models/llama.py MLP.forward, fastdms/layers/activation.py):
 *   y[rows, out/2] = round(round(silu(g)) * u),  g = round(x W[:out/2]^T + b[:out/2]),  u = round(x W[out/2:]^T + b[out/2:]),
 * bit for bit what fdms_linear_decode followed by fdms_silu_and_mul gives.  Same limits as fdms_linear_decode;
 * out_features (gate and up together) % 32 == 0. */
int32_t fdms_linear_decode_gated(const void* x, int64_t x_row_stride, const void* weight, int64_t w_row_stride,
                                 const void* bias, void* y, int64_t y_row_stride, int32_t dtype, int32_t rows,
                                 int32_t out_features, int32_t in_features, void* stream);

/* The same with the decoder block's RMSNorm (+ residual add) in front (the reference runs
 * RMSNorm.add_rms_forward, fastdms/layers/layernorm.py:16-48, then F.linear):
 *   xf = float(x) (+ float(residual));  residual_out = round(xf) (optional, must not alias x / residual);
 *   y = round(round(xf * rsqrt(mean(xf^2) + eps)) * norm_weight) * weight^T (+ bias).
 * residual may be NULL (first layer).  Same shape and alignment rules; norm_weight has in_features elements. */
int32_t fdms_linear_decode_norm(
    const void* x, int64_t x_row_stride, const void* residual, int64_t residual_row_stride, const void* norm_weight,
    float eps, void* residual_out, int64_t residual_out_row_stride, const void* weight, int64_t w_row_stride,
    const void* bias, void* y, int64_t y_row_stride, int32_t dtype, int32_t rows, int32_t out_features,
    int32_t in_features, void* stream);

/* Greedy head: out[r] = index of the largest of x[r, 0..n) -- `logits.argmax(dim=-1)` of the
 * temperature-0 path (fastdms/engine/model_runner.py:1147-1151; the reference fuses it for one
 * sequence only, fastdms/layers/embed_head.py:491-543).  Lowest index on ties, a NaN counts as the
 * largest value (torch's convention).  dtype FDMS_F32 / FDMS_BF16 / FDMS_F16; row_stride in
 * elements; rows < 65536, n < 2^32 - 1.  One launch, no host synchronisation.  `workspace`
 * (fdms_argmax_workspace_bytes(rows) bytes, 8-byte aligned) must be zero before the FIRST call; every
 * call leaves it zero again, so calls on one stream can share it. */
int64_t fdms_argmax_workspace_bytes(int64_t rows);
int32_t fdms_argmax_rows(const void* x, int64_t row_stride, int32_t dtype, int64_t rows, int64_t n,
                         int64_t* out, void* workspace, int64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (e) tensor parallel by KV head: the all-reduce after o_proj and down_proj
 * (fastdms/layers/linear.py:1044-1048 calls NCCL's all_reduce).  One-shot all-reduce over NVLink peer
 * memory for tensors of at most max_bytes: every rank pushes its input into a slot of every peer's region,
 * each 32-bit word next to the call's epoch (so a word carries its own "ready" mark: no fence, no flag), reads
 * the slots the peers pushed into its own region, waiting (bounded) for words of an older epoch, and sums all
 * inputs in rank order, so every rank gets the same bits.  peer_regions[r] is rank r's region of
 * fdms_allreduce_region_bytes(world, max_bytes) bytes, zero-filled once before the first call and
 * mapped into this process with fdms_ipc_region_open; the same call sequence must run on every rank.  in/out: n
 * elements of dtype (FDMS_F32 / FDMS_BF16 / FDMS_F16), 16-byte aligned, n * size a multiple of 16.
 * A peer that does not answer within about a second raises FDMS_DEV_WAIT_TIMEOUT and is left out; after that
 * the region must not be used again (the ranks' call counters may disagree): re-create it collectively.
 * --------------------------------------------------------------------------------------------- */
int64_t fdms_allreduce_region_bytes(int32_t world, int64_t max_bytes);
/* Peer regions (the one place this library allocates: the caller owns the result and destroys it).
 * create: a zero-filled device allocation of `bytes` on the current device and its 64-byte CUDA IPC
 * handle, to be sent to the peers.  open: maps a peer's region into the CURRENT device's address space
 * (call it with the rank's own device current: a mapping opened under another device is not reachable
 * from this device's kernels).  close / destroy undo open / create. */
int32_t fdms_ipc_region_create(int64_t bytes, void** ptr, void* handle64);
int32_t fdms_ipc_region_open(const void* handle64, void** ptr);
int32_t fdms_ipc_region_close(void* ptr);
int32_t fdms_ipc_region_destroy(void* ptr);
/* Enables peer access from the current device to peer_device (the direction the kernel's loads and
 * stores take; mapping a peer's region through CUDA IPC does not enable it).  Call once per peer,
 * with the rank's own device current, before the first fdms_allreduce_oneshot. */
int32_t fdms_enable_peer_access(int32_t peer_device);
int32_t fdms_allreduce_oneshot(
    void* const* peer_regions, int32_t rank, int32_t world, int64_t max_bytes,
    const void* in, void* out, int64_t n, int32_t dtype, int32_t* dev_status, void* stream);

/* The decode-sized linear layer with FP8 (e4m3) weights and one float32 scale per output column:
 * y = (x W8^T) * scale (+ bias); x and y 16-bit, weight_e4m3 [out_features, in_features] bytes with
 * 16-byte aligned rows, in_features % 2048 == 0, out_features % 16 == 0, rows <= 8.  Weight-only
 * quantisation: the bytes are converted exactly to f16 in registers and accumulated in float32 (the
 * reference's opt-in FP8 weight path, fastdms/layers/linear.py:548-662, also quantises the activations and
 * calls torch._scaled_mm). */
int32_t fdms_linear_decode_fp8(const void* x, int64_t x_row_stride, const void* weight_e4m3, int64_t w_row_stride,
                               const float* scale, const void* bias, void* y, int64_t y_row_stride, int32_t dtype,
                               int32_t rows, int32_t out_features, int32_t in_features, void* stream);

/* Row-parallel linear layer fused with its all-reduce, for decode-sized inputs (rows <= 8):
 *   y = sum over ranks of x_r W_r^T (+ bias), one kernel per rank instead of F.linear + NCCL all_reduce
 * (fastdms/layers/linear.py:1044-1048, the o_proj / down_proj call sites).  Every CTA pushes its float32
 * partial tile into a slot of each peer's mapped region (plain peer stores of {value, epoch} pairs: a value
 * carries its own "ready" mark, so there is no fence and no flag), waits (bounded) for the peers' values of this
 * call in its own region and sums the ranks' partials in rank order: identical bits on every rank, one rounding.  x [rows, in_features] and weight
 * [out_features, in_features] are this rank's shards (bf16 or f16, rows 16-byte aligned,
 * in_features % 256 == 0, out_features % 16 == 0, at most 512 CTAs: out_features <= 8192 for
 * in_features >= 2048); bias (may be null) is added once, pass the same vector on every rank.
 * peer_regions[r]: rank r's region of fdms_linear_allreduce_region_bytes(world) bytes, zero-filled once,
 * mapped with fdms_ipc_region_open; the same call sequence must run on every rank.  A peer that does not
 * answer within about a second raises FDMS_DEV_WAIT_TIMEOUT and is left out of the sum; after that the
 * region must not be used again (re-create it collectively). */
int64_t fdms_linear_allreduce_region_bytes(int32_t world);
int32_t fdms_linear_decode_allreduce(
    const void* x, int64_t x_row_stride, const void* weight, int64_t w_row_stride, const void* bias,
    void* y, int64_t y_row_stride, int32_t dtype, int32_t rows, int32_t out_features, int32_t in_features,
    void* const* peer_regions, int32_t rank, int32_t world, int32_t* dev_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FASTDMS_B200_H */

// Prefill pack: keep-mask, rank and scatter of post-RoPE K / raw V into compact spans.
//
// Two launches around the host-side span allocation (the allocator needs the live counts):
//   pack_count  : one CTA per (sequence, KV head) walks the prompt in 256-token chunks and writes
//                 the exclusive prefix of kept tokens per chunk plus the total.
//   pack_scatter: one CTA per (chunk, KV head, sequence) recomputes the chunk's keep flags, ranks
//                 them locally and copies the kept rows (cast to the pool dtype) to
//                 logical row chunk_offset + local_rank of the span.
// Only kept rows are read from the dense K/V activations.
#include "common.cuh"

namespace fdms {

constexpr int kPackThreads = 256;   // also the chunk length in tokens

__device__ __forceinline__ bool pack_keep(const uint8_t* evict, int64_t ev_st, int64_t tok0, int t, int T,
                                          int h, int window) {
    if (t >= T) return false;
    const int thr = max(0, T - 1 - window);
    return evict[(tok0 + t) * ev_st + h] == 0 || t >= thr;
}

__global__ void __launch_bounds__(kPackThreads) pack_count_kernel(
    const uint8_t* evict, int64_t ev_st, const int32_t* cu, int32_t* live_out, int32_t* chunk_offsets,
    int max_chunks, int hk, int window) {
    __shared__ int s_warp[kPackThreads / 32];
    const int s = blockIdx.x / hk, h = blockIdx.x % hk;
    const int64_t tok0 = cu[s];
    const int T = cu[s + 1] - cu[s];
    int running = 0;
    int32_t* offs = chunk_offsets + ((int64_t)s * hk + h) * max_chunks;
    const int nchunks = (T + kPackThreads - 1) / kPackThreads;
    for (int c = 0; c < nchunks && c < max_chunks; ++c) {
        const bool keep = pack_keep(evict, ev_st, tok0, c * kPackThreads + threadIdx.x, T, h, window);
        const unsigned b = __ballot_sync(0xffffffffu, keep);
        if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = __popc(b);
        __syncthreads();
        int total = 0;
#pragma unroll
        for (int w = 0; w < kPackThreads / 32; ++w) total += s_warp[w];
        if (threadIdx.x == 0) offs[c] = running;
        running += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) live_out[s * hk + h] = running;
}

struct ScatterParams {
    const void* k; const void* v; int act_dtype; int64_t kv_st, kv_sh;
    const uint8_t* evict; int64_t ev_st; const int32_t* cu;
    const int32_t* chunk_offsets; int max_chunks;
    const int32_t* live_in;
    const int32_t* prior_live; const int32_t* pos_offsets;   // chunked prefill: rows already in the span, first position
    void* k_pool; void* v_pool; int kv_dtype; int64_t pool_rows;
    const int32_t* base; int64_t base_ss;
    const int32_t* bt; int64_t bt_ss, bt_sh;
    const int32_t* seq_slots;
    int32_t* pos; int64_t pos_ss, pos_sh;
    uint8_t* evm; int64_t ev_ss, ev_sh;
    int32_t* live; int64_t meta_ss; int capacity;
    const float* k_scale; const float* v_scale;
    int hk, dim, window;
    int32_t* dev_status;
};

__global__ void __launch_bounds__(kPackThreads) pack_scatter_kernel(ScatterParams p) {
    __shared__ int s_warp[kPackThreads / 32];
    __shared__ int s_src[kPackThreads];
    const int c = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int srow = p.seq_slots ? p.seq_slots[s] : s;
    const int64_t tok0 = p.cu[s];
    const int T = p.cu[s + 1] - p.cu[s];
    const int prior = p.prior_live ? p.prior_live[s * p.hk + h] : 0;
    const int pos0 = p.pos_offsets ? p.pos_offsets[s] : 0;
    const int live = prior + p.live_in[s * p.hk + h];
    int32_t* pos = p.pos + (int64_t)srow * p.pos_ss + (int64_t)h * p.pos_sh;
    uint8_t* evm = p.evm + (int64_t)srow * p.ev_ss + (int64_t)h * p.ev_sh;

    // Reset the metadata row beyond the live prefix; the chunks share the work.
    {
        const int per = (p.capacity + gridDim.x - 1) / gridDim.x;
        const int lo = max(live, c * per), hi = min(p.capacity, (c + 1) * per);
        for (int i = lo + tid; i < hi; i += kPackThreads) { pos[i] = -1; evm[i] = 0; }
    }
    if (c == 0 && tid == 0) p.live[(int64_t)srow * p.meta_ss + h] = live;
    if (c * kPackThreads >= T) return;

    const int t = c * kPackThreads + tid;
    const bool keep = pack_keep(p.evict, p.ev_st, tok0, t, T, h, p.window);
    const unsigned ballot = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kPackThreads / 32; ++w) {
        if (w < warp) before += s_warp[w];
        total += s_warp[w];
    }
    const int chunk_off = prior + p.chunk_offsets[((int64_t)s * p.hk + h) * p.max_chunks + c];
    const int r = before + __popc(ballot & ((1u << lane) - 1u));
    if (keep) {
        s_src[r] = t;
        const int idx = chunk_off + r;
        if (idx < p.capacity) {
            pos[idx] = pos0 + t;
            evm[idx] = p.evict[(tok0 + t) * p.ev_st + h];
        } else if (p.dev_status) {
            atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
        }
    }
    __syncthreads();

    const int base = p.base ? p.base[(int64_t)srow * p.base_ss + h] : 0;
    const int32_t* bt = p.bt ? p.bt + (int64_t)srow * p.bt_ss + (int64_t)h * p.bt_sh : nullptr;
    const float ks = p.k_scale ? p.k_scale[h] : 1.0f;
    const float vs = p.v_scale ? p.v_scale[h] : 1.0f;
    for (int j = warp; j < total; j += kPackThreads / 32) {
        const int src_t = s_src[j];
        const int64_t row = span_row(base, bt, chunk_off + j);
        if (row < 0 || row >= p.pool_rows) {
            if (lane == 0 && p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
            continue;
        }
        const int64_t src = (tok0 + src_t) * p.kv_st + (int64_t)h * p.kv_sh;
        for (int d = lane; d < p.dim; d += 32) {
            float kx = load_as_float(p.k, src + d, p.act_dtype);
            float vx = load_as_float(p.v, src + d, p.act_dtype);
            if (p.k_scale) kx = __fdiv_rn(kx, ks);
            if (p.v_scale) vx = __fdiv_rn(vx, vs);
            store_from_float(p.k_pool, row * p.dim + d, p.kv_dtype, kx);
            store_from_float(p.v_pool, row * p.dim + d, p.kv_dtype, vx);
        }
    }
}

}  // namespace fdms

using namespace fdms;

extern "C" int32_t fdms_pack_count(
    const uint8_t* evict, int64_t evict_stride_t, const int32_t* cu_seqlens,
    int32_t* live_out, int32_t* chunk_offsets, int32_t max_chunks,
    int32_t num_seqs, int32_t num_kv_heads, int32_t window, void* stream) {
    clear_error();
    FDMS_REQUIRE(evict && cu_seqlens && live_out && chunk_offsets, FDMS_E_ARG, "fdms_pack_count: null pointer");
    FDMS_REQUIRE(num_seqs >= 0 && num_kv_heads > 0 && max_chunks > 0, FDMS_E_ARG, "fdms_pack_count: bad sizes");
    FDMS_REQUIRE(window >= 0, FDMS_E_ARG, "window_size must be non-negative, got %d", window);
    if (num_seqs == 0) return FDMS_OK;
    pack_count_kernel<<<num_seqs * num_kv_heads, kPackThreads, 0, (cudaStream_t)stream>>>(
        evict, evict_stride_t, cu_seqlens, live_out, chunk_offsets, max_chunks, num_kv_heads, window);
    FDMS_CHECK_LAUNCH("pack_count_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_pack_scatter_append(
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
    int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(k && v && evict && cu_seqlens && chunk_offsets && live_in && k_pool && v_pool &&
                     token_positions && evict_mask && live_counts,
                 FDMS_E_ARG, "fdms_pack_scatter: null pointer");
    FDMS_REQUIRE(base_offsets || block_tables, FDMS_E_ARG, "fdms_pack_scatter: base_offsets or block_tables required");
    FDMS_REQUIRE(act_dtype == FDMS_F32 || act_dtype == FDMS_BF16 || act_dtype == FDMS_F16, FDMS_E_DTYPE,
                 "fdms_pack_scatter: activation dtype %d not supported", act_dtype);
    FDMS_REQUIRE(kv_dtype >= FDMS_F32 && kv_dtype <= FDMS_E4M3, FDMS_E_DTYPE,
                 "fdms_pack_scatter: pool dtype %d not supported", kv_dtype);
    FDMS_REQUIRE(num_seqs >= 0 && num_kv_heads > 0 && head_dim > 0 && max_chunks > 0 && capacity > 0,
                 FDMS_E_ARG, "fdms_pack_scatter: bad sizes");
    FDMS_REQUIRE(num_seqs <= 65535 && num_kv_heads <= 65535, FDMS_E_CAPACITY, "fdms_pack_scatter: grid too large");
    if (num_seqs == 0) return FDMS_OK;
    ScatterParams p;
    p.k = k; p.v = v; p.act_dtype = act_dtype; p.kv_st = kv_stride_t; p.kv_sh = kv_stride_h;
    p.evict = evict; p.ev_st = evict_stride_t; p.cu = cu_seqlens;
    p.chunk_offsets = chunk_offsets; p.max_chunks = max_chunks; p.live_in = live_in;
    p.prior_live = prior_live; p.pos_offsets = pos_offsets;
    p.k_pool = k_pool; p.v_pool = v_pool; p.kv_dtype = kv_dtype; p.pool_rows = pool_rows;
    p.base = base_offsets; p.base_ss = base_stride_s;
    p.bt = block_tables; p.bt_ss = bt_stride_s; p.bt_sh = bt_stride_h;
    p.seq_slots = seq_slots;
    p.pos = token_positions; p.pos_ss = pos_stride_s; p.pos_sh = pos_stride_h;
    p.evm = evict_mask; p.ev_ss = ev_stride_s; p.ev_sh = ev_stride_h;
    p.live = live_counts; p.meta_ss = meta_stride_s; p.capacity = capacity;
    p.k_scale = k_scale; p.v_scale = v_scale;
    p.hk = num_kv_heads; p.dim = head_dim; p.window = window; p.dev_status = dev_status;
    dim3 grid(max_chunks, num_kv_heads, num_seqs);
    pack_scatter_kernel<<<grid, kPackThreads, 0, (cudaStream_t)stream>>>(p);
    FDMS_CHECK_LAUNCH("pack_scatter_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_pack_scatter(
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
    int32_t* dev_status, void* stream) {
    return fdms_pack_scatter_append(
        k, v, act_dtype, kv_stride_t, kv_stride_h, evict, evict_stride_t, cu_seqlens, chunk_offsets, max_chunks, live_in,
        nullptr, nullptr, k_pool, v_pool, kv_dtype, pool_rows, base_offsets, base_stride_s, block_tables, bt_stride_s,
        bt_stride_h, seq_slots, token_positions, pos_stride_s, pos_stride_h, evict_mask, ev_stride_s, ev_stride_h,
        live_counts, meta_stride_s, capacity, k_scale, v_scale, num_seqs, num_kv_heads, head_dim, window, dev_status, stream);
}

// DMS expiry: eviction of window-expired tokens and in-place stable compaction of every
// (layer, sequence, KV head) span, all layers in one launch.
//
// One CTA owns one span and sweeps it left to right in tiles of 256 slots.  For a kept slot the
// destination index (its rank among kept slots) is never larger than its source index, so an
// ordered sweep in which every tile finishes its loads before it stores can never overwrite a
// row that is still to be read.  Tiles in which nothing moves (no slot dropped so far) cost one
// 5-byte metadata read per slot and no K/V traffic.  Spans of any length are supported.
//
// HBM traffic per span: live * 5 B of metadata + 2 * row_bytes * (rows behind the first dropped
// slot), read and written once.
#include <limits.h>

#include "common.cuh"

namespace fdms {

constexpr int kExpiryThreads = 256;
constexpr int kMoveRegs = 4;   // 16-byte (or 4-byte) chunks staged per thread and pool per sub-tile

struct ExpiryParams {
    int32_t* pos; int64_t pos_sl, pos_ss, pos_sh;
    uint8_t* ev; int64_t ev_sl, ev_ss, ev_sh;
    int32_t* live; const int32_t* base; int64_t meta_sl, meta_ss;
    uint8_t* k_pool; uint8_t* v_pool; int64_t pool_layer_bytes; int row_bytes; int64_t pool_rows;
    int32_t* bt; int64_t bt_sl, bt_ss, bt_sh;
    int32_t* free_pages; int32_t* free_counts; int64_t pages_per_layer;
    const int32_t* seq_slots; const int64_t* cur;
    int layers, seqs, hk, capacity, window, mode;
    long long* stats; int32_t* dev_status;
};

// Exclusive scan of one flag per thread over the CTA; returns this thread's rank and the total.
__device__ __forceinline__ int block_scan_flags(bool flag, int* total, int* s_warp) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned ballot = __ballot_sync(0xffffffffu, flag);
    const int in_warp = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, sum = 0;
#pragma unroll
    for (int w = 0; w < kExpiryThreads / 32; ++w) {
        const int c = s_warp[w];
        if (w < warp) before += c;
        sum += c;
    }
    __syncthreads();
    *total = sum;
    return before + in_warp;
}

template <typename VecT>
__global__ void __launch_bounds__(kExpiryThreads) expire_compact_kernel(ExpiryParams p) {
    __shared__ int s_kept[kExpiryThreads];
    __shared__ int s_warp[kExpiryThreads / 32];
    __shared__ int s_first;

    const int item = blockIdx.x;
    const int h = item % p.hk;
    const int sidx = (item / p.hk) % p.seqs;
    const int l = item / (p.hk * p.seqs);
    const int srow = p.seq_slots ? p.seq_slots[sidx] : sidx;
    const int tid = threadIdx.x;

    const int64_t moff = (int64_t)l * p.meta_sl + (int64_t)srow * p.meta_ss + h;
    const int old_live = p.live[moff];
    const int base = p.base ? p.base[moff] : 0;
    const int32_t* bt = p.bt ? p.bt + (int64_t)l * p.bt_sl + (int64_t)srow * p.bt_ss + (int64_t)h * p.bt_sh : nullptr;
    int32_t* pos = p.pos + (int64_t)l * p.pos_sl + (int64_t)srow * p.pos_ss + (int64_t)h * p.pos_sh;
    uint8_t* ev = p.ev + (int64_t)l * p.ev_sl + (int64_t)srow * p.ev_ss + (int64_t)h * p.ev_sh;
    const long long cur = p.cur[sidx];
    int live = old_live;
    if (live > p.capacity) live = p.capacity;      // never walk past the metadata row
    const bool active = live > 0 && (bt != nullptr || base >= 0);

    int new_live = active ? 0 : old_live;
    if (active) {
        // Pre-pass without block-wide scans: index of the first slot that gets dropped
        // (evict-marked and out of the window).  Everything before it stays where it is, so the
        // compaction sweep can start at that slot's tile; in steady-state decode that is the last
        // tile or two of the span, and a span with nothing to drop costs only this pass.
        if (tid == 0) s_first = INT_MAX;
        __syncthreads();
        for (int t0 = 0; t0 < live; t0 += kExpiryThreads) {
            const int i = t0 + tid;
            bool expired = false;
            if (i < live) expired = ev[i] != 0 && (long long)pos[i] < cur - p.window;
            const unsigned any = __ballot_sync(0xffffffffu, expired);
            if (any && (tid & 31) == 0) atomicMin(&s_first, t0 + (tid & ~31) + __ffs(any) - 1);
        }
        __syncthreads();
        const int first = s_first;
        const int t_start = first == INT_MAX ? live : (first / kExpiryThreads) * kExpiryThreads;

        uint8_t* kp = p.k_pool + (int64_t)l * p.pool_layer_bytes;
        uint8_t* vp = p.v_pool + (int64_t)l * p.pool_layer_bytes;
        const int chunks = p.row_bytes / (int)sizeof(VecT);
        int run = min(t_start, live);
        for (int t0 = t_start; t0 < live; t0 += kExpiryThreads) {
            const int i = t0 + tid;
            const bool valid = i < live;
            int my_pos = -1;
            uint8_t my_ev = 0;
            if (valid) { my_pos = pos[i]; my_ev = ev[i]; }
            bool keep;
            if (p.mode == 1) keep = valid && i != first;
            else keep = valid && (my_ev == 0 || cur - (long long)my_pos <= p.window);
            int total;
            const int r = block_scan_flags(keep, &total, s_warp);
            if (keep) s_kept[r] = i;
            __syncthreads();
            if (keep && run + r != i) { pos[run + r] = my_pos; ev[run + r] = my_ev; }
            // Rows move only if the last kept row of the tile lands left of where it was.
            const bool moves = total > 0 && (run + total - 1 != s_kept[total - 1]);
            if (moves) {
                const int rows_per_pass = max(1, (kExpiryThreads * kMoveRegs) / chunks);
                for (int j0 = 0; j0 < total; j0 += rows_per_pass) {
                    const int nrows = min(rows_per_pass, total - j0);
                    const int work = nrows * chunks;
                    VecT kreg[kMoveRegs], vreg[kMoveRegs];
                    int64_t dst[kMoveRegs];
#pragma unroll
                    for (int u = 0; u < kMoveRegs; ++u) {
                        const int w = tid + u * kExpiryThreads;
                        dst[u] = -1;
                        if (w < work) {
                            const int j = j0 + w / chunks, c = w % chunks;
                            const int src_i = s_kept[j], dst_i = run + j;
                            if (src_i != dst_i) {
                                const int64_t srow_ = span_row(base, bt, src_i);
                                const int64_t drow_ = span_row(base, bt, dst_i);
                                if (srow_ < 0 || drow_ < 0 || srow_ >= p.pool_rows || drow_ >= p.pool_rows) {
                                    if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
                                } else {
                                    kreg[u] = *(const VecT*)(kp + srow_ * p.row_bytes + (int64_t)c * sizeof(VecT));
                                    vreg[u] = *(const VecT*)(vp + srow_ * p.row_bytes + (int64_t)c * sizeof(VecT));
                                    dst[u] = drow_ * p.row_bytes + (int64_t)c * sizeof(VecT);
                                }
                            }
                        }
                    }
                    __syncthreads();
#pragma unroll
                    for (int u = 0; u < kMoveRegs; ++u) {
                        if (dst[u] >= 0) {
                            *(VecT*)(kp + dst[u]) = kreg[u];
                            *(VecT*)(vp + dst[u]) = vreg[u];
                        }
                    }
                }
            }
            run += total;
            __syncthreads();
        }
        new_live = run;
        for (int i = new_live + tid; i < live; i += kExpiryThreads) { pos[i] = -1; ev[i] = 0; }
        // Pages that no longer hold a live row go back to the layer's free stack.
        if (p.bt && p.free_pages) {
            int32_t* btw = p.bt + (int64_t)l * p.bt_sl + (int64_t)srow * p.bt_ss + (int64_t)h * p.bt_sh;
            const int old_pages = (live + 15) >> 4, new_pages = (new_live + 15) >> 4;
            for (int pg = new_pages + tid; pg < old_pages; pg += kExpiryThreads) {
                const int32_t id = btw[pg];
                btw[pg] = -1;
                const int at = atomicAdd(&p.free_counts[l], 1);
                if (at >= 0 && at < p.pages_per_layer) p.free_pages[(int64_t)l * p.pages_per_layer + at] = id;
                else if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
            }
        }
        if (tid == 0) p.live[moff] = new_live;
    }
    if (tid == 0 && p.stats) {
        atomicAdd((unsigned long long*)&p.stats[0], (unsigned long long)(old_live - new_live));
        atomicMin(&p.stats[1], (long long)old_live);
        atomicMax(&p.stats[2], (long long)old_live);
        atomicMin(&p.stats[3], (long long)new_live);
        atomicMax(&p.stats[4], (long long)new_live);
    }
}

}  // namespace fdms

using namespace fdms;

extern "C" int32_t fdms_expire_compact(
    int32_t* token_positions, int64_t pos_stride_l, int64_t pos_stride_s, int64_t pos_stride_h,
    uint8_t* evict_mask, int64_t ev_stride_l, int64_t ev_stride_s, int64_t ev_stride_h,
    int32_t* live_counts, const int32_t* base_offsets,
    int64_t meta_stride_l, int64_t meta_stride_s,
    void* k_pool, void* v_pool, int64_t pool_layer_stride_bytes, int32_t row_bytes, int64_t pool_rows,
    int32_t* block_tables, int64_t bt_stride_l, int64_t bt_stride_s, int64_t bt_stride_h,
    int32_t* free_pages, int32_t* free_counts, int64_t pages_per_layer,
    const int32_t* seq_slots, const int64_t* current_positions,
    int32_t num_layers, int32_t num_seqs, int32_t num_kv_heads, int32_t capacity,
    int32_t window, int32_t mode, int64_t* stats, int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(token_positions && evict_mask && live_counts && k_pool && v_pool && current_positions,
                 FDMS_E_ARG, "fdms_expire_compact: null pointer");
    FDMS_REQUIRE(base_offsets || block_tables, FDMS_E_ARG,
                 "fdms_expire_compact: base_offsets or block_tables required");
    FDMS_REQUIRE(num_layers >= 0 && num_seqs >= 0 && num_kv_heads > 0 && capacity > 0, FDMS_E_ARG,
                 "fdms_expire_compact: bad sizes");
    FDMS_REQUIRE(window >= 0, FDMS_E_ARG, "window_size must be non-negative, got %d", window);
    FDMS_REQUIRE(mode == 0 || mode == 1, FDMS_E_ARG, "fdms_expire_compact: mode must be 0 or 1");
    FDMS_REQUIRE(row_bytes > 0 && row_bytes % 4 == 0, FDMS_E_ARG,
                 "fdms_expire_compact: row_bytes=%d must be a positive multiple of 4", row_bytes);
    const int64_t items = (int64_t)num_layers * num_seqs * num_kv_heads;
    if (items == 0) return FDMS_OK;
    FDMS_REQUIRE(items < (1ll << 31), FDMS_E_CAPACITY, "fdms_expire_compact: too many spans");
    ExpiryParams p;
    p.pos = token_positions; p.pos_sl = pos_stride_l; p.pos_ss = pos_stride_s; p.pos_sh = pos_stride_h;
    p.ev = evict_mask; p.ev_sl = ev_stride_l; p.ev_ss = ev_stride_s; p.ev_sh = ev_stride_h;
    p.live = live_counts; p.base = base_offsets; p.meta_sl = meta_stride_l; p.meta_ss = meta_stride_s;
    p.k_pool = (uint8_t*)k_pool; p.v_pool = (uint8_t*)v_pool;
    p.pool_layer_bytes = pool_layer_stride_bytes; p.row_bytes = row_bytes; p.pool_rows = pool_rows;
    p.bt = block_tables; p.bt_sl = bt_stride_l; p.bt_ss = bt_stride_s; p.bt_sh = bt_stride_h;
    p.free_pages = free_pages; p.free_counts = free_counts; p.pages_per_layer = pages_per_layer;
    p.seq_slots = seq_slots; p.cur = current_positions;
    p.layers = num_layers; p.seqs = num_seqs; p.hk = num_kv_heads; p.capacity = capacity;
    p.window = window; p.mode = mode; p.stats = (long long*)stats; p.dev_status = dev_status;
    const bool vec16 = row_bytes % 16 == 0 && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) &&
                       pool_layer_stride_bytes % 16 == 0;
    if (vec16)
        expire_compact_kernel<uint4><<<(unsigned)items, kExpiryThreads, 0, (cudaStream_t)stream>>>(p);
    else
        expire_compact_kernel<uint32_t><<<(unsigned)items, kExpiryThreads, 0, (cudaStream_t)stream>>>(p);
    FDMS_CHECK_LAUNCH("expire_compact_kernel");
    return FDMS_OK;
}

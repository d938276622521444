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
    int32_t* ri;                                   // optional logical -> physical row index, strides of pos
    int32_t* live; const int32_t* base; int64_t meta_sl, meta_ss;
    uint8_t* k_pool; uint8_t* v_pool; int64_t pool_layer_bytes; int row_bytes; int64_t pool_rows;
    int32_t* bt; int64_t bt_sl, bt_ss, bt_sh;
    int32_t* free_pages; int32_t* free_counts; int64_t pages_per_layer;
    const int32_t* seq_slots; const int64_t* cur;
    int layers, seqs, hk, capacity, window, mode;
    long long* stats; int32_t* dev_status;
    long long* exact;                              // optional, layout of `live`: position up to which a span is known to hold no expired slot
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

// Expiry with a row index (logical slot -> physical row of the span).  The logical order -- token
// positions, evict bits and the index itself -- is compacted exactly as above, but K/V rows do not
// follow it: the span's physical rows only have to stay dense, [0, live), because attention does not
// depend on the order of the rows it reads.  Every dropped slot frees one physical row; freed rows
// below the new length ("holes") are refilled with the rows that sit at or above it ("movers"), one
// row copy per hole instead of a shift of everything behind the dropped slot.  In steady-state decode
// that is at most one 2 * row_bytes copy per span and step instead of about `window` of them.
// Entries of the index at or beyond the live length are kept equal to their own position, so an
// appended token (logical slot live - 1, physical row live - 1) needs no index write.
//
// 128 threads and at most 72 registers, so that seven CTAs fit on an SM and the 1024 spans of a
// 16-layer, 8-sequence, 8-head decode step are resident in one wave.
constexpr int kIdxThreads = 128;
constexpr int kIdxSlotsPerThread = 16;                      // spans up to 2048 slots are staged in shared memory
constexpr int kIdxFast = kIdxThreads * kIdxSlotsPerThread;
constexpr int kHoleCap = 2048;                              // holes (dropped slots) handled per round

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ int idx_scan_flags(bool flag, int* total, int* s_warp) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned ballot = __ballot_sync(0xffffffffu, flag);
    const int in_warp = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, sum = 0;
#pragma unroll
    for (int w = 0; w < kIdxThreads / 32; ++w) {
        const int c = s_warp[w];
        if (w < warp) before += c;
        sum += c;
    }
    __syncthreads();
    *total = sum;
    return before + in_warp;
}

struct IdxSpan {
    int32_t* pos; int32_t* ri; uint8_t* ev;
    uint8_t* kp; uint8_t* vp;
    const int32_t* bt; int base;
};

// Copies the K and V row of physical row `src` of the span onto physical row `dst`.
template <typename VecT>
__device__ __forceinline__ bool idx_copy_row(const ExpiryParams& p, const IdxSpan& sp, int src, int dst) {
    const int64_t srow = span_row(sp.base, sp.bt, src), drow = span_row(sp.base, sp.bt, dst);
    if (srow < 0 || drow < 0 || srow >= p.pool_rows || drow >= p.pool_rows) {
        if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
        return false;
    }
    const int chunks = p.row_bytes / (int)sizeof(VecT);
    const VecT* ks = (const VecT*)(sp.kp + srow * p.row_bytes);
    const VecT* vs = (const VecT*)(sp.vp + srow * p.row_bytes);
    VecT* kd = (VecT*)(sp.kp + drow * p.row_bytes);
    VecT* vd = (VecT*)(sp.vp + drow * p.row_bytes);
    for (int c0 = 0; c0 < chunks; c0 += 4) {          // loads of a batch before its stores
        VecT a[4], b[4];
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (c0 + c < chunks) { a[c] = ks[c0 + c]; b[c] = vs[c0 + c]; }
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (c0 + c < chunks) { kd[c0 + c] = a[c]; vd[c0 + c] = b[c]; }
    }
    return true;
}

template <typename VecT>
__global__ void __launch_bounds__(kIdxThreads, 7) expire_indexed_kernel(ExpiryParams p) {
    __shared__ int s_holes[kHoleCap];
    __shared__ __align__(16) int s_pos[kIdxFast];
    __shared__ __align__(16) int s_ri[kIdxFast];
    __shared__ __align__(16) uint8_t s_ev[kIdxFast];
    __shared__ int s_warp[kIdxThreads / 32];
    __shared__ int s_first, s_drop, s_nh, s_nm;

    const int item = blockIdx.x;
    const int h = item % p.hk;
    const int sidx = (item / p.hk) % p.seqs;
    const int l = item / (p.hk * p.seqs);
    const int srow = p.seq_slots ? p.seq_slots[sidx] : sidx;
    const int tid = threadIdx.x, lane = tid & 31;
    pdl_trigger();                      // a dependent launch (the decode metadata) may become resident; it waits for this kernel

    const int64_t moff = (int64_t)l * p.meta_sl + (int64_t)srow * p.meta_ss + h;
    const int old_live = p.live[moff];
    IdxSpan sp;
    sp.base = p.base ? p.base[moff] : 0;
    sp.bt = p.bt ? p.bt + (int64_t)l * p.bt_sl + (int64_t)srow * p.bt_ss + (int64_t)h * p.bt_sh : nullptr;
    const int64_t poff = (int64_t)l * p.pos_sl + (int64_t)srow * p.pos_ss + (int64_t)h * p.pos_sh;
    sp.pos = p.pos + poff;
    sp.ri = p.ri + poff;
    sp.ev = p.ev + (int64_t)l * p.ev_sl + (int64_t)srow * p.ev_ss + (int64_t)h * p.ev_sh;
    sp.kp = p.k_pool + (int64_t)l * p.pool_layer_bytes;
    sp.vp = p.v_pool + (int64_t)l * p.pool_layer_bytes;
    int32_t* pos = sp.pos; int32_t* ri = sp.ri; uint8_t* ev = sp.ev;
    const long long cur = p.cur[sidx];
    int live = old_live;
    if (live > p.capacity) live = p.capacity;
    const bool active = live > 0 && (sp.bt != nullptr || sp.base >= 0);
    const int live_in = live;

    // ---- steady state of a decode loop: the span was left without an expired slot at position cur - 1 (recorded in
    // `exact` by that call) and one token has been appended since.  Slots are in position order and the tokens of the
    // window are all present, so the only slot that can have expired is the one at position cur - window - 1, which
    // sits window + 1 slots from the end (window + 2 if the token at `cur` is already in the span); and the physical
    // rows are dense with the newest token in the last one, so that row is the one that moves into the hole.  One slot
    // is inspected instead of the whole span; anything that does not match these expectations takes the general
    // path below. ----
    bool handled = false;
    // every thread reads the record before thread 0 rewrites it at the end of the kernel (all threads of the CTA must
    // take the same path below)
    const long long through = (active && p.exact) ? p.exact[moff] : -2;
    __syncthreads();
    if (active && p.exact && p.mode == 0 && through == cur - 1) {
        int idx = live - p.window - 1;
        if (idx >= 1 && (long long)pos[idx] != cur - p.window - 1) --idx;
        if (idx >= 0 && (long long)pos[idx] == cur - p.window - 1 && ri[live - 1] == live - 1) {
            handled = true;
            if (ev[idx] != 0) {
                const int r = ri[idx];
                const int new_live = live - 1;
                // the window's slots and the new token move down by one; loads of all threads before any store
                constexpr int kPer = 4;
                int mp[kPer], mr[kPer];
                uint8_t me[kPer];
#pragma unroll
                for (int j = 0; j < kPer; ++j) {
                    const int i = idx + 1 + tid + j * kIdxThreads;
                    if (i < live) { mp[j] = pos[i]; me[j] = ev[i]; mr[j] = ri[i]; }
                }
                const bool fits = live - (idx + 1) <= kPer * kIdxThreads;
                bool moved = true;
                if (tid == 0 && r != new_live) moved = fits && idx_copy_row<VecT>(p, sp, new_live, r);
                __syncthreads();
                if (fits) {
#pragma unroll
                    for (int j = 0; j < kPer; ++j) {
                        const int i = idx + 1 + tid + j * kIdxThreads;
                        if (i < live) {
                            pos[i - 1] = mp[j];
                            ev[i - 1] = me[j];
                            ri[i - 1] = (i == live - 1 && r != new_live) ? r : mr[j];
                        }
                    }
                    if (tid == 0) { pos[live - 1] = -1; ev[live - 1] = 0; ri[live - 1] = live - 1; }
                    live = new_live;
                } else {
                    handled = false;              // a window wider than this path holds: nothing was written
                }
                (void)moved;
            }
        }
    }

    if (handled) {
        // nothing else to do for this span
    } else if (active && live <= kIdxFast) {
        // ---- short spans (the common case): the span's metadata is staged in shared memory with
        // asynchronous 16-byte copies (one memory round trip, no registers held), every thread then
        // owns a run of consecutive slots.  Loops stay rolled: the kernel runs once per span, so its
        // time is mostly instruction fetch and dependent latencies, not arithmetic. ----
        if (tid == 0) { s_first = INT_MAX; s_nh = 0; s_nm = 0; }
        const bool al = (((uintptr_t)pos | (uintptr_t)ri | (uintptr_t)ev) & 15) == 0;
        const int lim = min(p.capacity, kIdxFast);
        for (int i = 4 * tid; i < live; i += 4 * kIdxThreads) {
            if (al && i + 4 <= lim) {
                cp_async16(&s_pos[i], pos + i);
                cp_async16(&s_ri[i], ri + i);
            } else {
                for (int j = i; j < min(i + 4, live); ++j) { s_pos[j] = pos[j]; s_ri[j] = ri[j]; }
            }
        }
        for (int i = 16 * tid; i < live; i += 16 * kIdxThreads) {
            if (al && i + 16 <= lim) cp_async16(&s_ev[i], ev + i);
            else for (int j = i; j < min(i + 16, live); ++j) s_ev[j] = ev[j];
        }
        cp_async_wait_all();
        __syncthreads();
        const int per = (live + kIdxThreads - 1) / kIdxThreads;            // <= 16 slots per thread
        const int lo = min(live, tid * per), hi = min(live, lo + per);
        unsigned drop_bits = 0;
        for (int i = lo; i < hi; ++i)
            if (s_ev[i] != 0 && (long long)s_pos[i] < cur - p.window) drop_bits |= 1u << (i - lo);
        if (drop_bits) atomicMin(&s_first, lo + __ffs(drop_bits) - 1);
        const int mine = __popc(drop_bits);
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        if (lane == 31) s_warp[tid >> 5] = incl;
        __syncthreads();
        int before = incl - mine, total = 0;
#pragma unroll
        for (int w = 0; w < kIdxThreads / 32; ++w) {
            const int c = s_warp[w];
            if (w < (tid >> 5)) before += c;
            total += c;
        }
        const int first = s_first;
        if (p.mode == 1 && total > 0) {                    // incremental: only the first expired slot goes
            drop_bits = (first >= lo && first < hi) ? 1u << (first - lo) : 0u;
            before = first < lo ? 1 : 0;
            total = 1;
        }
        const int new_live = live - total;
        if (total > 0) {
            for (unsigned m = drop_bits; m; m &= m - 1) {
                const int r = s_ri[lo + __ffs(m) - 1];
                if (r < new_live) s_holes[atomicAdd(&s_nh, 1)] = r;
            }
            __syncthreads();
            const int nh = s_nh;
            int shift = before;                            // dropped slots in front of slot i
            for (int i = lo; i < hi; ++i) {
                if (drop_bits >> (i - lo) & 1u) { ++shift; continue; }
                int r = s_ri[i];
                bool changed = shift != 0;
                if (r >= new_live) {                       // a mover: its row goes into a hole
                    const int k = atomicAdd(&s_nm, 1);
                    if (k < nh && r < live && idx_copy_row<VecT>(p, sp, r, s_holes[k])) {
                        r = s_holes[k];
                        changed = true;
                    } else if (p.dev_status) {
                        atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
                    }
                }
                if (changed) { pos[i - shift] = s_pos[i]; ev[i - shift] = s_ev[i]; ri[i - shift] = r; }
            }
            for (int i = new_live + tid; i < live; i += kIdxThreads) { pos[i] = -1; ev[i] = 0; ri[i] = i; }
        }
        live = new_live;
    } else if (active) {
        // ---- long spans: tiles of 128 slots, in rounds of at most kHoleCap dropped slots ----
        for (;;) {
            __syncthreads();
            if (tid == 0) { s_first = INT_MAX; s_drop = 0; s_nh = 0; s_nm = 0; }
            __syncthreads();
            int expired_seen = 0;
            for (int t0 = 0; t0 < live; t0 += kIdxThreads) {
                const int i = t0 + tid;
                bool expired = false;
                if (i < live) expired = ev[i] != 0 && (long long)pos[i] < cur - p.window;
                const unsigned any = __ballot_sync(0xffffffffu, expired);
                if (any && lane == 0) {
                    atomicMin(&s_first, t0 + (tid & ~31) + __ffs(any) - 1);
                    expired_seen += __popc(any);
                }
            }
            if (lane == 0 && expired_seen) atomicAdd(&s_drop, expired_seen);
            __syncthreads();
            const int first = s_first, total_expired = s_drop;
            if (first == INT_MAX) break;
            const int d = p.mode == 1 ? 1 : min(total_expired, kHoleCap);
            const int new_live = live - d;
            int run = (first / kIdxThreads) * kIdxThreads, dropped_run = 0;
            for (int t0 = run; t0 < live; t0 += kIdxThreads) {
                const int i = t0 + tid;
                const bool valid = i < live;
                int my_pos = -1, my_ri = 0;
                uint8_t my_ev = 0;
                if (valid) { my_pos = pos[i]; my_ev = ev[i]; my_ri = ri[i]; }
                bool expired;
                if (p.mode == 1) expired = valid && i == first;
                else expired = valid && my_ev != 0 && cur - (long long)my_pos > p.window;
                int e_total;
                const int e_rank = idx_scan_flags(expired, &e_total, s_warp);     // loads above, stores below
                const int allowed = max(0, d - dropped_run);
                const bool dropped = expired && e_rank < allowed;
                const int dropped_before = min(e_rank, allowed);
                if (dropped && my_ri < new_live) s_holes[atomicAdd(&s_nh, 1)] = my_ri;
                const int dst = run + tid - dropped_before;
                if (valid && !dropped && dst != i) { pos[dst] = my_pos; ev[dst] = my_ev; ri[dst] = my_ri; }
                const int nvalid = min(kIdxThreads, live - t0);
                const int tile_dropped = min(e_total, allowed);
                run += nvalid - tile_dropped;
                dropped_run += tile_dropped;
                __syncthreads();
            }
            for (int i = new_live + tid; i < live; i += kIdxThreads) { pos[i] = -1; ev[i] = 0; ri[i] = i; }
            __syncthreads();
            const int nh = s_nh;
            if (nh > 0) {
                for (int i = tid; i < new_live; i += kIdxThreads) {
                    const int r = ri[i];
                    if (r < new_live) continue;
                    const int k = atomicAdd(&s_nm, 1);
                    if (k < nh && r < live && idx_copy_row<VecT>(p, sp, r, s_holes[k])) ri[i] = s_holes[k];
                    else if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
                }
            }
            live = new_live;
            if (p.mode == 1 || total_expired <= kHoleCap) break;
        }
    }
    if (active && live != live_in) {
        // Pages that no longer hold a live row go back to the layer's free stack.
        if (p.bt && p.free_pages) {
            int32_t* btw = p.bt + (int64_t)l * p.bt_sl + (int64_t)srow * p.bt_ss + (int64_t)h * p.bt_sh;
            const int old_pages = (live_in + 15) >> 4, new_pages = (live + 15) >> 4;
            __syncthreads();                          // row copies read the block table entries released below
            for (int pg = new_pages + tid; pg < old_pages; pg += kIdxThreads) {
                const int32_t id = btw[pg];
                btw[pg] = -1;
                const int at = atomicAdd(&p.free_counts[l], 1);
                if (at >= 0 && at < p.pages_per_layer) p.free_pages[(int64_t)l * p.pages_per_layer + at] = id;
                else if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
            }
        }
        if (tid == 0) p.live[moff] = live;
    }
    // an all-slots call leaves no expired slot behind; an incremental one may
    if (p.exact && tid == 0) p.exact[moff] = (active && p.mode == 0) ? cur : -1;
    const int new_live_out = active ? live : old_live;
    if (tid == 0 && p.stats) {
        atomicAdd((unsigned long long*)&p.stats[0], (unsigned long long)(old_live - new_live_out));
        atomicMin(&p.stats[1], (long long)old_live);
        atomicMax(&p.stats[2], (long long)old_live);
        atomicMin(&p.stats[3], (long long)new_live_out);
        atomicMax(&p.stats[4], (long long)new_live_out);
    }
}

}  // namespace fdms

using namespace fdms;

extern "C" int32_t fdms_expire_compact(
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
    int32_t window, int32_t mode, int64_t* stats, int64_t* exact_through, int32_t* dev_status, void* stream) {
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
    p.ri = row_index;
    p.live = live_counts; p.base = base_offsets; p.meta_sl = meta_stride_l; p.meta_ss = meta_stride_s;
    p.k_pool = (uint8_t*)k_pool; p.v_pool = (uint8_t*)v_pool;
    p.pool_layer_bytes = pool_layer_stride_bytes; p.row_bytes = row_bytes; p.pool_rows = pool_rows;
    p.bt = block_tables; p.bt_sl = bt_stride_l; p.bt_ss = bt_stride_s; p.bt_sh = bt_stride_h;
    p.free_pages = free_pages; p.free_counts = free_counts; p.pages_per_layer = pages_per_layer;
    p.seq_slots = seq_slots; p.cur = current_positions;
    p.layers = num_layers; p.seqs = num_seqs; p.hk = num_kv_heads; p.capacity = capacity;
    p.window = window; p.mode = mode; p.stats = (long long*)stats; p.dev_status = dev_status;
    p.exact = row_index ? (long long*)exact_through : nullptr;        // the steady-state path exists with a row index only
    const bool vec16 = row_bytes % 16 == 0 && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) &&
                       pool_layer_stride_bytes % 16 == 0;
    if (row_index) {
        if (vec16) expire_indexed_kernel<uint4><<<(unsigned)items, kIdxThreads, 0, (cudaStream_t)stream>>>(p);
        else expire_indexed_kernel<uint32_t><<<(unsigned)items, kIdxThreads, 0, (cudaStream_t)stream>>>(p);
        FDMS_CHECK_LAUNCH("expire_indexed_kernel");
        return FDMS_OK;
    }
    if (vec16)
        expire_compact_kernel<uint4><<<(unsigned)items, kExpiryThreads, 0, (cudaStream_t)stream>>>(p);
    else
        expire_compact_kernel<uint32_t><<<(unsigned)items, kExpiryThreads, 0, (cudaStream_t)stream>>>(p);
    FDMS_CHECK_LAUNCH("expire_compact_kernel");
    return FDMS_OK;
}

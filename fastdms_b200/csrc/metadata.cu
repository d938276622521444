// Ragged-batch decode metadata built on the GPU, for all layers in one launch, plus the
// per-step decision recording and the page allocator used by the paged layout.
//
// Everything here is a few kilobytes of int32 per step; the point is to keep the step free of
// host round trips (no .item()/.tolist()), so that the whole decode step stays on the stream.
#include "common.cuh"

namespace fdms {

constexpr int kMetaThreads = 256;

// All-or-nothing pop of n entries from a free stack whose size is *count: returns the old top (the
// caller owns entries [top - n, top)) or -1 when fewer than n are left, in which case the counter is
// not touched.  A subtract-then-undo pop is not safe when spans ask for different amounts: between a
// failed subtract and its undo the counter is too low, a concurrent smaller pop can fail although
// pages are left or succeed from a stale top, and the stack ends up with duplicates.  The compare-
// and-swap retries only when another pop or push got in between, so it always makes progress; the
// iteration limit is a backstop that fails the pop instead of looping.
__device__ __forceinline__ int pop_pages(int32_t* count, int n) {
    int cur = *(volatile int32_t*)count;
    for (int it = 0; it < (1 << 20); ++it) {
        if (cur < n) return -1;
        const int seen = atomicCAS(count, cur, cur - n);
        if (seen == cur) return cur;
        cur = seen;
    }
    return -1;
}

struct MetaParams {
    int32_t* live; const int32_t* base; int64_t meta_sl, meta_ss;
    int32_t* bt; int64_t bt_sl, bt_ss, bt_sh; int max_pages;
    int32_t* free_pages; int32_t* free_counts; int64_t pages_per_layer;
    const int32_t* seq_slots;
    int32_t* base_out; int32_t* live_out; int32_t* slot_out; int32_t* cu_live_out;
    int layers, batch, hk;
    int32_t* dev_status;
};

// One CTA per layer; threads stride over the layer's batch*kv_heads spans.  The exclusive prefix
// sum of the incremented live counts is produced with a block scan carried across strides.
__global__ void __launch_bounds__(kMetaThreads) build_decode_metadata_kernel(MetaParams p) {
    __shared__ int s_warp[kMetaThreads / 32];
    __shared__ int s_carry;
    const int l = blockIdx.x;
    const int items = p.batch * p.hk;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_carry = 0;
    pdl_trigger();                      // the next launch of the stream may become resident
    pdl_wait();                         // live counts and block tables come from the preceding kernel (expiry)
    __syncthreads();
    for (int i0 = 0; i0 < items; i0 += kMetaThreads) {
        const int i = i0 + tid;
        int new_live = 0;
        if (i < items) {
            const int b = i / p.hk, h = i - b * p.hk;
            const int srow = p.seq_slots ? p.seq_slots[b] : b;
            const int64_t moff = (int64_t)l * p.meta_sl + (int64_t)srow * p.meta_ss + h;
            const int live = p.live[moff];
            const int base = p.base ? p.base[moff] : 0;
            int slot;
            if (p.bt) {
                int32_t* bt = p.bt + (int64_t)l * p.bt_sl + (int64_t)srow * p.bt_ss + (int64_t)h * p.bt_sh;
                const int pg = live >> 4;
                slot = -1;
                if (pg >= p.max_pages) {
                    if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
                } else {
                    if ((live & 15) == 0) {
                        const int top = pop_pages(&p.free_counts[l], 1);
                        if (top > 0) {
                            bt[pg] = p.free_pages[(int64_t)l * p.pages_per_layer + top - 1];
                        } else {                       // pool exhausted: flag, skip the append
                            if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
                            bt[pg] = -1;
                        }
                    }
                    const int page = bt[pg];
                    if (page >= 0) slot = page * 16 + (live & 15);
                }
            } else {
                slot = base + live;
            }
            new_live = live + 1;
            p.live[moff] = new_live;
            const int64_t o = ((int64_t)l * p.batch + b) * p.hk + h;
            p.base_out[o] = base;
            p.live_out[o] = new_live;
            p.slot_out[o] = slot;
        }
        if (p.cu_live_out) {
            // inclusive warp scan, then across warps
            int x = new_live;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, x, d);
                if (lane >= d) x += y;
            }
            if (lane == 31) s_warp[warp] = x;
            __syncthreads();
            int before = s_carry;
            for (int w = 0; w < warp; ++w) before += s_warp[w];
            if (i < items) p.cu_live_out[(int64_t)l * (items + 1) + i + 1] = before + x;
            __syncthreads();
            if (tid == kMetaThreads - 1) s_carry = before + x;
            __syncthreads();
        }
    }
    if (p.cu_live_out && tid == 0) p.cu_live_out[(int64_t)l * (items + 1)] = 0;
}

__global__ void record_decisions_kernel(
    int32_t* pos, int64_t pos_sl, int64_t pos_ss, int64_t pos_sh,
    uint8_t* ev, int64_t ev_sl, int64_t ev_ss, int64_t ev_sh,
    const int32_t* live, int64_t meta_sl, int64_t meta_ss,
    const uint8_t* evict_all, int64_t ea_sl, int64_t ea_sb,
    int64_t* positions, const int32_t* seq_slots,
    int total, int batch, int hk, int capacity, unsigned long long* true_count, int advance) {
  // With `advance` the launch is a single CTA that strides over all spans and, once every read of
  // positions[] is done, adds one to each of them (the step's last use of the positions).
  pdl_trigger();
  pdl_wait();                           // the decisions come from the preceding kernels
  for (int i0 = blockIdx.x * blockDim.x; i0 < total; i0 += gridDim.x * blockDim.x) {     // uniform per CTA
    const int i = i0 + threadIdx.x;
    bool e = false;
    if (i < total) {
        const int l = i / (batch * hk);
        const int rem = i - l * batch * hk;
        const int b = rem / hk, h = rem - b * hk;
        const int srow = seq_slots ? seq_slots[b] : b;
        const int idx = live[(int64_t)l * meta_sl + (int64_t)srow * meta_ss + h] - 1;
        e = evict_all[(int64_t)l * ea_sl + (int64_t)b * ea_sb + h] != 0;
        if (idx >= 0 && idx < capacity) {
            pos[(int64_t)l * pos_sl + (int64_t)srow * pos_ss + (int64_t)h * pos_sh + idx] = (int32_t)positions[b];
            ev[(int64_t)l * ev_sl + (int64_t)srow * ev_ss + (int64_t)h * ev_sh + idx] = e ? 1 : 0;
        }
    }
    if (true_count) {
        const unsigned m = __ballot_sync(0xffffffffu, e);
        if ((threadIdx.x & 31) == 0 && m) atomicAdd(true_count, (unsigned long long)__popc(m));
    }
  }
  if (advance) {
      __syncthreads();
      for (int b = threadIdx.x; b < batch; b += blockDim.x) positions[b] += 1;
  }
}

// Pops ceil(rows_needed / 16) pages per span from the layer's free stack into its block table
// (prefill of the paged layout).  One thread per span; the pop is all-or-nothing per span.
__global__ void alloc_pages_kernel(const int32_t* rows_needed, int32_t* bt, int64_t bt_ss, int64_t bt_sh,
                                   int max_pages, const int32_t* seq_slots, int32_t* free_pages,
                                   int32_t* free_count, int num_seqs, int hk, int32_t* dev_status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_seqs * hk) return;
    const int s = i / hk, h = i - s * hk;
    const int srow = seq_slots ? seq_slots[s] : s;
    int32_t* row = bt + (int64_t)srow * bt_ss + (int64_t)h * bt_sh;
    int n = (rows_needed[i] + 15) >> 4;
    if (n > max_pages) {
        n = max_pages;
        if (dev_status) atomicOr(dev_status, FDMS_DEV_BAD_INDEX);
    }
    const int top = pop_pages(free_count, n);      // pages [top-n, top) of the stack are ours
    if (top < 0) {
        if (dev_status) atomicOr(dev_status, FDMS_DEV_BAD_INDEX);
        for (int pg = 0; pg < n; ++pg) row[pg] = -1;
        return;
    }
    for (int pg = 0; pg < n; ++pg) row[pg] = free_pages[top - 1 - pg];
}

// Pops the pages with indices [ceil(before/16), ceil(after/16)) of every listed span.
__global__ void grow_pages_kernel(const int32_t* rows_before, const int32_t* rows_after, int32_t* bt, int64_t bt_ss,
                                  int64_t bt_sh, int max_pages, const int32_t* seq_slots, int32_t* free_pages,
                                  int32_t* free_count, int num_seqs, int hk, int32_t* dev_status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_seqs * hk) return;
    const int s = i / hk, h = i - s * hk;
    const int srow = seq_slots ? seq_slots[s] : s;
    int32_t* row = bt + (int64_t)srow * bt_ss + (int64_t)h * bt_sh;
    const int have = (max(rows_before[i], 0) + 15) >> 4;
    int want = (max(rows_after[i], 0) + 15) >> 4;
    if (want > max_pages) {
        want = max_pages;
        if (dev_status) atomicOr(dev_status, FDMS_DEV_BAD_INDEX);
    }
    const int n = want - have;
    if (n <= 0) return;
    const int top = pop_pages(free_count, n);
    if (top < 0) {
        if (dev_status) atomicOr(dev_status, FDMS_DEV_BAD_INDEX);
        for (int pg = have; pg < want; ++pg) row[pg] = -1;
        return;
    }
    for (int pg = 0; pg < n; ++pg) row[have + pg] = free_pages[top - 1 - pg];
}

// Returns every page of the listed spans to the free stack and clears their block-table rows.
__global__ void free_pages_kernel(const int32_t* live, int64_t meta_ss, int32_t* bt, int64_t bt_ss,
                                  int64_t bt_sh, int max_pages, const int32_t* seq_slots,
                                  int32_t* free_pages, int32_t* free_count, int64_t pages_per_layer,
                                  int num_seqs, int hk, int32_t* dev_status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_seqs * hk) return;
    const int s = i / hk, h = i - s * hk;
    const int srow = seq_slots ? seq_slots[s] : s;
    int32_t* row = bt + (int64_t)srow * bt_ss + (int64_t)h * bt_sh;
    for (int pg = 0; pg < max_pages; ++pg) {
        const int32_t id = row[pg];
        if (id < 0) continue;
        row[pg] = -1;
        const int at = atomicAdd(free_count, 1);
        if (at < pages_per_layer) free_pages[at] = id;
        else if (dev_status) atomicOr(dev_status, FDMS_DEV_BAD_INDEX);
    }
}

}  // namespace fdms

using namespace fdms;

extern "C" int32_t fdms_build_decode_metadata(
    int32_t* live_counts, const int32_t* base_offsets, int64_t meta_stride_l, int64_t meta_stride_s,
    int32_t* block_tables, int64_t bt_stride_l, int64_t bt_stride_s, int64_t bt_stride_h, int32_t max_pages,
    int32_t* free_pages, int32_t* free_counts, int64_t pages_per_layer,
    const int32_t* seq_slots,
    int32_t* base_out, int32_t* live_out, int32_t* slot_out, int32_t* cu_live_out,
    int32_t num_layers, int32_t batch, int32_t num_kv_heads, int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(live_counts && base_out && live_out && slot_out, FDMS_E_ARG,
                 "fdms_build_decode_metadata: null pointer");
    FDMS_REQUIRE(base_offsets || block_tables, FDMS_E_ARG,
                 "fdms_build_decode_metadata: base_offsets or block_tables required");
    FDMS_REQUIRE(!block_tables || (free_pages && free_counts && max_pages > 0 && pages_per_layer > 0), FDMS_E_ARG,
                 "fdms_build_decode_metadata: the paged layout needs the free-page stacks");
    FDMS_REQUIRE(num_layers >= 0 && batch >= 0 && num_kv_heads > 0, FDMS_E_ARG,
                 "fdms_build_decode_metadata: bad sizes");
    if (num_layers == 0 || batch == 0) return FDMS_OK;
    MetaParams p;
    p.live = live_counts; p.base = base_offsets; p.meta_sl = meta_stride_l; p.meta_ss = meta_stride_s;
    p.bt = block_tables; p.bt_sl = bt_stride_l; p.bt_ss = bt_stride_s; p.bt_sh = bt_stride_h; p.max_pages = max_pages;
    p.free_pages = free_pages; p.free_counts = free_counts; p.pages_per_layer = pages_per_layer;
    p.seq_slots = seq_slots;
    p.base_out = base_out; p.live_out = live_out; p.slot_out = slot_out; p.cu_live_out = cu_live_out;
    p.layers = num_layers; p.batch = batch; p.hk = num_kv_heads; p.dev_status = dev_status;
    FDMS_CUDA_OK(launch_chained(build_decode_metadata_kernel, dim3((unsigned)num_layers), dim3(kMetaThreads), (cudaStream_t)stream,
                                chain_launches(), p));
    FDMS_CHECK_LAUNCH("build_decode_metadata_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_record_decisions(
    int32_t* token_positions, int64_t pos_stride_l, int64_t pos_stride_s, int64_t pos_stride_h,
    uint8_t* evict_mask, int64_t ev_stride_l, int64_t ev_stride_s, int64_t ev_stride_h,
    const int32_t* live_counts, int64_t meta_stride_l, int64_t meta_stride_s,
    const uint8_t* evict_all, int64_t ea_stride_l, int64_t ea_stride_b,
    int64_t* positions, const int32_t* seq_slots,
    int32_t num_layers, int32_t batch, int32_t num_kv_heads, int32_t capacity,
    int64_t* true_count, int32_t advance_positions, void* stream) {
    clear_error();
    FDMS_REQUIRE(token_positions && evict_mask && live_counts && evict_all && positions, FDMS_E_ARG,
                 "fdms_record_decisions: null pointer");
    FDMS_REQUIRE(num_layers >= 0 && batch >= 0 && num_kv_heads > 0 && capacity > 0, FDMS_E_ARG,
                 "fdms_record_decisions: bad sizes");
    const int64_t total = (int64_t)num_layers * batch * num_kv_heads;
    if (total == 0) return FDMS_OK;
    FDMS_REQUIRE(total < (1ll << 31), FDMS_E_CAPACITY, "fdms_record_decisions: too many spans");
    const int threads = advance_positions ? 1024 : 256;
    const unsigned blocks = advance_positions ? 1u : (unsigned)((total + threads - 1) / threads);
    FDMS_CUDA_OK(launch_chained(
        record_decisions_kernel, dim3(blocks), dim3((unsigned)threads), (cudaStream_t)stream, chain_launches(),
        token_positions, pos_stride_l, pos_stride_s, pos_stride_h, evict_mask, ev_stride_l, ev_stride_s,
        ev_stride_h, live_counts, meta_stride_l, meta_stride_s, evict_all, ea_stride_l, ea_stride_b, positions,
        seq_slots, (int)total, batch, num_kv_heads, capacity, (unsigned long long*)true_count, advance_positions ? 1 : 0));
    FDMS_CHECK_LAUNCH("record_decisions_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_alloc_pages(
    const int32_t* rows_needed, int32_t* block_tables, int64_t bt_stride_s, int64_t bt_stride_h,
    int32_t max_pages, const int32_t* seq_slots, int32_t* free_pages, int32_t* free_count,
    int32_t num_seqs, int32_t num_kv_heads, int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(rows_needed && block_tables && free_pages && free_count, FDMS_E_ARG, "fdms_alloc_pages: null pointer");
    FDMS_REQUIRE(num_seqs >= 0 && num_kv_heads > 0 && max_pages > 0, FDMS_E_ARG, "fdms_alloc_pages: bad sizes");
    const int total = num_seqs * num_kv_heads;
    if (total == 0) return FDMS_OK;
    alloc_pages_kernel<<<(total + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        rows_needed, block_tables, bt_stride_s, bt_stride_h, max_pages, seq_slots, free_pages, free_count,
        num_seqs, num_kv_heads, dev_status);
    FDMS_CHECK_LAUNCH("alloc_pages_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_grow_pages(
    const int32_t* rows_before, const int32_t* rows_after, int32_t* block_tables, int64_t bt_stride_s,
    int64_t bt_stride_h, int32_t max_pages, const int32_t* seq_slots, int32_t* free_pages, int32_t* free_count,
    int32_t num_seqs, int32_t num_kv_heads, int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(rows_before && rows_after && block_tables && free_pages && free_count, FDMS_E_ARG, "fdms_grow_pages: null pointer");
    FDMS_REQUIRE(num_seqs >= 0 && num_kv_heads > 0 && max_pages > 0, FDMS_E_ARG, "fdms_grow_pages: bad sizes");
    const int total = num_seqs * num_kv_heads;
    if (total == 0) return FDMS_OK;
    grow_pages_kernel<<<(total + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        rows_before, rows_after, block_tables, bt_stride_s, bt_stride_h, max_pages, seq_slots, free_pages, free_count,
        num_seqs, num_kv_heads, dev_status);
    FDMS_CHECK_LAUNCH("grow_pages_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_free_pages(
    const int32_t* live_counts, int64_t meta_stride_s, int32_t* block_tables, int64_t bt_stride_s,
    int64_t bt_stride_h, int32_t max_pages, const int32_t* seq_slots, int32_t* free_pages,
    int32_t* free_count, int64_t pages_per_layer, int32_t num_seqs, int32_t num_kv_heads,
    int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(block_tables && free_pages && free_count, FDMS_E_ARG, "fdms_free_pages: null pointer");
    FDMS_REQUIRE(num_seqs >= 0 && num_kv_heads > 0 && max_pages > 0, FDMS_E_ARG, "fdms_free_pages: bad sizes");
    const int total = num_seqs * num_kv_heads;
    if (total == 0) return FDMS_OK;
    free_pages_kernel<<<(total + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        live_counts, meta_stride_s, block_tables, bt_stride_s, bt_stride_h, max_pages, seq_slots, free_pages,
        free_count, pages_per_layer, num_seqs, num_kv_heads, dev_status);
    FDMS_CHECK_LAUNCH("free_pages_kernel");
    return FDMS_OK;
}

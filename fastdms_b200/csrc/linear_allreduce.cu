// Row-parallel linear layer of tensor-parallel decode fused with its all-reduce:
//   y[M, N] = sum over ranks r of  x_r[M, K_r] * W_r[N, K_r]^T   (+ bias),  M <= 8 rows,
// in ONE kernel per rank (the reference runs F.linear and then NCCL's all_reduce on the [batch, hidden]
// result after o_proj and down_proj, fastdms/layers/linear.py:1044-1048: two launches and a collective
// whose cost at 64 KB is pure latency, 72 times per decode step of the 8B shape).
//
// A CTA owns 16 * TPC output columns.  Its 8 warps split (tile, K range): with K_r / 256 >= 8 steps all
// eight warps share one tile's K; narrower shards (K_r = 512 at eight ranks) put several tiles on one
// CTA.  Weight rows sit on the M side of mma.sync.m16n8k16, the <= 8 activation rows on N, exactly as in
// the decode linear kernel; partial tiles of the warps are summed through shared memory in float32.
//
// Epilogue = the collective, in the style of a low-latency all-reduce.  The CTA PUSHES its float32 partial tile
// into a slot of every peer's mapped region over NVLink, each pair of values as one 16-byte store
// {value, epoch, value, epoch}: an 8-byte half of such a store arrives whole, so the epoch word next to a value says
// that the value is the one of this call, and no fence, flag or second round trip is needed.  It then reads the
// slots the peers pushed into its OWN memory, polling every 16-byte word until both epoch words match (bounded),
// adds the ranks' partials in rank order (its own from shared memory), adds the bias once, rounds once and stores
// y.  Every rank ends up with identical bits; partials cross the link in float32, so the result is rounded once
// instead of once per rank.  No multicast objects, no library kernel touches peer memory.
//
// Region of a rank:  slots[2][world][kLarMaxCtas][2 * kLarSlotFloats] 32-bit words | epoch[kLarMaxCtas].  Slots are
// indexed by CTA, not by column, so a CTA's slot is only ever touched by the CTAs of the same index; call e uses
// parity e & 1.  A rank can be at most one call ahead of a peer (to start call e + 2 it has finished call e + 1,
// for which it needed the peer's values of call e + 1, which the peer's CTA pushes only after it has finished
// reading call e), so two parities are enough and a stale slot carries epoch e - 2.  The epoch lives on the
// device so that a captured CUDA graph replays the call; the region starts zeroed and epochs start at 1.
//
// A wait that runs out (about a second) raises FDMS_DEV_WAIT_TIMEOUT, leaves the silent rank out of the
// sum and returns.  After that the ranks' epochs may disagree: the status bit is FATAL for the region,
// which must be re-created collectively before it is used again.
#include <string.h>

#include "common.cuh"

namespace fdms {

constexpr int kLarWarps = 8;
constexpr int kLarThreads = kLarWarps * 32;
constexpr int kLarStep = 256;              // k elements per warp and step
constexpr int kLarMaxTpc = 8;              // tiles of 16 columns per CTA
constexpr int kLarSlotFloats = kLarMaxTpc * 128;      // 8 rows x 16 columns per tile
constexpr int kLarMaxCtas = 512;
constexpr int kLarMaxWorld = 8;
constexpr unsigned kLarSpinLimit = 1u << 20;      // polls of one word before giving up (about a second)

struct LarParams {
    const uint16_t* x; int64_t x_stride;
    const uint16_t* w; int64_t w_stride;
    const uint16_t* bias;
    uint16_t* y; int64_t y_stride;
    int M, N, K, ks, tpc;                  // ks K-splits x tpc tiles = 8 warps
    uint32_t* slots[kLarMaxWorld];         // region of every rank (index = rank)
    uint32_t* epoch;                       // local
    int rank, world;
    int32_t* dev_status;
};

// 16 bytes {value, epoch, value, epoch}; system-scope relaxed accesses that bypass L1
__device__ __forceinline__ void lar_st_pair(uint32_t* p, float a, float b, uint32_t e) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(__float_as_uint(a)), "r"(e), "r"(__float_as_uint(b)), "r"(e) : "memory");
}
__device__ __forceinline__ uint4 lar_ld_pair(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template <bool BF16>
__device__ __forceinline__ void lar_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Offset (in 32-bit words) of the slot of (parity, source rank, CTA) inside a region.
__device__ __forceinline__ size_t lar_slot(int parity, int src, int cta, int world) {
    return (((size_t)parity * world + src) * kLarMaxCtas + cta) * (2 * kLarSlotFloats);
}

template <bool BF16>
__global__ void __launch_bounds__(kLarThreads) linear_allreduce_kernel(LarParams p) {
    __shared__ float s_part[kLarWarps][128];             // per warp: its tile's 16 columns x 8 rows
    __shared__ __align__(16) float s_sum[kLarMaxTpc * 128];
    __shared__ volatile int s_missing[kLarMaxWorld];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int c = blockIdx.x;
    const int tile_local = warp / p.ks, split = warp - tile_local * p.ks;
    const int tile = c * p.tpc + tile_local;
    const int n0 = tile * 16;
    const int steps = p.K / kLarStep;
    const int s_begin = (int)((int64_t)split * steps / p.ks), s_end = (int)((int64_t)(split + 1) * steps / p.ks);
    const bool active = n0 < p.N && s_begin < s_end;
    if (tid < kLarMaxWorld) s_missing[tid] = 0;

    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // Weights do not depend on the preceding kernel: the first step's vectors are requested before the
    // dependency is resolved.
    pdl_trigger();
    uint4 wa[8], wb[8];
    const uint16_t* w0 = p.w + (int64_t)(n0 + g) * p.w_stride + 8 * t;
    const uint16_t* w1 = w0 + 8 * p.w_stride;
    if (active) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            wa[j] = __ldcs((const uint4*)(w0 + s_begin * kLarStep + 32 * j));
            wb[j] = __ldcs((const uint4*)(w1 + s_begin * kLarStep + 32 * j));
        }
    }
    pdl_wait();
    if (active) {
        const uint16_t* xr = p.x + (int64_t)g * p.x_stride + 8 * t;
        for (int s = s_begin; s < s_end; ++s) {
            uint4 xb[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                xb[j] = g < p.M ? __ldg((const uint4*)(xr + s * kLarStep + 32 * j)) : make_uint4(0u, 0u, 0u, 0u);
            if (s != s_begin) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    wa[j] = __ldcs((const uint4*)(w0 + s * kLarStep + 32 * j));
                    wb[j] = __ldcs((const uint4*)(w1 + s * kLarStep + 32 * j));
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                lar_mma<BF16>(acc, wa[j].x, wb[j].x, wa[j].y, wb[j].y, xb[j].x, xb[j].y);
                lar_mma<BF16>(acc, wa[j].z, wb[j].z, wa[j].w, wb[j].w, xb[j].z, xb[j].w);
            }
        }
    }
    // acc[0..1]: column n0 + g, rows 2t, 2t+1;  acc[2..3]: column n0 + g + 8.  Layout of a tile: [column][row].
    *(float2*)&s_part[warp][g * 8 + 2 * t] = make_float2(acc[0], acc[1]);
    *(float2*)&s_part[warp][(g + 8) * 8 + 2 * t] = make_float2(acc[2], acc[3]);
    __syncthreads();
    const int tile_floats = p.tpc * 128;
    for (int idx = tid; idx < tile_floats; idx += kLarThreads) {
        const int tl = idx >> 7, r = idx & 127;
        float sum = 0.0f;
        for (int s = 0; s < p.ks; ++s) sum += s_part[tl * p.ks + s][r];
        s_sum[idx] = sum;
    }
    __syncthreads();

    // ---- the collective ----
    const uint32_t e = p.epoch[c] + 1;
    const int parity = (int)(e & 1u);
    const int pairs = tile_floats / 2;
    for (int i = tid; i < (p.world - 1) * pairs; i += kLarThreads) {
        int r = i / pairs;
        const int v = i - r * pairs;
        r += r >= p.rank ? 1 : 0;                                   // peers only
        lar_st_pair(p.slots[r] + lar_slot(parity, p.rank, c, p.world) + 4 * v, s_sum[2 * v], s_sum[2 * v + 1], e);
    }
    // sum in rank order (own partial from shared memory, the peers' from this rank's region), bias once, one rounding
    const uint32_t* mine = p.slots[p.rank];
    const int vecs = tile_floats / 4;
    for (int v = tid; v < vecs; v += kLarThreads) {
        // every peer's words are requested at once (one round trip when they have all arrived); only then does the
        // thread wait, peer by peer in rank order, for those whose epoch words do not match yet
        uint4 lo[kLarMaxWorld], hi[kLarMaxWorld];
#pragma unroll
        for (int r = 0; r < kLarMaxWorld; ++r) {
            if (r < p.world && r != p.rank) {
                const uint32_t* src = mine + lar_slot(parity, r, c, p.world) + 8 * v;
                lo[r] = lar_ld_pair(src);
                hi[r] = lar_ld_pair(src + 4);
            }
        }
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int r = 0; r < kLarMaxWorld; ++r) {
            if (r >= p.world) continue;
            float4 a;
            if (r == p.rank) {
                a = ((const float4*)s_sum)[v];
            } else {
                const uint32_t* src = mine + lar_slot(parity, r, c, p.world) + 8 * v;
                unsigned spins = 0;
                while (lo[r].y != e || lo[r].w != e || hi[r].y != e || hi[r].w != e) {
                    if (s_missing[r] || ++spins >= kLarSpinLimit) {
                        if (!s_missing[r]) {
                            s_missing[r] = 1;
                            if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_WAIT_TIMEOUT);
                        }
                        break;
                    }
                    lo[r] = lar_ld_pair(src);
                    hi[r] = lar_ld_pair(src + 4);
                }
                if (lo[r].y != e || lo[r].w != e || hi[r].y != e || hi[r].w != e) continue;      // silent rank: left out
                a = make_float4(__uint_as_float(lo[r].x), __uint_as_float(lo[r].z), __uint_as_float(hi[r].x), __uint_as_float(hi[r].z));
            }
            sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
        }
        // vector v = tile v / 32, column (v % 32) / 2, rows 4 * (v & 1) .. + 3
        const int tl = v >> 5, col = (v & 31) >> 1, row0 = (v & 1) * 4;
        const int n = (c * p.tpc + tl) * 16 + col;
        if (n >= p.N) continue;
        float b = 0.0f;
        if (p.bias) b = BF16 ? __uint_as_float((uint32_t)p.bias[n] << 16) : __half2float(*(const __half*)&p.bias[n]);
        const float vals[4] = {sum.x + b, sum.y + b, sum.z + b, sum.w + b};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = row0 + i;
            if (m >= p.M) continue;
            uint16_t o;
            if (BF16) { const __nv_bfloat16 bb = __float2bfloat16_rn(vals[i]); o = *(const uint16_t*)&bb; }
            else { const __half hh = __float2half_rn(vals[i]); o = *(const uint16_t*)&hh; }
            p.y[(int64_t)m * p.y_stride + n] = o;
        }
    }
    __syncthreads();
    if (tid == 0) p.epoch[c] = e;
}

}  // namespace fdms

using namespace fdms;

extern "C" int64_t fdms_linear_allreduce_region_bytes(int32_t world) {
    if (world < 2 || world > kLarMaxWorld) return -1;
    const int64_t slots = 2ll * world * kLarMaxCtas * (2 * kLarSlotFloats) * 4;
    const int64_t epoch = (int64_t)kLarMaxCtas * 4;
    return slots + epoch;
}

extern "C" int32_t fdms_linear_decode_allreduce(
    const void* x, int64_t x_row_stride, const void* weight, int64_t w_row_stride, const void* bias,
    void* y, int64_t y_row_stride, int32_t dtype, int32_t rows, int32_t out_features, int32_t in_features,
    void* const* peer_regions, int32_t rank, int32_t world, int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(x && weight && y && peer_regions, FDMS_E_ARG, "fdms_linear_decode_allreduce: null pointer");
    FDMS_REQUIRE(dtype == FDMS_BF16 || dtype == FDMS_F16, FDMS_E_DTYPE, "fdms_linear_decode_allreduce: bf16 or f16 only");
    FDMS_REQUIRE(world >= 2 && world <= kLarMaxWorld && rank >= 0 && rank < world, FDMS_E_ARG,
                 "fdms_linear_decode_allreduce: world must be 2..%d and rank inside it", kLarMaxWorld);
    FDMS_REQUIRE(rows >= 0 && rows <= 8, FDMS_E_CAPACITY, "fdms_linear_decode_allreduce: at most 8 rows, got %d", rows);
    FDMS_REQUIRE(out_features > 0 && out_features % 16 == 0 && in_features > 0 && in_features % kLarStep == 0, FDMS_E_ARG,
                 "fdms_linear_decode_allreduce: out_features %% 16 and in_features %% %d must be 0 (got %d, %d)", kLarStep,
                 out_features, in_features);
    FDMS_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)weight & 15) == 0 && (x_row_stride * 2) % 16 == 0 &&
                     (w_row_stride * 2) % 16 == 0,
                 FDMS_E_ARG, "fdms_linear_decode_allreduce: x and weight rows must be 16-byte aligned");
    if (rows == 0) return FDMS_OK;
    const int steps = in_features / kLarStep;
    int ks = 1;
    while (ks * 2 <= kLarWarps && ks * 2 <= steps) ks *= 2;
    const int tpc = kLarWarps / ks;
    const int tiles = out_features / 16;
    const int ctas = (tiles + tpc - 1) / tpc;
    FDMS_REQUIRE(ctas <= kLarMaxCtas, FDMS_E_CAPACITY,
                 "fdms_linear_decode_allreduce: %d CTAs needed, the region has slots for %d (out_features too large)", ctas,
                 kLarMaxCtas);
    LarParams p;
    p.x = (const uint16_t*)x; p.x_stride = x_row_stride; p.w = (const uint16_t*)weight; p.w_stride = w_row_stride;
    p.bias = (const uint16_t*)bias; p.y = (uint16_t*)y; p.y_stride = y_row_stride;
    p.M = rows; p.N = out_features; p.K = in_features; p.ks = ks; p.tpc = tpc;
    const size_t slot_words = 2ull * world * kLarMaxCtas * (2 * kLarSlotFloats);
    for (int r = 0; r < kLarMaxWorld; ++r) p.slots[r] = nullptr;
    for (int r = 0; r < world; ++r) {
        FDMS_REQUIRE(peer_regions[r] != nullptr, FDMS_E_ARG, "fdms_linear_decode_allreduce: region of rank %d is null", r);
        p.slots[r] = (uint32_t*)peer_regions[r];
    }
    p.epoch = p.slots[rank] + slot_words;
    p.rank = rank; p.world = world; p.dev_status = dev_status;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == FDMS_BF16)
        FDMS_CUDA_OK(launch_chained(linear_allreduce_kernel<true>, dim3((unsigned)ctas), dim3(kLarThreads), st, chain_launches(), p));
    else
        FDMS_CUDA_OK(launch_chained(linear_allreduce_kernel<false>, dim3((unsigned)ctas), dim3(kLarThreads), st, chain_launches(), p));
    FDMS_CHECK_LAUNCH("linear_allreduce_kernel");
    return FDMS_OK;
}

// Compact decode attention over ragged per-(sequence, KV head) spans of the compact KV pool.
//
// Fast path (FP8 e4m3 pools, head_dim 64 or 128, group size <= 8)
// ----------------------------------------------------------------
//   * Split-K across the compact length on thread-block clusters.  A span (one sequence, one KV
//     head) is cut into `splits` equal page ranges; the CTAs of one cluster take one range each.
//     Partial (m, l, O) results travel to the cluster's first CTA through distributed shared memory
//     (remote stores + one cluster barrier), which folds them and writes the output: no global
//     round trip, no second launch.  The host picks splits (1..16) so that the grid is about one
//     wave of 2 CTAs per SM.  Very long spans at tiny batch use several clusters per span
//     (`chunks` > 1); only then do cluster leaders meet in the global workspace, where the last one
//     to arrive at a per-span counter folds the chunk partials (threadfence + atomic, no spinning).
//   * Eight warps per CTA each own every 8th 16-row page of the CTA's range and there is no barrier in the
//     page loop.  Two kernels share the page math and differ in how a page reaches the warp:
//       - direct (default): every lane loads its K and V MMA fragments straight from the pool (16 bytes of K
//         and two 8-byte V pieces per lane and page), `DEPTH` pages ahead in registers;
//       - staged (FDMS_ATTN_LOADER=staged): lane s of a warp issues two 1 KiB bulk asynchronous copies
//         (cp.async.bulk, the TMA unit's untiled form) into slot s of the warp's own shared-memory ring;
//         they complete on a per-slot mbarrier and the warp reads its fragments from shared memory.
//   * Per page a warp computes the GQA-packed S = q K^T and O += P V tiles with tensor-core MMAs (q heads on
//     the M axis, f32 accumulate).  Warps with few pages convert the FP8 K bytes exactly to f16
//     (mma.sync.m16n8k16); warps with `kQk8MinPages` or more use the K bytes as an e4m3 operand as they are
//     (mma.sync.m16n8k32) against q split into an e4m3 value and an amplified e4m3 residual.  V is always
//     converted to f16.  The softmax is the online form with warp-shuffle row reductions in the log2 domain.
//   * With FDMS_ATTN_OVERLAP_PREVIOUS everything that does not depend on the preceding kernel (metadata, block
//     tables, cos/sin, the first pages) is issued before `griddepcontrol.wait`.
// Every wait on an mbarrier is bounded; on expiry the staged kernel raises FDMS_DEV_WAIT_TIMEOUT in the
// status word, stops issuing copies, drains with short waits and still takes part in every
// cluster barrier before it returns.
//
// Algorithmic HBM bytes per launch: sum over spans of live * 2 * head_dim (FP8 K + V), plus
// batch*q_heads*head_dim*(q + out) and 8-12 bytes of metadata per span.
//
// Generic path: any pool dtype (f32/bf16/f16/e4m3), any head_dim <= 256, any group size.  One CTA per
// (sequence, q head); used for the reference's small float32 fixtures, not for speed.
#include <cuda.h>
#include <stdlib.h>

#include <atomic>
#include <type_traits>

#include "common.cuh"

namespace fdms {

constexpr int kPage = 16;
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kMaxGroup = 8;
constexpr int kMaxSplits = 16;           // cluster size limit (8 portable, 16 with the opt-in attribute)
constexpr int kMaxChunks = 64;           // clusters per span
constexpr int kWaitHintNs = 20000;       // each mbarrier.try_wait may sleep this long before it reports "not yet"
constexpr int kWaitLimit = 50000;        // polls before giving up (about a second)
constexpr int kWaitLimitDrain = 100;
constexpr float kLog2e = 1.4426950408889634f;

// ------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(kWaitHintNs) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int limit) {
    for (int i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// 1-D bulk copy global -> shared, completing `bytes` on the mbarrier.  Addresses and size are
// multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_bar() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}
// Cluster barrier, split phase.  Every thread of every CTA of the cluster executes each call once.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Address of `local` (this CTA's shared memory) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(const void* local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Programmatic dependent launch.  `grid_dependency_wait` returns once the preceding kernel of the
// stream has completed and its writes are visible (immediately when the launch was an ordinary one);
// `grid_launch_dependents` lets a dependent launch that opted in start its own preamble early.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
    uint32_t r;
    asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(r) : "r"(two_bytes));
    return r;
}
// Both halves of a 32-bit word (4 e4m3 bytes) at once: lo = bytes 0,1 and hi = bytes 2,3 as f16x2.
__device__ __forceinline__ void e4m3x4_to_f16x2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
    asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
        : "=r"(lo), "=r"(hi) : "r"(w));
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *(uint32_t*)&h;
}
// D(16x8, f32) += A(16x16, f16) * B(16x8, f16) with A rows 8..15 identically zero (a1 = a3 = 0):
// only c0, c1 (row g) carry data.
__device__ __forceinline__ void mma_top(float& c0, float& c1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float d2, d3;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
        : "+f"(c0), "+f"(c1), "=f"(d2), "=f"(d3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.0f));
    (void)d2; (void)d3;
}

// D(16x8, f32) += A(16x16, f16) * B(16x8, f16), all four A registers and accumulators in use.
__device__ __forceinline__ void mma_full(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8, f32) += A(16x32, e4m3) * B(32x8, e4m3): the FP8 form of the warp-level MMA.  The pool's K bytes
// go in as the A operand exactly as they were loaded, no conversion.
__device__ __forceinline__ void mma_fp8(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// q as the FP8 B operand of the score product, used by warps that own many pages (long spans): it removes
// the FP8 -> f16 conversion of K, a third of the instructions of a page, at the price of quantising q once
// per warp, which a warp with two or three pages does not earn back (those keep the f16 product).
// A lane holds 16 consecutive elements of its head per 64-element chunk (the f16 pairs of `qa`).  They are scaled by a power of two c chosen from the largest
// magnitude in the head group so that c * |q| lies in [128, 256), then split into two e4m3 values:
//   hi = e4m3(c q),   lo = e4m3(16 (c q - hi)),   c q = hi + lo / 16 up to 2^-8 relative
// (q itself is a 16-bit activation with 2^-9 relative rounding).  The score of a token is then
// (K . hi + (K . lo) / 16) / c with both products exact in the MMA's float32 accumulator; K needs no
// conversion at all.  Every warp of every CTA of a span derives the same c from the same q.
constexpr float kQLoGain = 16.0f;
constexpr int kQk8MinPages = 8;            // a warp with at least this many pages takes the FP8 score product
template <int D>
__device__ __forceinline__ void quantize_q(uint32_t (&qa)[D / 16][2], float& inv_c) {
    float x[D / 4];
#pragma unroll
    for (int w = 0; w < D / 16; ++w) {
        const __half2 p0 = *(const __half2*)&qa[w][0], p1 = *(const __half2*)&qa[w][1];
        x[4 * w + 0] = __low2float(p0); x[4 * w + 1] = __high2float(p0);
        x[4 * w + 2] = __low2float(p1); x[4 * w + 3] = __high2float(p1);
    }
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < D / 4; ++i) mx = fmaxf(mx, fabsf(x[i]));
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // c = 2^(7 - floor(log2 mx)), from the exponent field (exact, identical in every warp)
    const int e = (__float_as_int(mx) >> 23) & 0xff;
    const bool ok = e >= 8 && e <= 250;
    const float c = ok ? __int_as_float((261 - e) << 23) : 1.0f;
    inv_c = ok ? __int_as_float((e - 7) << 23) : 1.0f;
#pragma unroll
    for (int w = 0; w < D / 16; ++w) {
        uint32_t hi = 0u, lo = 0u;
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
            const float a = x[4 * w + 2 * pr] * c, b = x[4 * w + 2 * pr + 1] * c;
            const __nv_fp8x2_storage_t h2 = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
            const __half2_raw back = __nv_cvt_fp8x2_to_halfraw2(h2, __NV_E4M3);
            const __half2 bh = *(const __half2*)&back;
            const float ra = (a - __low2float(bh)) * kQLoGain, rb = (b - __high2float(bh)) * kQLoGain;
            const __nv_fp8x2_storage_t l2 = __nv_cvt_float2_to_fp8x2(make_float2(ra, rb), __NV_SATFINITE, __NV_E4M3);
            hi |= (uint32_t)h2 << (16 * pr);
            lo |= (uint32_t)l2 << (16 * pr);
        }
        qa[w][0] = hi;          // from here on the array holds the two e4m3 parts, word by word
        qa[w][1] = lo;
    }
}

// Transpose of an 8x8 matrix of 16-bit elements held one register per lane (row = lane / 4).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// Physical row inside a page for MMA column n of n-tile u.  Two permutations:
//  * staged loader (LIN = false): keeps the shared-memory K reads (rows tokrow(u, g), 16 bytes per
//    lane) free of bank conflicts and the V reads (rows tokrow(u, 2t), tokrow(u, 2t+1), 8 bytes per
//    lane) at the 2-way minimum that 64-byte rows allow;
//  * direct loader (LIN = true): the four V rows one instruction reads (columns 2t, or 2t+1, of all
//    quads) are consecutive rows, so that with 64-byte rows every V load covers whole 128-byte lines.
template <bool LIN>
__device__ __forceinline__ int tokrow(int u, int n) {
    if (LIN) return 8 * u + (n >> 1) + 4 * (n & 1);
    const int tp = n >> 1;
    return 8 * u + 2 * tp + ((n & 1) ^ (tp & 1));
}

// Phase probe (compiled in only with -DFDMS_ATTN_PROBE, e.g. `python -m fastdms_b200.build --probe`):
// thread 0 of every CTA of the fast kernels records the global nanosecond timer at the phases below,
// and fdms_attn_probe_read copies the table of the most recent launch to the host
// (benchmarks/attn_timeline.py prints it).  Off by default: the production kernels carry no probe code.
enum { kProbeStart = 0, kProbeIssued, kProbeDependency, kProbeQReady, kProbePagesDone, kProbeCtaFolded, kProbeEnd, kProbePhases };
constexpr int kProbeMaxCtas = 4096;
#ifdef FDMS_ATTN_PROBE
__device__ unsigned long long g_attn_probe[kProbePhases][kProbeMaxCtas];
#define FDMS_PROBE(phase)                                                                      \
    do {                                                                                       \
        if (threadIdx.x == 0) {                                                                \
            const unsigned cta_ = blockIdx.y * gridDim.x + blockIdx.x;                         \
            unsigned long long t_;                                                             \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                             \
            if (cta_ < (unsigned)kProbeMaxCtas) g_attn_probe[(phase)][cta_] = t_;              \
        }                                                                                      \
    } while (0)
#else
#define FDMS_PROBE(phase) do { } while (0)
#endif

struct AttnParams;
__device__ __forceinline__ int64_t checked_rope_position(const AttnParams& p, int b);

struct AttnParams {
    const void* q; int q_dtype; int64_t q_sb, q_sh;
    const uint8_t* k_pool; const uint8_t* v_pool; int64_t pool_rows;
    const int32_t* base; const int32_t* live; int64_t meta_sb;
    const int32_t* bt; int64_t bt_sb, bt_sh; int bt_pages;
    const float* k_scale; const float* v_scale;
    void* out; int out_dtype; int64_t out_sb, out_sh;
    int batch, hq, hk, group;
    float scale;
    const int64_t* rope_pos; const float* rope_cs; int64_t rope_stride; int64_t rope_rows;
    int32_t* counters; float* part_ml; float* part_o;     // only used when chunks > 1
    int32_t* dev_status;
    int stages, splits, chunks, overlap;
    // fused append (direct kernel only): the step's new K/V row is rotated, quantised, written to the
    // pool and attended to in the same launch; q is rotated on the fly (rope_pos / rope_cs above)
    int append;
    const void* k_new; int64_t kn_sb, kn_sh;
    const void* v_new; int64_t vn_sb, vn_sh;
    uint8_t* k_pool_w; uint8_t* v_pool_w;
    uint8_t* evict_out; int64_t evict_sb;
    DecisionRule rule;
};

// Position of sequence b for the cos/sin lookup; a value outside the table is flagged and replaced by 0
// (positions are caller data: an index, so it is checked like slots and pages).
__device__ __forceinline__ int64_t checked_rope_position(const AttnParams& p, int b) {
    const int64_t pos = p.rope_pos[b];
    if (pos < 0 || pos >= p.rope_rows) {
        if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
        return 0;
    }
    return pos;
}

// ------------------------------------------------------------------------------------------------
// Fast kernel
// ------------------------------------------------------------------------------------------------
template <int D>
struct FastCfg {
    static constexpr int kCh = D / 64;          // 64-element chunks of a row
    static constexpr int kKSteps = D / 16;      // MMA k-steps of S = q K^T
    static constexpr int kNT = D / 8;           // MMA n-tiles of O = P V
    static constexpr int kPageBytes = kPage * D;
    static constexpr int kStageBytes = 2 * kPageBytes;
};

// q element (with optional inline neox RoPE and decision-lane zeroing), float32.
__device__ __forceinline__ float load_q_elem(const AttnParams& p, int b, int head, int g, int d, int dim) {
    const int64_t off = (int64_t)b * p.q_sb + (int64_t)head * p.q_sh;
    float x = load_as_float(p.q, off + d, p.q_dtype);
    if (p.rope_pos == nullptr) return x;
    const int half = dim >> 1;
    const bool lower = d < half;
    const int i = lower ? d : d - half;
    float x1 = lower ? x : load_as_float(p.q, off + i, p.q_dtype);
    float x2 = lower ? load_as_float(p.q, off + half + i, p.q_dtype) : x;
    if (g == 0 && i == half - 1) x2 = 0.0f;      // the borrowed decision channel (head_dim - 1)
    const float* cs = p.rope_cs + checked_rope_position(p, b) * p.rope_stride;
    const float c = cs[i], s = cs[half + i];
    return lower ? __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)) : __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
}

// A-fragments of q for head g of the group: qa[4*ch + s] = {q[d0], q[d0+1]} , {q[d0+2], q[d0+3]} with
// d0 = 64*ch + 16*t + 4*s, i.e. lane t reads 16 consecutive elements per 64-element chunk.
template <int D>
__device__ __forceinline__ void load_q_frags(const AttnParams& p, int b, int h, int g, int t,
                                             uint32_t (&qa)[FastCfg<D>::kKSteps][2]) {
    using C = FastCfg<D>;
    const bool active = g < p.group;
    const int head = h * p.group + g;
    const bool vec = p.rope_pos == nullptr && p.q_dtype != FDMS_F32 &&
                     (((uintptr_t)p.q | (uintptr_t)(p.q_sb * 2) | (uintptr_t)(p.q_sh * 2)) & 15) == 0;
#pragma unroll
    for (int ch = 0; ch < C::kCh; ++ch) {
        const int d0 = 64 * ch + 16 * t;
        if (!active) {
#pragma unroll
            for (int s = 0; s < 4; ++s) { qa[4 * ch + s][0] = 0u; qa[4 * ch + s][1] = 0u; }
        } else if (vec) {
            const uint16_t* src = (const uint16_t*)p.q + (int64_t)b * p.q_sb + (int64_t)head * p.q_sh + d0;
            const uint4 w0 = *(const uint4*)src, w1 = *(const uint4*)(src + 8);
            const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int s = 0; s < 4; ++s) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    uint32_t x = w[2 * s + e];
                    if (p.q_dtype == FDMS_BF16) {     // bf16 pair -> f16 pair through float32
                        const float lo = __uint_as_float(x << 16), hi = __uint_as_float(x & 0xffff0000u);
                        x = pack_f16x2(lo, hi);
                    }
                    qa[4 * ch + s][e] = x;
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                float x[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) x[e] = load_q_elem(p, b, head, g, d0 + 4 * s + e, D);
                qa[4 * ch + s][0] = pack_f16x2(x[0], x[1]);
                qa[4 * ch + s][1] = pack_f16x2(x[2], x[3]);
            }
        }
    }
}

// Register image of one 16-row page in the MMA fragment layout of lane (g, t):
//   k[u][ch]  : 16 bytes of K row tokrow(u, g), elements 64*ch + 16*t .. +15
//   va/vb[u][ch]: 8 bytes of V rows tokrow(u, 2t) / tokrow(u, 2t+1), elements 64*ch + 8*g .. +7
template <int D>
struct PageFrags {
    uint4 k[2][FastCfg<D>::kCh];
    uint2 va[2][FastCfg<D>::kCh];
    uint2 vb[2][FastCfg<D>::kCh];
};

// Fragment loads from a page staged in shared memory.
template <int D>
__device__ __forceinline__ void load_frags_smem(const uint8_t* Ks, const uint8_t* Vs, int g, int t, PageFrags<D>& f) {
    using C = FastCfg<D>;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int r = tokrow<false>(u, g);
        if (C::kCh == 1) {
            f.k[u][0] = *(const uint4*)(Ks + r * D + 16 * t);
        } else {
            // 128-byte rows: odd rows read the upper half first so that the two rows of a
            // quarter-warp hit different banks
            const int sw = r & 1;
            const uint4 a = *(const uint4*)(Ks + r * D + 64 * sw + 16 * t);
            const uint4 c = *(const uint4*)(Ks + r * D + 64 * (sw ^ 1) + 16 * t);
            f.k[u][0] = sw ? c : a;
            f.k[u][C::kCh - 1] = sw ? a : c;
        }
        const int rA = tokrow<false>(u, 2 * t), rB = tokrow<false>(u, 2 * t + 1);
#pragma unroll
        for (int ch = 0; ch < C::kCh; ++ch) {
            f.va[u][ch] = *(const uint2*)(Vs + rA * D + 64 * ch + 8 * g);
            f.vb[u][ch] = *(const uint2*)(Vs + rB * D + 64 * ch + 8 * g);
        }
    }
}

// Byte offsets inside a page of the fragments of lane (g, t); computed once per thread.
template <int D, bool LIN>
struct LaneOffsets {
    int k[2], va[2], vb[2];
    __device__ __forceinline__ LaneOffsets(int g, int t) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            k[u] = tokrow<LIN>(u, g) * D + 16 * t;
            va[u] = tokrow<LIN>(u, 2 * t) * D + 8 * g;
            vb[u] = tokrow<LIN>(u, 2 * t + 1) * D + 8 * g;
        }
    }
};

// Fragment loads straight from the pool in global memory (page = 16 consecutive rows at Kg / Vg).
// Per instruction a warp reads whole 32-byte sectors: K 8 rows x 64 bytes, V 4 rows x 64 bytes.
// In a partial page, rows at or beyond `rows` are not read (they may lie outside the pool) and come
// back as zeros.
template <int D, bool LIN>
__device__ __forceinline__ void load_frags_global(const uint8_t* Kg, const uint8_t* Vg, int rows, int g, int t,
                                                  const LaneOffsets<D, LIN>& lo, PageFrags<D>& f) {
    using C = FastCfg<D>;
    if (rows == kPage) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
            for (int ch = 0; ch < C::kCh; ++ch) {
                f.k[u][ch] = __ldcs((const uint4*)(Kg + lo.k[u] + 64 * ch));
                f.va[u][ch] = __ldcs((const uint2*)(Vg + lo.va[u] + 64 * ch));
                f.vb[u][ch] = __ldcs((const uint2*)(Vg + lo.vb[u] + 64 * ch));
            }
        }
        return;
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int r = tokrow<LIN>(u, g);
        const int rA = tokrow<LIN>(u, 2 * t), rB = tokrow<LIN>(u, 2 * t + 1);
#pragma unroll
        for (int ch = 0; ch < C::kCh; ++ch) {
            f.k[u][ch] = r < rows ? __ldcs((const uint4*)(Kg + lo.k[u] + 64 * ch)) : make_uint4(0u, 0u, 0u, 0u);
            f.va[u][ch] = rA < rows ? __ldcs((const uint2*)(Vg + lo.va[u] + 64 * ch)) : make_uint2(0u, 0u);
            f.vb[u][ch] = rB < rows ? __ldcs((const uint2*)(Vg + lo.vb[u] + 64 * ch)) : make_uint2(0u, 0u);
        }
    }
}

// One page (`rows` of its 16 rows valid): online-softmax update of the warp's running state.
// Tokens sit on the M side of both products, so a page costs 4 + 4 MMAs per 64 elements of head_dim
// (no half-empty tiles):
//   S^T[token, head] = K_page[token, d] q[head, d]      A = K (rows tokrow(0, g), tokrow(1, g)), B = q
//   O^T[d, head]    += V_page^T[d, token] P^T[token, head]   A = V^T, B = P^T (movmatrix transpose of S^T's layout)
// A lane (g, t) holds, for heads 2t and 2t+1: scores of tokens tokrow(0, g), tokrow(1, g); running
// maximum m[e] (complete, reduced over g) and partial sum l[e] (this lane's tokens only); and
// o[4 ch + j][2 r + e] = O[head 2t + e][64 ch + 8 g + 2 j + r].
// Fragments of invalid rows must hold finite values (they are masked, not trusted).
template <int D, bool LIN, bool QK8>
__device__ __forceinline__ void process_page(const PageFrags<D>& f, int rows, int g, int t, float sl2,
                                             const uint32_t (&qa)[D / 16][2], float (&m_run)[2],
                                             float (&l_run)[2], float (&o)[FastCfg<D>::kNT / 2][4]) {
    using C = FastCfg<D>;
    // ---- S^T = K q^T ----
    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float sc[2][2];                                  // [token row u][head e]
    if (QK8) {
        // FP8 product: the K bytes are the A operand as loaded (rows tokrow(0, g) and tokrow(1, g); a lane's 16 bytes
        // per row are two k-groups of 8), q is the B operand in two e4m3 parts (qa[w][0] high part, qa[w][1] low
        // part of word w); `sl2` carries 1 / c
#pragma unroll
        for (int ch = 0; ch < C::kCh; ++ch) {
            const uint32_t w0[4] = {f.k[0][ch].x, f.k[0][ch].y, f.k[0][ch].z, f.k[0][ch].w};
            const uint32_t w1[4] = {f.k[1][ch].x, f.k[1][ch].y, f.k[1][ch].z, f.k[1][ch].w};
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                mma_fp8(c, w0[2 * m], w1[2 * m], w0[2 * m + 1], w1[2 * m + 1], qa[4 * ch + 2 * m][0], qa[4 * ch + 2 * m + 1][0]);
                mma_fp8(c2, w0[2 * m], w1[2 * m], w0[2 * m + 1], w1[2 * m + 1], qa[4 * ch + 2 * m][1], qa[4 * ch + 2 * m + 1][1]);
            }
        }
        constexpr float kLo = 1.0f / kQLoGain;
        sc[0][0] = (c[0] + c2[0] * kLo) * sl2; sc[0][1] = (c[1] + c2[1] * kLo) * sl2;
        sc[1][0] = (c[2] + c2[2] * kLo) * sl2; sc[1][1] = (c[3] + c2[3] * kLo) * sl2;
    } else {
        // f16 product: two accumulators, even and odd k-steps, so that the dependent MMA chain is half as long
#pragma unroll
        for (int ch = 0; ch < C::kCh; ++ch) {
            const uint32_t w0[4] = {f.k[0][ch].x, f.k[0][ch].y, f.k[0][ch].z, f.k[0][ch].w};
            const uint32_t w1[4] = {f.k[1][ch].x, f.k[1][ch].y, f.k[1][ch].z, f.k[1][ch].w};
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                uint32_t a0, a1, a2, a3;
                e4m3x4_to_f16x2x2(w0[s], a0, a2);
                e4m3x4_to_f16x2x2(w1[s], a1, a3);
                if (s & 1) mma_full(c2, a0, a1, a2, a3, qa[4 * ch + s][0], qa[4 * ch + s][1]);
                else mma_full(c, a0, a1, a2, a3, qa[4 * ch + s][0], qa[4 * ch + s][1]);
            }
        }
        sc[0][0] = (c[0] + c2[0]) * sl2; sc[0][1] = (c[1] + c2[1]) * sl2;
        sc[1][0] = (c[2] + c2[2]) * sl2; sc[1][1] = (c[3] + c2[3]) * sl2;
    }
    if (rows < kPage) {
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if (tokrow<LIN>(u, g) >= rows) { sc[u][0] = -INFINITY; sc[u][1] = -INFINITY; }
    }
    // ---- online softmax per head (column) with a lazily updated reference: the exponentials are taken
    // relative to m_run, which is only raised (reduce over the two rows and the eight row-lanes, rescale
    // l and O) when some score exceeds it by more than kMaxSlack, i.e. on the first page and rarely
    // afterwards; weights stay below 2^kMaxSlack, far inside f16 / f32 range. ----
    constexpr float kMaxSlack = 8.0f;
    float alpha[2] = {1.0f, 1.0f}, pr[2][2];
    const bool raise = fmaxf(sc[0][0], sc[1][0]) > m_run[0] + kMaxSlack || fmaxf(sc[0][1], sc[1][1]) > m_run[1] + kMaxSlack ||
                       m_run[0] == -INFINITY || m_run[1] == -INFINITY;
    if (__any_sync(0xffffffffu, raise)) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float mx = fmaxf(sc[0][e], sc[1][e]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m_run[e], mx);
            alpha[e] = ex2(m_run[e] - m_new);
            l_run[e] *= alpha[e];
            m_run[e] = m_new;
        }
#pragma unroll
        for (int j = 0; j < C::kNT / 2; ++j) { o[j][0] *= alpha[0]; o[j][1] *= alpha[1]; o[j][2] *= alpha[0]; o[j][3] *= alpha[1]; }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        pr[0][e] = ex2(sc[0][e] - m_run[e]);
        pr[1][e] = ex2(sc[1][e] - m_run[e]);
        l_run[e] += pr[0][e] + pr[1][e];
    }
    const uint32_t b0 = movmatrix_trans(pack_f16x2(pr[0][0], pr[0][1]));       // P^T for tokens 0..7 of the tile
    const uint32_t b1 = movmatrix_trans(pack_f16x2(pr[1][0], pr[1][1]));       // ... tokens 8..15
    // ---- O^T += V^T P^T ----
#pragma unroll
    for (int ch = 0; ch < C::kCh; ++ch) {
        uint2 va0 = f.va[0][ch], vb0 = f.vb[0][ch], va1 = f.va[1][ch], vb1 = f.vb[1][ch];
        if (rows < kPage) {                       // stale bytes must not reach the MMA
            if (tokrow<LIN>(0, 2 * t) >= rows) va0 = make_uint2(0u, 0u);
            if (tokrow<LIN>(0, 2 * t + 1) >= rows) vb0 = make_uint2(0u, 0u);
            if (tokrow<LIN>(1, 2 * t) >= rows) va1 = make_uint2(0u, 0u);
            if (tokrow<LIN>(1, 2 * t + 1) >= rows) vb1 = make_uint2(0u, 0u);
        }
        const uint32_t lo0[2] = {va0.x, va0.y}, hi0[2] = {vb0.x, vb0.y}, lo1[2] = {va1.x, va1.y}, hi1[2] = {vb1.x, vb1.y};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t sel = (j & 1) ? 0x7362u : 0x5140u;
            uint32_t a0, a1, a2, a3;
            e4m3x4_to_f16x2x2(__byte_perm(lo0[j >> 1], hi0[j >> 1], sel), a0, a1);
            e4m3x4_to_f16x2x2(__byte_perm(lo1[j >> 1], hi1[j >> 1], sel), a2, a3);
            mma_full(o[4 * ch + j], a0, a1, a2, a3, b0, b1);
        }
    }
}

// Shared tail of the fast kernels (called by the 256 consumer threads of a CTA): folds the warps'
// partial (m, l, O) in shared memory, sends the CTA's partial to the cluster leader through
// distributed shared memory, and lets the leader (or, with several clusters per span, the last
// leader to arrive) write the output.
template <int D>
constexpr int kPartialStride = D + 4;          // floats per (warp, head) row of the in-CTA partial buffer

template <int D>
__device__ __forceinline__ void fold_and_write(const AttnParams& p, float* s_m, float* s_l, float* s_o, float* r_ml,
                                               float* r_o, int* s_last_ptr, int tid, int warp, int g, int t, int b,
                                               int h, int item, int rank, int chunk, float (&m_run)[2], float (&l_run)[2],
                                               float (&o)[FastCfg<D>::kNT / 2][4]) {
    using C = FastCfg<D>;
    const int S = p.splits, CH = p.chunks, G = p.group;
    // ---- merge the warps' partial (m, l, O): lane (g, t) holds heads 2t, 2t+1 and elements 8g .. 8g+7 ----
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        float l = l_run[e];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        const int hh = 2 * t + e;
        if (g == 0) { s_m[warp * kMaxGroup + hh] = m_run[e]; s_l[warp * kMaxGroup + hh] = l; }
        if (hh < G) {
            // eight consecutive elements per 64-element chunk: two 128-bit stores into the padded row
            float* so = s_o + ((size_t)warp * kMaxGroup + hh) * kPartialStride<D>;
#pragma unroll
            for (int ch = 0; ch < C::kCh; ++ch) {
                float4* dst = (float4*)(so + 64 * ch + 8 * g);
                dst[0] = make_float4(o[4 * ch + 0][e], o[4 * ch + 0][2 + e], o[4 * ch + 1][e], o[4 * ch + 1][2 + e]);
                dst[1] = make_float4(o[4 * ch + 2][e], o[4 * ch + 2][2 + e], o[4 * ch + 3][e], o[4 * ch + 3][2 + e]);
            }
        }
    }
    consumer_bar();
    if (S > 1) cluster_wait_acquire();          // phase 1 complete: the leader's shared memory exists
    const float vs = p.v_scale ? p.v_scale[h] : 1.0f;
    const uint32_t r_ml0 = S > 1 ? map_to_rank(r_ml, 0) : 0u;
    const uint32_t r_o0 = S > 1 ? map_to_rank(r_o, 0) : 0u;
    for (int e = tid; e < G * D; e += kConsumerThreads) {
        const int gg = e / D, d = e - gg * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, s_m[w * kMaxGroup + gg]);
        float acc = 0.0f, Lsum = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                const float f = ex2(s_m[w * kMaxGroup + gg] - M);
                acc += f * s_o[((size_t)w * kMaxGroup + gg) * kPartialStride<D> + d];
                Lsum += f * s_l[w * kMaxGroup + gg];
            }
        }
        if (S == 1 && CH == 1) {
            store_from_float(p.out, (int64_t)b * p.out_sb + (int64_t)(h * G + gg) * p.out_sh + d, p.out_dtype,
                             Lsum > 0.0f ? acc / Lsum * vs : 0.0f);
        } else if (S == 1) {
            r_o[gg * D + d] = acc;
            if (d == 0) { r_ml[gg * 2] = M; r_ml[gg * 2 + 1] = Lsum; }
        } else {
            st_cluster_f32(r_o0 + (uint32_t)(((rank * G + gg) * D + d) * 4), acc);
            if (d == 0) {
                st_cluster_f32(r_ml0 + (uint32_t)(((rank * G + gg) * 2) * 4), M);
                st_cluster_f32(r_ml0 + (uint32_t)(((rank * G + gg) * 2 + 1) * 4), Lsum);
            }
        }
    }
    FDMS_PROBE(kProbeCtaFolded);
    if (S == 1 && CH == 1) return;
    if (S > 1) {
        cluster_arrive_release();               // phase 2: partials are in the leader's shared memory
        cluster_wait_acquire();
        if (rank != 0) return;
    } else {
        consumer_bar();
    }

    // ---- cluster leader: fold the S partials ----
    const int pslot = item * CH + chunk;
    for (int e = tid; e < G * D; e += kConsumerThreads) {
        const int gg = e / D, d = e - gg * D;
        float M = -INFINITY;
        for (int r = 0; r < S; ++r) M = fmaxf(M, r_ml[(r * G + gg) * 2]);
        float acc = 0.0f, Lsum = 0.0f;
        if (M != -INFINITY) {
            for (int r = 0; r < S; ++r) {
                const float f = ex2(r_ml[(r * G + gg) * 2] - M);
                acc += f * r_o[(r * G + gg) * D + d];
                Lsum += f * r_ml[(r * G + gg) * 2 + 1];
            }
        }
        if (CH == 1) {
            store_from_float(p.out, (int64_t)b * p.out_sb + (int64_t)(h * G + gg) * p.out_sh + d, p.out_dtype,
                             Lsum > 0.0f ? acc / Lsum * vs : 0.0f);
        } else {
            p.part_o[((size_t)pslot * kMaxGroup + gg) * D + d] = acc;
            if (d == 0) {
                p.part_ml[((size_t)pslot * kMaxGroup + gg) * 2] = M;
                p.part_ml[((size_t)pslot * kMaxGroup + gg) * 2 + 1] = Lsum;
            }
        }
    }
    FDMS_PROBE(kProbeEnd);
    if (CH == 1) return;

    // ---- several clusters per span: the last leader to arrive folds the chunk partials ----
    __threadfence();
    consumer_bar();
    if (tid == 0) {
        const int prev = atomicAdd(&p.counters[item], 1);
        const int last = prev == CH - 1;
        if (last) p.counters[item] = 0;          // leave the workspace ready for the next call
        *s_last_ptr = last;
    }
    consumer_bar();
    if (*(volatile int*)s_last_ptr) {
        __threadfence();
        for (int e = tid; e < G * D; e += kConsumerThreads) {
            const int gg = e / D, d = e - gg * D;
            float M = -INFINITY;
            for (int c = 0; c < CH; ++c)
                M = fmaxf(M, __ldcg(&p.part_ml[((size_t)(item * CH + c) * kMaxGroup + gg) * 2]));
            float acc = 0.0f, Lsum = 0.0f;
            if (M != -INFINITY) {
                for (int c = 0; c < CH; ++c) {
                    const size_t ps = (size_t)(item * CH + c) * kMaxGroup + gg;
                    const float f = ex2(__ldcg(&p.part_ml[ps * 2]) - M);
                    acc += f * __ldcg(&p.part_o[ps * D + d]);
                    Lsum += f * __ldcg(&p.part_ml[ps * 2 + 1]);
                }
            }
            store_from_float(p.out, (int64_t)b * p.out_sb + (int64_t)(h * G + gg) * p.out_sh + d, p.out_dtype,
                             Lsum > 0.0f ? acc / Lsum * vs : 0.0f);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Staged variant of the fast kernel.  Every warp owns a ring of R page slots in shared memory (a slot
// holds the K page and the V page of one 16-row page) and one mbarrier per slot.  Lane s of the warp
// is the issuer of slot s: it resolves the page (block table or span base), arms the barrier with the
// byte count and starts two bulk asynchronous copies (cp.async.bulk, the TMA unit's untiled form,
// no multicast) that complete on it; all lanes then wait on the barrier, read their MMA fragments from
// the slot and lane s refills it with the warp's page R further on.  There is no producer warp and no
// CTA-wide barrier in the page loop: eight issuers per CTA run in parallel, the prefetch depth costs
// no registers, and a CTA whose range fits its rings (R pages per warp) has ALL of its K/V in flight
// before the dependency on the preceding kernel is resolved.  With the default ring of 3 slots a CTA of head_dim 64
// takes 69 KB of shared memory and about 80 registers per thread, so three CTAs fit on an SM (the host sizes the
// grid for that; FDMS_ATTN_WAVE=1 launches one CTA per SM instead, which leaves room for the next launch of the
// stream to be resident beside this one).
// Every mbarrier wait is bounded; when one runs out the warp raises FDMS_DEV_WAIT_TIMEOUT, stops
// issuing, gives its copies in flight a short time to land and goes on to the merge.
// ------------------------------------------------------------------------------------------------
constexpr int kMaxRing = 8;

template <int D, bool APPEND>
__global__ void __launch_bounds__(kConsumerThreads, (D == 64 ? 3 : 1)) attn_decode_staged_kernel(AttnParams p) {
    using C = FastCfg<D>;
    constexpr int half = D / 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const int R = p.stages;                       // ring slots per warp, 1..kMaxRing
    const int S = p.splits, CH = p.chunks, G = p.group;
    uint8_t* s_ring = smem;                                                   // [warps][R][K page | V page]
    uint64_t* s_bar = (uint64_t*)(s_ring + (size_t)kConsumerWarps * R * C::kStageBytes);   // [warps][R]
    float* s_m = (float*)(s_bar + kConsumerWarps * kMaxRing);                 // [warps][8]
    float* s_l = s_m + kConsumerWarps * kMaxGroup;                            // [warps][8]
    float* s_o = s_l + kConsumerWarps * kMaxGroup;                            // [warps][8][D + 4]
    float* r_ml = s_o + kConsumerWarps * kMaxGroup * kPartialStride<D>;       // [S][G][2]
    float* r_o = r_ml + S * G * 2;                                            // [S][G][D]
    __shared__ int s_last;
    __shared__ __align__(16) __half s_q[APPEND ? kMaxGroup * D : 8];          // rotated q, [G][D]
    __shared__ __align__(16) uint8_t s_new[APPEND ? 2 * D : 16];              // new K row | new V row (FP8)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int item = blockIdx.y;
    const int rank = blockIdx.x % S;
    const int chunk = blockIdx.x / S;
    const int part = chunk * S + rank, nparts = S * CH;
    const int b = item / p.hk, h = item - b * p.hk;

    FDMS_PROBE(kProbeStart);
    if (S > 1) cluster_arrive_relaxed();        // phase 1: "every CTA of the cluster has started"
    grid_launch_dependents();
    if (tid == 0) s_last = 0;

    uint8_t* ring = s_ring + (size_t)warp * R * C::kStageBytes;
    uint64_t* bars = s_bar + warp * kMaxRing;
    if (lane < R) mbar_init(&bars[lane], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();

    // Pages are dealt round-robin twice, as in the direct kernel: warp-local page i is span page
    // pg0 + i * stride_pg.  Lane s looks after the pages i = s, s + R, s + 2R, ...
    const int32_t* btrow = p.bt ? p.bt + (int64_t)b * p.bt_sb + (int64_t)h * p.bt_sh : nullptr;
    const int stride_pg = kConsumerWarps * nparts;
    const int pg0 = part + warp * nparts;
    int32_t my_id = 0;                           // page id of the page this lane issues next
    if (btrow && lane < R) {
        const int pi = pg0 + lane * stride_pg;
        if (pi < p.bt_pages) my_id = btrow[pi];
    }
    const int live = max(0, p.live[(int64_t)b * p.meta_sb + h]);
    const int64_t base = p.bt ? 0 : (int64_t)p.base[(int64_t)b * p.meta_sb + h];
    const int npg = (live + kPage - 1) / kPage;
    const int nw = pg0 < npg ? (npg - pg0 + stride_pg - 1) / stride_pg : 0;     // pages of this warp
    const int tail_pi = npg - 1;

    // fused append: see the direct kernel
    constexpr int kItemsK = half, kItemsV = D / 2;
    const bool tail_cta = APPEND && live > 0 && (tail_pi % nparts) == part;
    const int n_items = APPEND ? G * half + (tail_cta ? kItemsK + kItemsV : 0) : 0;
    const float* cs_row = APPEND ? p.rope_cs + checked_rope_position(p, b) * p.rope_stride : nullptr;
    // The cos/sin pair of this thread's first rotation item does not depend on the preceding kernel; the
    // activation it will rotate does, so only its cache line is requested into L2 here (a hint: the value
    // itself is read after the dependency has been resolved).
    float pre_c = 1.0f, pre_s = 0.0f;
    if (APPEND && tid < n_items && tid < G * half + kItemsK) {
        const bool isq = tid < G * half;
        const int gg = isq ? tid / half : 0, i = isq ? tid - gg * half : tid - G * half;
        pre_c = cs_row[i];
        pre_s = cs_row[half + i];
        const int64_t row = isq ? (int64_t)b * p.q_sb + (int64_t)(h * G + gg) * p.q_sh : (int64_t)b * p.kn_sb + (int64_t)h * p.kn_sh;
        const char* src = (const char*)(isq ? p.q : p.k_new) + (row + i) * dtype_size(p.q_dtype);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
    }

    // Issues warp-local page i into slot i % R (called by the slot's lane only).  Returns false when
    // the page address is out of range: the slot's barrier is completed without a copy and the page is
    // skipped by the consumer.
    auto issue = [&](int i, int s, int32_t id) -> bool {
        const int pi = pg0 + i * stride_pg;
        const int rows = min(kPage, live - pi * kPage);
        // in append mode the span's last row is not in the pool yet: it is patched into the slot
        const int have = (APPEND && pi == tail_pi) ? rows - 1 : rows;
        const int64_t row0 = btrow ? (int64_t)id * kPage : base + (int64_t)pi * kPage;
        if (row0 < 0 || row0 + rows > p.pool_rows) {
            if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
            mbar_arrive(&bars[s]);
            return false;
        }
        if (have == 0) { mbar_arrive(&bars[s]); return true; }
        const uint32_t bytes = (uint32_t)have * D;
        uint8_t* dst = ring + (size_t)s * C::kStageBytes;
        // the warp's reads of the slot (generic proxy) are ordered before the copy's writes (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(&bars[s], 2 * bytes);
        bulk_g2s(dst, p.k_pool + row0 * D, bytes, &bars[s]);
        bulk_g2s(dst + C::kPageBytes, p.v_pool + row0 * D, bytes, &bars[s]);
        return true;
    };
    auto next_id = [&](int i) {                  // start fetching the id of warp-local page i
        const int pi = pg0 + i * stride_pg;
        if (btrow && pi < npg && pi < p.bt_pages) my_id = btrow[pi];
    };

    bool my_ok = true;
    // Without append the span's last page holds the row that the preceding kernel of the stream (the
    // store) has just written; it is fetched only after the dependency has been resolved.
    const bool my_first = lane < R && lane < nw;
    const bool deferred = !APPEND && my_first && pg0 + lane * stride_pg == tail_pi;
    if (my_first && !deferred) {
        my_ok = issue(lane, lane, my_id);
        next_id(lane + R);
    }
    int64_t tail_row = -1;                           // pool row of the new token (block tables are older state)
    if (APPEND && tail_cta) {
        const int64_t trow0 = btrow ? (tail_pi < p.bt_pages ? (int64_t)btrow[tail_pi] * kPage : -1)
                                    : base + (int64_t)tail_pi * kPage;
        const int64_t r = trow0 + (live - 1 - tail_pi * kPage);
        tail_row = (trow0 >= 0 && r < p.pool_rows) ? r : -2;
    }
    FDMS_PROBE(kProbeIssued);
    grid_dependency_wait();
    FDMS_PROBE(kProbeDependency);
    if (deferred) {
        my_ok = issue(lane, lane, my_id);
        next_id(lane + R);
    }

    const float sl2 = p.scale * (p.k_scale ? p.k_scale[h] : 1.0f) * kLog2e;
    uint32_t qa[C::kKSteps][2];
    if (APPEND) {
        for (int it = tid; it < n_items; it += kConsumerThreads) {
            if (it < G * half + kItemsK) {
                // one rotation pair of a q head (it < G * half) or of the new K row
                const bool isq = it < G * half;
                const int gg = isq ? it / half : 0, i = isq ? it - gg * half : it - G * half;
                const void* src = isq ? p.q : p.k_new;
                const int64_t row = isq ? (int64_t)b * p.q_sb + (int64_t)(h * G + gg) * p.q_sh
                                        : (int64_t)b * p.kn_sb + (int64_t)h * p.kn_sh;
                const float x1 = load_as_float(src, row + i, p.q_dtype);
                float x2 = load_as_float(src, row + half + i, p.q_dtype);
                const float c = it == tid ? pre_c : cs_row[i], sn = it == tid ? pre_s : cs_row[half + i];
                if (isq && gg == 0 && i == half - 1) {
                    // the group's first q head carries the DMS decision in its last channel
                    if (tail_cta && p.evict_out) p.evict_out[(int64_t)b * p.evict_sb + h] = p.rule.evict(x2) ? 1 : 0;
                    x2 = 0.0f;
                }
                // float32, unfused, rounded to the activation dtype: the store kernel's arithmetic
                const float lo = round_to_dtype(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn)), p.q_dtype);
                const float hi = round_to_dtype(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn)), p.q_dtype);
                if (isq) {
                    s_q[gg * D + i] = __float2half_rn(lo);
                    s_q[gg * D + half + i] = __float2half_rn(hi);
                } else {
                    const float ksc = p.k_scale ? p.k_scale[h] : 1.0f;
                    const uint8_t bl = float_to_e4m3(p.k_scale ? __fdiv_rn(lo, ksc) : lo);
                    const uint8_t bh = float_to_e4m3(p.k_scale ? __fdiv_rn(hi, ksc) : hi);
                    s_new[i] = bl;
                    s_new[half + i] = bh;
                    if (tail_row >= 0) {
                        p.k_pool_w[tail_row * D + i] = bl;
                        p.k_pool_w[tail_row * D + half + i] = bh;
                    }
                    if (tail_row == -2 && i == 0 && p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
                }
            } else {
                // two elements of the new V row
                const int i = 2 * (it - G * half - kItemsK);
                const int64_t e0 = (int64_t)b * p.vn_sb + (int64_t)h * p.vn_sh + i;
                float y0 = load_as_float(p.v_new, e0, p.q_dtype), y1 = load_as_float(p.v_new, e0 + 1, p.q_dtype);
                if (p.v_scale) { const float vsc = p.v_scale[h]; y0 = __fdiv_rn(y0, vsc); y1 = __fdiv_rn(y1, vsc); }
                const uchar2 bv = make_uchar2(float_to_e4m3(y0), float_to_e4m3(y1));
                *(uchar2*)(s_new + D + i) = bv;
                if (tail_row >= 0) *(uchar2*)(p.v_pool_w + tail_row * D + i) = bv;
            }
        }
        __syncthreads();
#pragma unroll
        for (int ch = 0; ch < C::kCh; ++ch) {
            uint4 w0 = make_uint4(0u, 0u, 0u, 0u), w1 = w0;
            if (g < G) {
                const uint4* src = (const uint4*)(s_q + g * D + 64 * ch + 16 * t);
                w0 = src[0]; w1 = src[1];
            }
            qa[4 * ch + 0][0] = w0.x; qa[4 * ch + 0][1] = w0.y; qa[4 * ch + 1][0] = w0.z; qa[4 * ch + 1][1] = w0.w;
            qa[4 * ch + 2][0] = w1.x; qa[4 * ch + 2][1] = w1.y; qa[4 * ch + 3][0] = w1.z; qa[4 * ch + 3][1] = w1.w;
        }
    } else {
        load_q_frags<D>(p, b, h, g, t, qa);
    }
    FDMS_PROBE(kProbeQReady);

    const int r_new = live - 1 - tail_pi * kPage;            // row of the new token inside the span's last page
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[C::kNT / 2][4];
#pragma unroll
    for (int j = 0; j < C::kNT / 2; ++j) { o[j][0] = 0.0f; o[j][1] = 0.0f; o[j][2] = 0.0f; o[j][3] = 0.0f; }

    // The page loop, once per form of the score product; a warp with many pages quantises q and takes the FP8 form.
    auto page_loop = [&](auto qk8_tag, float sl2w) {
        constexpr bool QK8 = decltype(qk8_tag)::value;
        int issued = min(nw, R);                 // warp-local pages whose slot has been armed
        int s = 0;
        uint32_t phase = 0;
        for (int i = 0; i < nw; ++i) {
            const bool landed = mbar_wait(&bars[s], phase, kWaitLimit);
            if (!__all_sync(0xffffffffu, landed)) {
                if (lane == 0 && p.dev_status) atomicOr(p.dev_status, FDMS_DEV_WAIT_TIMEOUT);
                for (int j = i; j < issued; ++j) mbar_wait(&bars[j % R], (uint32_t)(j / R) & 1u, kWaitLimitDrain);
                break;
            }
            const int pi = pg0 + i * stride_pg;
            const int rows = min(kPage, live - pi * kPage);
            const bool good = __shfl_sync(0xffffffffu, my_ok, s);
            uint8_t* Ks = ring + (size_t)s * C::kStageBytes;
            if (APPEND && pi == tail_pi) {
                // the new row of the span is not in the pool image the copy brought: write it into the slot
                if (lane < D / 16) *(uint4*)(Ks + r_new * D + 16 * lane) = *(const uint4*)(s_new + 16 * lane);
                else if (lane < D / 8) *(uint4*)(Ks + C::kPageBytes + r_new * D + 16 * (lane - D / 16)) = *(const uint4*)(s_new + D + 16 * (lane - D / 16));
                __syncwarp();
            }
            if (good) {
                PageFrags<D> f;
                load_frags_smem<D>(Ks, Ks + C::kPageBytes, g, t, f);
                process_page<D, false, QK8>(f, rows, g, t, sl2w, qa, m_run, l_run, o);
            }
            __syncwarp();                         // every lane has consumed its fragments of the slot
            if (i + R < nw) {
                if (lane == s) { my_ok = issue(i + R, s, my_id); next_id(i + 2 * R); }
                ++issued;
            }
            if (++s == R) { s = 0; phase ^= 1u; }
        }
    };
    if (nw >= kQk8MinPages) {
        float inv_c;
        quantize_q<D>(qa, inv_c);
        page_loop(std::true_type{}, sl2 * inv_c);
    } else {
        page_loop(std::false_type{}, sl2);
    }
    __syncthreads();                              // s_last initialised, all warps done with their pages
    FDMS_PROBE(kProbePagesDone);
    fold_and_write<D>(p, s_m, s_l, s_o, r_ml, r_o, &s_last, tid, warp, g, t, b, h, item, rank, chunk, m_run, l_run, o);
}

// ------------------------------------------------------------------------------------------------
// Direct-load variant of the fast kernel: no staging in shared memory.  Every warp reads the pages it
// owns straight from the pool into registers, already in MMA fragment layout, with 128-bit (K) and
// 64-bit (V) loads that cover whole 32-byte sectors, and keeps DEPTH pages in flight ahead of the
// one it is computing on.  Measured on B200 (a pure-load kernel over the same pages): per-lane vector loads of
// 1 KiB K + 1 KiB V pages reach the streaming rate (6.7 TB/s), bulk copies of the same pages into per-warp rings
// 5.4 TB/s; in the attention kernel itself the staged variant loses on instruction count, not on the copies.
// ------------------------------------------------------------------------------------------------
constexpr int kDirectThreads = kConsumerThreads;

// APPEND = true is the fused store + attention launch: the step's new K/V row is not in the pool yet.
// After the dependency wait a few threads build, through shared memory and once per CTA,
//   * the rotated q of the whole head group (f16, what the MMA consumes), and
//   * in the CTA that owns the span's last page, the new row: DMS decision, rotated K and V quantised
//     to FP8, written to the pool and patched into the register image of that page.
// Work is split in 8-element units so that every unit is one 16-byte load per operand.
template <int D, int DEPTH, bool APPEND>
__global__ void __launch_bounds__(kDirectThreads, (D == 64 ? 2 : 1)) attn_decode_direct_kernel(AttnParams p) {
    using C = FastCfg<D>;
    constexpr int half = D / 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const int S = p.splits, CH = p.chunks, G = p.group;
    float* s_m = (float*)smem;                                // [warps][8]
    float* s_l = s_m + kConsumerWarps * kMaxGroup;            // [warps][8]
    float* s_o = s_l + kConsumerWarps * kMaxGroup;            // [warps][8][D]
    float* r_ml = s_o + kConsumerWarps * kMaxGroup * kPartialStride<D>;       // [S][G][2]
    float* r_o = r_ml + S * G * 2;                            // [S][G][D]
    __shared__ int s_last;
    __shared__ __align__(16) __half s_q[APPEND ? kMaxGroup * D : 8];     // rotated q, [G][D]
    __shared__ __align__(16) uint8_t s_new[APPEND ? 2 * D : 16];         // new K row | new V row (FP8)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int item = blockIdx.y;
    const int rank = blockIdx.x % S;
    const int chunk = blockIdx.x / S;
    const int part = chunk * S + rank, nparts = S * CH;
    const int b = item / p.hk, h = item - b * p.hk;

    FDMS_PROBE(kProbeStart);
    if (S > 1) cluster_arrive_relaxed();        // phase 1: "every CTA of the cluster has started"
    grid_launch_dependents();
    if (tid == 0) s_last = 0;

    // Pages are dealt round-robin twice: page pi of the span belongs to CTA pi % nparts, and inside a
    // CTA its local pages go to warps round-robin.  Warp-local page i is span page
    // part + (warp + 8 i) * nparts, which is known before the span length is.
    const int32_t* btrow = p.bt ? p.bt + (int64_t)b * p.bt_sb + (int64_t)h * p.bt_sh : nullptr;
    const int stride_pg = kConsumerWarps * nparts;
    const int pg0 = part + warp * nparts;
    int32_t idreg[DEPTH];
#pragma unroll
    for (int s = 0; s < DEPTH; ++s) {
        const int pi = pg0 + s * stride_pg;
        idreg[s] = (btrow && pi < p.bt_pages) ? btrow[pi] : 0;
    }
    const int live = max(0, p.live[(int64_t)b * p.meta_sb + h]);
    const int64_t base = p.bt ? 0 : (int64_t)p.base[(int64_t)b * p.meta_sb + h];
    const int npg = (live + kPage - 1) / kPage;
    const int nw = pg0 < npg ? (npg - pg0 + stride_pg - 1) / stride_pg : 0;     // pages of this warp
    const int tail_pi = npg - 1;

    // ---- fused append ----
    // After the dependency wait the CTA builds, one (lower, upper) rotation pair per thread so that no
    // thread runs a long serial chain: the rotated q of the head group (G * D/2 pairs, every CTA) and,
    // in the CTA that owns the span's last page, the new K row (D/2 pairs) and V row (2 elements per
    // thread).  Only the position's cos/sin row address is resolved before the wait.
    constexpr int kItemsK = half, kItemsV = D / 2;
    const bool tail_cta = APPEND && live > 0 && (tail_pi % nparts) == part;
    const int n_items = APPEND ? G * half + (tail_cta ? kItemsK + kItemsV : 0) : 0;
    const float* cs_row = APPEND ? p.rope_cs + checked_rope_position(p, b) * p.rope_stride : nullptr;
    // The cos/sin pair of this thread's first rotation item does not depend on the preceding kernel; the
    // activation it will rotate does, so only its cache line is requested into L2 here (a hint: the value
    // itself is read after the dependency has been resolved).
    float pre_c = 1.0f, pre_s = 0.0f;
    if (APPEND && tid < n_items && tid < G * half + kItemsK) {
        const bool isq = tid < G * half;
        const int gg = isq ? tid / half : 0, i = isq ? tid - gg * half : tid - G * half;
        pre_c = cs_row[i];
        pre_s = cs_row[half + i];
        const int64_t row = isq ? (int64_t)b * p.q_sb + (int64_t)(h * G + gg) * p.q_sh : (int64_t)b * p.kn_sb + (int64_t)h * p.kn_sh;
        const char* src = (const char*)(isq ? p.q : p.k_new) + (row + i) * dtype_size(p.q_dtype);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
    }

    const LaneOffsets<D, true> lofs(g, t);
    PageFrags<D> buf[DEPTH];
    int brow[DEPTH];
    // Issues the loads of warp-local page i into buffer slot s (page id taken from idreg[s]), then
    // starts fetching the page id that slot s will need next.
    auto issue = [&](int s, int i) {
        const int pi = pg0 + i * stride_pg;
        const int rows = min(kPage, live - pi * kPage);
        const int64_t row0 = btrow ? (int64_t)idreg[s] * kPage : base + (int64_t)pi * kPage;
        if (row0 < 0 || row0 + rows > p.pool_rows) {
            if (lane == 0 && p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
            brow[s] = 0;
        } else {
            brow[s] = rows;
            // in append mode the span's last row is not in the pool yet: it is patched in below
            const int have = (APPEND && pi == tail_pi) ? rows - 1 : rows;
            load_frags_global<D, true>(p.k_pool + row0 * D, p.v_pool + row0 * D, have, g, t, lofs, buf[s]);
        }
        const int nxt = pi + DEPTH * stride_pg;
        if (btrow && nxt < npg && nxt < p.bt_pages) idreg[s] = btrow[nxt];
    };
#pragma unroll
    for (int s = 0; s < DEPTH; ++s) {
        brow[s] = 0;
        if (s < nw && pg0 + s * stride_pg != tail_pi) issue(s, s);
    }
    int64_t tail_row = -1;                           // pool row of the new token (block tables are older state)
    if (APPEND && tail_cta) {
        const int64_t trow0 = btrow ? (tail_pi < p.bt_pages ? (int64_t)btrow[tail_pi] * kPage : -1)
                                    : base + (int64_t)tail_pi * kPage;
        const int64_t r = trow0 + (live - 1 - tail_pi * kPage);
        tail_row = (trow0 >= 0 && r < p.pool_rows) ? r : -2;
    }
    // The span's last page holds the row written by the preceding kernel of the stream (or, in append
    // mode, older rows only), and q / k / v come from it: all are read only after the dependency has
    // been resolved.
    FDMS_PROBE(kProbeIssued);
    grid_dependency_wait();
    FDMS_PROBE(kProbeDependency);
#pragma unroll
    for (int s = 0; s < DEPTH; ++s)
        if (s < nw && pg0 + s * stride_pg == tail_pi) issue(s, s);

    const float sl2 = p.scale * (p.k_scale ? p.k_scale[h] : 1.0f) * kLog2e;
    uint32_t qa[C::kKSteps][2];
    if (APPEND) {
        for (int it = tid; it < n_items; it += kDirectThreads) {
            if (it < G * half + kItemsK) {
                // one rotation pair of a q head (it < G * half) or of the new K row
                const bool isq = it < G * half;
                const int gg = isq ? it / half : 0, i = isq ? it - gg * half : it - G * half;
                const void* src = isq ? p.q : p.k_new;
                const int64_t row = isq ? (int64_t)b * p.q_sb + (int64_t)(h * G + gg) * p.q_sh
                                        : (int64_t)b * p.kn_sb + (int64_t)h * p.kn_sh;
                const float x1 = load_as_float(src, row + i, p.q_dtype);
                float x2 = load_as_float(src, row + half + i, p.q_dtype);
                const float c = it == tid ? pre_c : cs_row[i], sn = it == tid ? pre_s : cs_row[half + i];
                if (isq && gg == 0 && i == half - 1) {
                    // the group's first q head carries the DMS decision in its last channel
                    if (tail_cta && p.evict_out) p.evict_out[(int64_t)b * p.evict_sb + h] = p.rule.evict(x2) ? 1 : 0;
                    x2 = 0.0f;
                }
                // float32, unfused, rounded to the activation dtype: the store kernel's arithmetic
                const float lo = round_to_dtype(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn)), p.q_dtype);
                const float hi = round_to_dtype(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn)), p.q_dtype);
                if (isq) {
                    s_q[gg * D + i] = __float2half_rn(lo);
                    s_q[gg * D + half + i] = __float2half_rn(hi);
                } else {
                    const float ksc = p.k_scale ? p.k_scale[h] : 1.0f;
                    const uint8_t bl = float_to_e4m3(p.k_scale ? __fdiv_rn(lo, ksc) : lo);
                    const uint8_t bh = float_to_e4m3(p.k_scale ? __fdiv_rn(hi, ksc) : hi);
                    s_new[i] = bl;
                    s_new[half + i] = bh;
                    if (tail_row >= 0) {
                        p.k_pool_w[tail_row * D + i] = bl;
                        p.k_pool_w[tail_row * D + half + i] = bh;
                    }
                    if (tail_row == -2 && i == 0 && p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
                }
            } else {
                // two elements of the new V row
                const int i = 2 * (it - G * half - kItemsK);
                const int64_t e0 = (int64_t)b * p.vn_sb + (int64_t)h * p.vn_sh + i;
                float y0 = load_as_float(p.v_new, e0, p.q_dtype), y1 = load_as_float(p.v_new, e0 + 1, p.q_dtype);
                if (p.v_scale) { const float vsc = p.v_scale[h]; y0 = __fdiv_rn(y0, vsc); y1 = __fdiv_rn(y1, vsc); }
                const uchar2 bv = make_uchar2(float_to_e4m3(y0), float_to_e4m3(y1));
                *(uchar2*)(s_new + D + i) = bv;
                if (tail_row >= 0) *(uchar2*)(p.v_pool_w + tail_row * D + i) = bv;
            }
        }
        __syncthreads();
#pragma unroll
        for (int ch = 0; ch < C::kCh; ++ch) {
            uint4 w0 = make_uint4(0u, 0u, 0u, 0u), w1 = w0;
            if (g < G) {
                const uint4* src = (const uint4*)(s_q + g * D + 64 * ch + 16 * t);
                w0 = src[0]; w1 = src[1];
            }
            qa[4 * ch + 0][0] = w0.x; qa[4 * ch + 0][1] = w0.y; qa[4 * ch + 1][0] = w0.z; qa[4 * ch + 1][1] = w0.w;
            qa[4 * ch + 2][0] = w1.x; qa[4 * ch + 2][1] = w1.y; qa[4 * ch + 3][0] = w1.z; qa[4 * ch + 3][1] = w1.w;
        }
    } else {
        load_q_frags<D>(p, b, h, g, t, qa);
    }
    FDMS_PROBE(kProbeQReady);

    // the warp that owns the span's last page patches the new row into its register image
    const bool own_tail = APPEND && nw > 0 && tail_pi >= pg0 && (tail_pi - pg0) % stride_pg == 0;
    const int r_new = live - 1 - tail_pi * kPage;            // row of the new token inside that page

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[C::kNT / 2][4];
#pragma unroll
    for (int j = 0; j < C::kNT / 2; ++j) { o[j][0] = 0.0f; o[j][1] = 0.0f; o[j][2] = 0.0f; o[j][3] = 0.0f; }

    // The page loop, once per form of the score product; a warp with many pages quantises q and takes the FP8 form.
    auto page_loop = [&](auto qk8_tag, float sl2w) {
        constexpr bool QK8 = decltype(qk8_tag)::value;
        for (int i0 = 0; i0 < nw; i0 += DEPTH) {
#pragma unroll
            for (int s = 0; s < DEPTH; ++s) {
                const int i = i0 + s;
                if (i < nw) {
                    if (APPEND && own_tail && pg0 + i * stride_pg == tail_pi) {
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
#pragma unroll
                            for (int ch = 0; ch < C::kCh; ++ch) {
                                if (tokrow<true>(u, g) == r_new) buf[s].k[u][ch] = *(const uint4*)(s_new + 64 * ch + 16 * t);
                                if (tokrow<true>(u, 2 * t) == r_new) buf[s].va[u][ch] = *(const uint2*)(s_new + D + 64 * ch + 8 * g);
                                if (tokrow<true>(u, 2 * t + 1) == r_new) buf[s].vb[u][ch] = *(const uint2*)(s_new + D + 64 * ch + 8 * g);
                            }
                        }
                    }
                    if (brow[s] > 0) process_page<D, true, QK8>(buf[s], brow[s], g, t, sl2w, qa, m_run, l_run, o);
                    if (i + DEPTH < nw) issue(s, i + DEPTH);
                }
            }
        }
    };
    if (nw >= kQk8MinPages) {
        float inv_c;
        quantize_q<D>(qa, inv_c);
        page_loop(std::true_type{}, sl2 * inv_c);
    } else {
        page_loop(std::false_type{}, sl2);
    }
    __syncthreads();                              // s_last initialised, all warps done with their pages
    FDMS_PROBE(kProbePagesDone);
    fold_and_write<D>(p, s_m, s_l, s_o, r_ml, r_o, &s_last, tid, warp, g, t, b, h, item, rank, chunk, m_run, l_run, o);
}

// ------------------------------------------------------------------------------------------------
// Generic kernel: one CTA (4 warps) per (sequence, q head); warps stride over the span's rows,
// lanes over head_dim.
// ------------------------------------------------------------------------------------------------
constexpr int kGenWarps = 4;
constexpr int kGenMaxPerLane = 8;      // head_dim <= 256

struct GenParams {
    AttnParams a;
    const void* k_pool; const void* v_pool; int kv_dtype; int dim;
};

__global__ void __launch_bounds__(kGenWarps * 32) attn_decode_generic_kernel(GenParams gp) {
    const AttnParams& p = gp.a;
    const int D = gp.dim;
    __shared__ float s_m[kGenWarps], s_l[kGenWarps];
    __shared__ float s_o[kGenWarps][kGenMaxPerLane * 32];
    const int b = blockIdx.x / p.hq, hq = blockIdx.x % p.hq;
    const int h = hq / p.group, g = hq % p.group;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int live = max(0, p.live[(int64_t)b * p.meta_sb + h]);
    const int base = p.base ? p.base[(int64_t)b * p.meta_sb + h] : 0;
    const int32_t* bt = p.bt ? p.bt + (int64_t)b * p.bt_sb + (int64_t)h * p.bt_sh : nullptr;
    const float ksc = p.scale * (p.k_scale ? p.k_scale[h] : 1.0f);
    float q[kGenMaxPerLane], acc[kGenMaxPerLane];
#pragma unroll
    for (int e = 0; e < kGenMaxPerLane; ++e) {
        const int d = lane + 32 * e;
        q[e] = d < D ? load_q_elem(p, b, hq, g, d, D) : 0.0f;
        acc[e] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int i = warp; i < live; i += kGenWarps) {
        const int64_t row = span_row(base, bt, i);
        if (row < 0 || row >= p.pool_rows) {
            if (lane == 0 && p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
            continue;
        }
        float dot = 0.0f;
#pragma unroll
        for (int e = 0; e < kGenMaxPerLane; ++e) {
            const int d = lane + 32 * e;
            if (d < D) dot += q[e] * load_as_float(gp.k_pool, row * D + d, gp.kv_dtype);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float s = dot * ksc;
        const float m_new = fmaxf(m, s);
        const float alpha = __expf(m - m_new), pr = __expf(s - m_new);
        l = l * alpha + pr;
        m = m_new;
#pragma unroll
        for (int e = 0; e < kGenMaxPerLane; ++e) {
            const int d = lane + 32 * e;
            if (d < D) acc[e] = acc[e] * alpha + pr * load_as_float(gp.v_pool, row * D + d, gp.kv_dtype);
        }
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < kGenMaxPerLane; ++e) s_o[warp][lane + 32 * e] = acc[e];
    __syncthreads();
    const float vs = p.v_scale ? p.v_scale[h] : 1.0f;
    for (int d = threadIdx.x; d < D; d += kGenWarps * 32) {
        float M = -INFINITY;
        for (int w = 0; w < kGenWarps; ++w) M = fmaxf(M, s_m[w]);
        float a = 0.0f, L = 0.0f;
        for (int w = 0; w < kGenWarps; ++w) {
            const float f = (s_m[w] == -INFINITY) ? 0.0f : __expf(s_m[w] - M);
            a += f * s_o[w][d];
            L += f * s_l[w];
        }
        const float r = live > 0 ? a / L * vs : 0.0f;
        store_from_float(p.out, (int64_t)b * p.out_sb + (int64_t)hq * p.out_sh + d, p.out_dtype, r);
    }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
constexpr int kMaxPartialSlots = 1024;     // spans * chunks when chunks > 1

struct DeviceInfo { int sms; int smem_optin; bool ok; };

static DeviceInfo device_info() {
    // One entry per device ordinal, filled on first use (the values never change).
    static DeviceInfo cache[64];
    static bool have[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DeviceInfo{0, 0, false};
    if (!have[dev]) {
        DeviceInfo d{0, 0, true};
        if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) d.ok = false;
        if (cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) d.ok = false;
        cache[dev] = d;
        have[dev] = true;
    }
    return cache[dev];
}

static int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    if (!v || !*v) return dflt;
    return atoi(v);
}

static size_t staged_smem_bytes(int D, int ring, int splits, int group) {
    size_t s = (size_t)kConsumerWarps * ring * 2 * kPage * D;       // per-warp rings
    s += (size_t)kConsumerWarps * kMaxRing * sizeof(uint64_t);     // barriers
    s += (size_t)kConsumerWarps * kMaxGroup * (2 + D + 4) * sizeof(float);
    s += (size_t)splits * group * (2 + D) * sizeof(float);
    return s + 128;
}

static size_t direct_smem_bytes(int D, int splits, int group) {
    return (size_t)kConsumerWarps * kMaxGroup * (2 + D + 4) * sizeof(float) + (size_t)splits * group * (2 + D) * sizeof(float) + 128;
}

typedef void (*AttnKernel)(AttnParams);

static void fill_launch_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int threads, int splits, int chunks,
                               int items, size_t smem, cudaStream_t stream, bool overlap = false) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3((unsigned)(splits * chunks), (unsigned)items, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (overlap) {
        attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
        ++cfg.numAttrs;
    }
    // cluster placement: load balancing measured 2 % faster per launch than the default (spread) at 64 clusters of 4
    const int policy = env_int("FDMS_ATTN_CLUSTER_POLICY", 2);      // 0 = driver default, 1 = spread, 2 = load balancing
    if (policy == 1 || policy == 2) {
        attr[cfg.numAttrs].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
        attr[cfg.numAttrs].val.clusterSchedulingPolicyPreference =
            policy == 1 ? cudaClusterSchedulingPolicySpread : cudaClusterSchedulingPolicyLoadBalancing;
        ++cfg.numAttrs;
    }
}

// Whether a cluster of `splits` CTAs with `smem` bytes each can be resident on this device.
// Asked once per (kernel variant, splits, smem) and remembered.
static bool cluster_fits(AttnKernel kern, int variant, int threads, int splits, size_t smem) {
    static size_t known_smem[8][kMaxSplits + 1] = {{0}};
    static int known[8][kMaxSplits + 1] = {{0}};     // 0 unknown, 1 fits, -1 does not
    if (splits == 1) return true;
    if (known[variant][splits] != 0 && known_smem[variant][splits] == smem) return known[variant][splits] > 0;
    bool ok = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
    if (ok && splits > 8) ok = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    if (ok) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[3];
        fill_launch_config(cfg, attr, threads, splits, 1, 1, smem, nullptr);
        int n = 0;
        ok = cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0;
    }
    cudaGetLastError();                               // a failed query must not poison the next launch check
    known[variant][splits] = ok ? 1 : -1;
    known_smem[variant][splits] = smem;
    return ok;
}

static cudaError_t launch_attn(AttnKernel kern, int threads, const AttnParams& p, int items, size_t smem, cudaStream_t stream,
                               bool max_shared) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (max_shared) {
        // the staged kernel wants two CTAs of about 100 KB on an SM: ask for the largest shared-memory carve-out
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
    }
    if (p.splits > 8) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[3];
    fill_launch_config(cfg, attr, threads, p.splits, p.chunks, items, smem, stream, p.overlap != 0);
    return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace fdms

using namespace fdms;

extern "C" int64_t fdms_attn_decode_workspace_bytes(int32_t batch, int32_t num_kv_heads, int32_t head_dim) {
    if (batch < 0 || num_kv_heads <= 0 || head_dim <= 0) return -1;
    const int64_t counters = (((int64_t)batch * num_kv_heads * 4 + 255) / 256) * 256;
    const int64_t ml = (int64_t)kMaxPartialSlots * kMaxGroup * 2 * 4;
    const int64_t po = (int64_t)kMaxPartialSlots * kMaxGroup * head_dim * 4;
    return counters + ml + po;
}

namespace fdms {
struct AppendArgs {
    const void* k_new; int64_t kn_sb, kn_sh;
    const void* v_new; int64_t vn_sb, vn_sh;
    uint8_t* evict_out; int64_t evict_sb;
    double alpha_scale, alpha_offset;
};
}  // namespace fdms

// Argument checks shared by every attention entry point (nothing is enqueued before they pass).
static int32_t validate_attn_args(
    const void* q, int32_t q_dtype, const void* k_pool, const void* v_pool, int32_t kv_dtype,
    const int32_t* base_offsets, const int32_t* live_counts, const int32_t* block_tables, int32_t bt_max_pages,
    const void* out, int32_t out_dtype, int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
    const int64_t* q_rope_positions, const float* q_rope_cos_sin, int64_t cos_sin_rows) {
    FDMS_REQUIRE(q && k_pool && v_pool && live_counts && out, FDMS_E_ARG, "fdms_attn_decode: null pointer");
    FDMS_REQUIRE(base_offsets || block_tables, FDMS_E_ARG, "fdms_attn_decode: base_offsets or block_tables required");
    FDMS_REQUIRE(!block_tables || bt_max_pages > 0, FDMS_E_ARG, "fdms_attn_decode: bt_max_pages must be positive");
    FDMS_REQUIRE(batch >= 0 && num_q_heads > 0 && num_kv_heads > 0 && head_dim > 0, FDMS_E_ARG,
                 "fdms_attn_decode: bad sizes");
    FDMS_REQUIRE(num_q_heads % num_kv_heads == 0, FDMS_E_ARG, "q_heads=%d must be divisible by kv_heads=%d",
                 num_q_heads, num_kv_heads);
    FDMS_REQUIRE(head_dim <= 256, FDMS_E_CAPACITY, "head_dim=%d is above the kernel limit of 256", head_dim);
    FDMS_REQUIRE(q_dtype == FDMS_F32 || q_dtype == FDMS_BF16 || q_dtype == FDMS_F16, FDMS_E_DTYPE,
                 "fdms_attn_decode: q dtype %d not supported", q_dtype);
    FDMS_REQUIRE(out_dtype == FDMS_F32 || out_dtype == FDMS_BF16 || out_dtype == FDMS_F16, FDMS_E_DTYPE,
                 "fdms_attn_decode: out dtype %d not supported", out_dtype);
    FDMS_REQUIRE(kv_dtype >= FDMS_F32 && kv_dtype <= FDMS_E4M3, FDMS_E_DTYPE,
                 "fdms_attn_decode: pool dtype %d not supported", kv_dtype);
    FDMS_REQUIRE((q_rope_positions == nullptr) == (q_rope_cos_sin == nullptr), FDMS_E_ARG,
                 "inline q RoPE requires both positions and cos_sin_cache");
    FDMS_REQUIRE(!q_rope_positions || head_dim % 2 == 0, FDMS_E_ARG, "inline q RoPE requires even head_dim, got %d", head_dim);
    FDMS_REQUIRE(q_rope_positions == nullptr || cos_sin_rows > 0, FDMS_E_ARG, "fdms_attn_decode: cos_sin_rows must be positive");
    return FDMS_OK;
}

static int32_t attn_decode_common(
    const void* q, int32_t q_dtype, int64_t q_stride_b, int64_t q_stride_h,
    const void* k_pool, const void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, const int32_t* live_counts, int64_t meta_stride_b,
    const int32_t* block_tables, int64_t bt_stride_b, int64_t bt_stride_h, int32_t bt_max_pages,
    const float* k_scale, const float* v_scale,
    void* out, int32_t out_dtype, int64_t out_stride_b, int64_t out_stride_h,
    int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
    const int64_t* q_rope_positions, const float* q_rope_cos_sin, int64_t cos_sin_stride, int64_t cos_sin_rows,
    void* workspace, int64_t workspace_bytes, int32_t flags, int32_t* dev_status, void* stream,
    const fdms::AppendArgs* app) {
    clear_error();
    {
        const int32_t rc = validate_attn_args(q, q_dtype, k_pool, v_pool, kv_dtype, base_offsets, live_counts, block_tables,
                                              bt_max_pages, out, out_dtype, batch, num_q_heads, num_kv_heads, head_dim,
                                              q_rope_positions, q_rope_cos_sin, cos_sin_rows);
        if (rc != FDMS_OK) return rc;
    }
    if (batch == 0) return FDMS_OK;
    const int group = num_q_heads / num_kv_heads;
    const int items = batch * num_kv_heads;

    AttnParams p;
    p.q = q; p.q_dtype = q_dtype; p.q_sb = q_stride_b; p.q_sh = q_stride_h;
    p.k_pool = (const uint8_t*)k_pool; p.v_pool = (const uint8_t*)v_pool; p.pool_rows = pool_rows;
    p.base = base_offsets; p.live = live_counts; p.meta_sb = meta_stride_b;
    p.bt = block_tables; p.bt_sb = bt_stride_b; p.bt_sh = bt_stride_h; p.bt_pages = bt_max_pages;
    p.k_scale = k_scale; p.v_scale = v_scale;
    p.out = out; p.out_dtype = out_dtype; p.out_sb = out_stride_b; p.out_sh = out_stride_h;
    p.batch = batch; p.hq = num_q_heads; p.hk = num_kv_heads; p.group = group;
    p.scale = scale;
    p.rope_pos = q_rope_positions; p.rope_cs = q_rope_cos_sin; p.rope_stride = cos_sin_stride; p.rope_rows = cos_sin_rows;
    p.counters = nullptr; p.part_ml = nullptr; p.part_o = nullptr;
    p.dev_status = dev_status;
    p.stages = 0; p.splits = 1; p.chunks = 1; p.overlap = (flags & FDMS_ATTN_OVERLAP_PREVIOUS) ? 1 : 0;
    p.append = 0;
    p.k_new = nullptr; p.kn_sb = p.kn_sh = 0; p.v_new = nullptr; p.vn_sb = p.vn_sh = 0;
    p.k_pool_w = nullptr; p.v_pool_w = nullptr; p.evict_out = nullptr; p.evict_sb = 0;
    p.rule = make_rule(1.0, 0.0);

    const bool fast = kv_dtype == FDMS_E4M3 && (head_dim == 64 || head_dim == 128) && group <= kMaxGroup &&
                      items <= 65535 && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) &&
                      env_int("FDMS_ATTN_FORCE_GENERIC", 0) == 0;
    if (app) {
        FDMS_REQUIRE(fast, FDMS_E_DTYPE,
                     "fdms_attn_decode_append needs FP8 e4m3 pools, head_dim 64 or 128 and group size <= %d", kMaxGroup);
        FDMS_REQUIRE(app->k_new && app->v_new && q_rope_positions && q_rope_cos_sin, FDMS_E_ARG,
                     "fdms_attn_decode_append: k, v, positions and cos_sin_cache are required");
        FDMS_REQUIRE(app->alpha_scale != 0.0 || !app->evict_out, FDMS_E_ARG, "alpha_scale must be non-zero");
        p.append = 1;
        p.k_new = app->k_new; p.kn_sb = app->kn_sb; p.kn_sh = app->kn_sh;
        p.v_new = app->v_new; p.vn_sb = app->vn_sb; p.vn_sh = app->vn_sh;
        p.k_pool_w = (uint8_t*)k_pool; p.v_pool_w = (uint8_t*)v_pool;
        p.evict_out = app->evict_out; p.evict_sb = app->evict_sb;
        p.rule = make_rule(app->alpha_scale, app->alpha_offset);
    }
    if (fast) {
        const DeviceInfo di = device_info();
        FDMS_REQUIRE(di.ok && di.sms > 0, FDMS_E_CUDA, "fdms_attn_decode: cannot query the device");
        // Loader: "direct" reads pages straight into registers; "staged" (FDMS_ATTN_LOADER=staged)
        // brings them into per-warp shared-memory rings with bulk copies.
        const char* loader = getenv("FDMS_ATTN_LOADER");
        const bool direct = !(loader && loader[0] == 's');
        const int ctas_per_sm = head_dim == 64 ? (direct ? 2 : 3) : 1;
        // CTAs per SM the grid is sized for: what the kernel's registers and shared memory allow (two for the
        // direct loader, three for the staged one at head_dim 64); FDMS_ATTN_WAVE=n sizes it for fewer.
        int wave = env_int("FDMS_ATTN_WAVE", 0);
        if (wave < 1) wave = ctas_per_sm;
        if (wave > ctas_per_sm) wave = ctas_per_sm;
        const int target = di.sms * wave;
        int ring = env_int("FDMS_ATTN_RING", 0);
        if (ring < 1) ring = 3;
        if (ring > kMaxRing) ring = kMaxRing;
        const int variant = (app ? 2 : 0) + (head_dim == 64 ? 0 : 1) + (direct ? 0 : 4);
        AttnKernel kern;
        if (direct) {
            if (app) kern = head_dim == 64 ? (AttnKernel)attn_decode_direct_kernel<64, 3, true> : (AttnKernel)attn_decode_direct_kernel<128, 2, true>;
            else kern = head_dim == 64 ? (AttnKernel)attn_decode_direct_kernel<64, 3, false> : (AttnKernel)attn_decode_direct_kernel<128, 2, false>;
        } else {
            if (app) kern = head_dim == 64 ? (AttnKernel)attn_decode_staged_kernel<64, true> : (AttnKernel)attn_decode_staged_kernel<128, true>;
            else kern = head_dim == 64 ? (AttnKernel)attn_decode_staged_kernel<64, false> : (AttnKernel)attn_decode_staged_kernel<128, false>;
        }
        const int threads = kConsumerThreads;
        auto smem_for = [&](int sp) {
            return direct ? direct_smem_bytes(head_dim, sp, group) : staged_smem_bytes(head_dim, ring, sp, group);
        };
        // splits: largest power of two that keeps the grid within the target number of CTAs
        int max_splits = env_int("FDMS_ATTN_MAX_SPLITS", 8);
        if (max_splits > kMaxSplits) max_splits = kMaxSplits;
        int splits = 1;
        while (splits * 2 <= max_splits && (int64_t)items * splits * 2 <= target) splits *= 2;
        const int forced = env_int("FDMS_ATTN_SPLITS", 0);
        if (forced >= 1 && forced <= kMaxSplits && (forced & (forced - 1)) == 0) splits = forced;
        while (splits > 1 && (smem_for(splits) > (size_t)di.smem_optin ||
                              !cluster_fits(kern, variant, threads, splits, smem_for(splits))))
            splits /= 2;
        // chunks: more clusters per span when even the largest cluster leaves most SMs idle
        int chunks = 1;
        if ((int64_t)items * splits * 2 <= target) {
            chunks = target / (items * splits);
            if (chunks > kMaxChunks) chunks = kMaxChunks;
            while (chunks > 1 && (int64_t)items * chunks > kMaxPartialSlots) --chunks;
        }
        const int forced_chunks = env_int("FDMS_ATTN_CHUNKS", 0);
        if (forced_chunks >= 1 && forced_chunks <= kMaxChunks && (int64_t)items * forced_chunks <= kMaxPartialSlots)
            chunks = forced_chunks;
        if (chunks > 1) {
            FDMS_REQUIRE(workspace != nullptr, FDMS_E_WORKSPACE, "fdms_attn_decode: workspace is required");
            FDMS_REQUIRE((uintptr_t)workspace % 256 == 0, FDMS_E_WORKSPACE, "fdms_attn_decode: workspace must be 256-byte aligned");
            const int64_t need = fdms_attn_decode_workspace_bytes(batch, num_kv_heads, head_dim);
            FDMS_REQUIRE(workspace_bytes >= need, FDMS_E_WORKSPACE,
                         "fdms_attn_decode: workspace of %lld bytes is smaller than the %lld required",
                         (long long)workspace_bytes, (long long)need);
            const int64_t counters = (((int64_t)items * 4 + 255) / 256) * 256;
            p.counters = (int32_t*)workspace;
            p.part_ml = (float*)((uint8_t*)workspace + counters);
            p.part_o = p.part_ml + (size_t)kMaxPartialSlots * kMaxGroup * 2;
        }
        const size_t smem = smem_for(splits);
        FDMS_REQUIRE(smem <= (size_t)di.smem_optin, FDMS_E_CAPACITY,
                     "fdms_attn_decode: %zu bytes of shared memory needed (limit %d)", smem, di.smem_optin);
        p.stages = ring; p.splits = splits; p.chunks = chunks;
        const cudaError_t e = launch_attn(kern, threads, p, items, smem, (cudaStream_t)stream, !direct);
        if (e != cudaSuccess) return fail(FDMS_E_CUDA, "attention kernel launch failed: %s", cudaGetErrorString(e));
        FDMS_CHECK_LAUNCH("attention kernel");
        return FDMS_OK;
    }

    GenParams gp;
    gp.a = p; gp.k_pool = k_pool; gp.v_pool = v_pool; gp.kv_dtype = kv_dtype; gp.dim = head_dim;
    attn_decode_generic_kernel<<<batch * num_q_heads, kGenWarps * 32, 0, (cudaStream_t)stream>>>(gp);
    FDMS_CHECK_LAUNCH("attn_decode_generic_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_attn_decode(
    const void* q, int32_t q_dtype, int64_t q_stride_b, int64_t q_stride_h,
    const void* k_pool, const void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, const int32_t* live_counts, int64_t meta_stride_b,
    const int32_t* block_tables, int64_t bt_stride_b, int64_t bt_stride_h, int32_t bt_max_pages,
    const float* k_scale, const float* v_scale,
    void* out, int32_t out_dtype, int64_t out_stride_b, int64_t out_stride_h,
    int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
    const int64_t* q_rope_positions, const float* q_rope_cos_sin, int64_t cos_sin_stride, int64_t cos_sin_rows,
    void* workspace, int64_t workspace_bytes, int32_t flags, int32_t* dev_status, void* stream) {
    return attn_decode_common(q, q_dtype, q_stride_b, q_stride_h, k_pool, v_pool, kv_dtype, pool_rows, base_offsets,
                              live_counts, meta_stride_b, block_tables, bt_stride_b, bt_stride_h, bt_max_pages, k_scale,
                              v_scale, out, out_dtype, out_stride_b, out_stride_h, batch, num_q_heads, num_kv_heads,
                              head_dim, scale, q_rope_positions, q_rope_cos_sin, cos_sin_stride, cos_sin_rows, workspace,
                              workspace_bytes, flags, dev_status, stream, nullptr);
}

extern "C" int32_t fdms_attn_decode_append(
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
    void* workspace, int64_t workspace_bytes, int32_t flags, int32_t* dev_status, void* stream) {
    fdms::AppendArgs app;
    app.k_new = k; app.kn_sb = k_stride_b; app.kn_sh = k_stride_h;
    app.v_new = v; app.vn_sb = v_stride_b; app.vn_sh = v_stride_h;
    app.evict_out = evict_out; app.evict_sb = evict_stride_b;
    app.alpha_scale = alpha_scale; app.alpha_offset = alpha_offset;
    return attn_decode_common(q, act_dtype, q_stride_b, q_stride_h, k_pool, v_pool, kv_dtype, pool_rows, base_offsets,
                              live_counts, meta_stride_b, block_tables, bt_stride_b, bt_stride_h, bt_max_pages, k_scale,
                              v_scale, out, out_dtype, out_stride_b, out_stride_h, batch, num_q_heads, num_kv_heads,
                              head_dim, scale, positions, cos_sin, cos_sin_stride, cos_sin_rows, workspace, workspace_bytes, flags,
                              dev_status, stream, &app);
}

// ------------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// fdms_attn_decode needs a caller-provided split-K workspace.  Some hosts have nowhere to get one
// from: a serving process that hands its whole device-memory budget to the KV pool at start-up and
// forbids later cudaMalloc calls (they synchronise the device and can fail late), or a plugin loaded
// through a foreign-function interface into a runtime written in another language, which has
// pointers to the tensors it was given but no device allocator of its own to call.  For them the
// workspace lives in this library's image: a fixed array in device memory that every GPU loading the
// library holds until the process exits.
//
// Size and limits: counters for 4096 spans + 1024 partial slots of 8 heads x (128 + 2) floats
// = 4,276,224 bytes.  Hence batch * kv_heads <= 4096 and head_dim <= 128 (larger sizes are rejected;
// use fdms_attn_decode with your own workspace).
//
// The array's name is a host-side stand-in in host code, not a device address; the real address is
// resolved once per device with cudaGetSymbolAddress while that device is current, and that pointer
// is what the kernel receives.  The FIRST call on each device does this resolution, so make that
// first call outside any stream capture.
//
// All calls share the one array and it keeps whatever the previous call left in it.  The span
// counters at its start must be zero when a launch begins, so every call clears them on its stream
// first.  Two calls whose kernels overlap on the GPU (different streams, or the same stream with
// launch overlap) race on the array and give wrong results: serialise them.
// ------------------------------------------------------------------------------------------------
namespace fdms {
constexpr int kStaticMaxSpans = 4096;
constexpr int kStaticMaxHeadDim = 128;
constexpr size_t kStaticCounterBytes = (size_t)kStaticMaxSpans * sizeof(int32_t);
constexpr size_t kStaticScratchBytes = kStaticCounterBytes + (size_t)kMaxPartialSlots * kMaxGroup * 2 * sizeof(float) +
                                       (size_t)kMaxPartialSlots * kMaxGroup * kStaticMaxHeadDim * sizeof(float);
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

// Device address of the scratch array on the current device (nullptr + error code on failure).
// The per-device cache is written with atomic stores: two host threads that race on the first call
// both resolve the same address, and neither can read a half-written pointer.
static void* static_scratch_address(cudaError_t* err) {
    static std::atomic<void*> cached[64];
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
    void* ptr = cached[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        *err = cudaGetSymbolAddress(&ptr, g_attn_static_scratch);
        if (*err != cudaSuccess) return nullptr;
        cached[dev].store(ptr, std::memory_order_release);
    }
    return ptr;
}
}  // namespace fdms

extern "C" int32_t fdms_attn_decode_noalloc(
    const void* q, int32_t q_dtype, int64_t q_stride_b, int64_t q_stride_h,
    const void* k_pool, const void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, const int32_t* live_counts, int64_t meta_stride_b,
    const int32_t* block_tables, int64_t bt_stride_b, int64_t bt_stride_h, int32_t bt_max_pages,
    const float* k_scale, const float* v_scale,
    void* out, int32_t out_dtype, int64_t out_stride_b, int64_t out_stride_h,
    int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
    const int64_t* q_rope_positions, const float* q_rope_cos_sin, int64_t cos_sin_stride, int64_t cos_sin_rows,
    int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(batch >= 0 && num_kv_heads > 0 && head_dim > 0, FDMS_E_ARG, "fdms_attn_decode_noalloc: bad sizes");
    FDMS_REQUIRE((int64_t)batch * num_kv_heads <= kStaticMaxSpans, FDMS_E_CAPACITY,
                 "fdms_attn_decode_noalloc: batch*kv_heads=%lld exceeds the built-in scratch limit of %d spans; "
                 "use fdms_attn_decode with a caller workspace",
                 (long long)batch * num_kv_heads, kStaticMaxSpans);
    FDMS_REQUIRE(head_dim <= kStaticMaxHeadDim, FDMS_E_CAPACITY,
                 "fdms_attn_decode_noalloc: head_dim=%d exceeds the built-in scratch limit of %d; "
                 "use fdms_attn_decode with a caller workspace", head_dim, kStaticMaxHeadDim);
    {
        // every argument check of the ordinary entry point runs before anything is enqueued
        const int32_t rc = validate_attn_args(q, q_dtype, k_pool, v_pool, kv_dtype, base_offsets, live_counts, block_tables,
                                              bt_max_pages, out, out_dtype, batch, num_q_heads, num_kv_heads, head_dim,
                                              q_rope_positions, q_rope_cos_sin, cos_sin_rows);
        if (rc != FDMS_OK) return rc;
    }
    if (batch == 0) return FDMS_OK;
    cudaError_t e = cudaSuccess;
    void* scratch = static_scratch_address(&e);
    if (scratch == nullptr || e != cudaSuccess)
        return fail(FDMS_E_CUDA, "fdms_attn_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    // the span counters must start at zero; the rest of the array is fully rewritten before it is read
    e = cudaMemsetAsync(scratch, 0, (size_t)batch * num_kv_heads * sizeof(int32_t), (cudaStream_t)stream);
    if (e != cudaSuccess)
        return fail(FDMS_E_CUDA, "fdms_attn_decode_noalloc: clearing the counters failed: %s", cudaGetErrorString(e));
    return fdms_attn_decode(q, q_dtype, q_stride_b, q_stride_h, k_pool, v_pool, kv_dtype, pool_rows, base_offsets,
                            live_counts, meta_stride_b, block_tables, bt_stride_b, bt_stride_h, bt_max_pages, k_scale,
                            v_scale, out, out_dtype, out_stride_b, out_stride_h, batch, num_q_heads, num_kv_heads,
                            head_dim, scale, q_rope_positions, q_rope_cos_sin, cos_sin_stride, cos_sin_rows, scratch,
                            (int64_t)kStaticScratchBytes, 0, dev_status, stream);
}

#ifdef FDMS_ATTN_PROBE
// Probe builds only: copies the phase table of the most recent fast-kernel launch, [phases][ctas] nanoseconds
// of the global timer, to `host` (phases * ctas values, ctas <= 4096).  Synchronises the device.
extern "C" int32_t fdms_attn_probe_read(unsigned long long* host, int32_t phases, int32_t ctas) {
    clear_error();
    FDMS_REQUIRE(host && phases > 0 && phases <= kProbePhases && ctas > 0 && ctas <= kProbeMaxCtas, FDMS_E_ARG,
                 "fdms_attn_probe_read: bad arguments");
    FDMS_CUDA_OK(cudaDeviceSynchronize());
    for (int ph = 0; ph < phases; ++ph)
        FDMS_CUDA_OK(cudaMemcpyFromSymbol(host + (size_t)ph * ctas, g_attn_probe, (size_t)ctas * sizeof(unsigned long long),
                                          (size_t)ph * kProbeMaxCtas * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return FDMS_OK;
}
#endif

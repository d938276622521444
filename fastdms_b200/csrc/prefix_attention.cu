// Prefill-tail attention: the queries of a prefill chunk against the compact prefix of their
// sequence, i.e. the rows that earlier chunks of the same prompt left in the compact pool (FP8 or
// wider, contiguous spans or 16-row pages), merged with the chunk's own dense causal attention.
//
// The reference prefills a prompt in one dense pass (fastdms/layers/attention.py:85-92,
// fastdms/engine/model_runner.py:655-657) and has no counterpart of this kernel.  Semantics here: a
// query at position p of chunk [s, e) sees (1) every row its (sequence, KV head) span holds when the
// chunk starts -- all of them older than s -- and (2) the chunk's tokens at positions <= p.  Part
// (2) is an ordinary causal attention over the chunk's own K/V and is computed by the caller (it
// hands in the normalised result and its log-sum-exp); this kernel computes part (1) and folds the
// two with the usual log-sum-exp merge.
//
// Work split: a CTA owns up to 8 warps = (q heads of one KV group) x (16-token query tiles); every
// warp keeps one 16 x head_dim output tile in registers and walks the whole span.  The span is
// staged 64 rows at a time: all threads convert the tile's K and V rows to f16 in shared memory
// (exact for e4m3), the warps read them back as MMA fragments with ldmatrix (V transposed), so
// the conversion is paid once per (group, 16..128 queries) instead of once per query row.
// mma.sync m16n8k16, f32 accumulation, online softmax in the log2 domain.
#include "common.cuh"

namespace fdms {

constexpr int kPfxTile = 64;            // span rows per staged tile
constexpr int kPfxMaxWarps = 8;
constexpr float kPfxLog2eF = 1.4426950408889634f;
constexpr float kPfxLn2F = 0.6931471805599453f;

struct PrefixParams {
    const void* q; int act_dtype; int64_t q_st, q_sh;
    const int32_t* cu; int max_q;
    const void* k_pool; const void* v_pool; int kv_dtype; int64_t pool_rows;
    const int32_t* base; const int32_t* live; int64_t meta_ss;
    const int32_t* bt; int64_t bt_ss, bt_sh; int bt_max_pages;
    const int32_t* seq_slots;
    const float* k_scale; const float* v_scale;
    void* out; int64_t o_st, o_sh;
    const float* dense_lse; int64_t lse_sh, lse_st;
    float* lse_out; int64_t lo_sh, lo_st;
    int hq, hk, group, tiles_per_cta;
    float scale;
    int32_t* dev_status;
};

__device__ __forceinline__ void pfx_e4m3x4_to_f16x2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
    asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
        : "=r"(lo), "=r"(hi) : "r"(w));
}
__device__ __forceinline__ uint32_t pfx_pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *(uint32_t*)&h;
}
__device__ __forceinline__ float pfx_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void pfx_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pfx_ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void pfx_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// Two consecutive elements of a 16-bit / 32-bit activation row as packed f16.
__device__ __forceinline__ uint32_t pfx_load2_f16(const void* p, int64_t i, int dt) {
    if (dt == FDMS_F16) return *(const uint32_t*)((const uint16_t*)p + i);
    return pfx_pack(load_as_float(p, i, dt), load_as_float(p, i + 1, dt));
}

// Stages rows [i0, i0 + 64) of the span as f16 into Ks / Vs (row stride D + 8 halves); rows at or
// beyond `live` become zeros.  FP8 pools take 16 bytes per thread and step, other pool types one
// element at a time.
template <int D>
__device__ __forceinline__ void pfx_stage_tile(const PrefixParams& p, int base, const int32_t* bt, int live, int i0,
                                               __half* Ks, __half* Vs, int tid, int nthreads) {
    constexpr int LD = D + 8;
    if (p.kv_dtype == FDMS_E4M3) {
        constexpr int VPR = D / 16;                       // 16-byte vectors per row
        for (int x = tid; x < kPfxTile * VPR; x += nthreads) {
            const int r = x / VPR, c = x - r * VPR;
            uint4 kb = make_uint4(0u, 0u, 0u, 0u), vb = kb;
            if (i0 + r < live) {
                const int64_t row = span_row(base, bt, i0 + r);
                if (row >= 0 && row < p.pool_rows) {
                    kb = *(const uint4*)((const uint8_t*)p.k_pool + row * D + 16 * c);
                    vb = *(const uint4*)((const uint8_t*)p.v_pool + row * D + 16 * c);
                } else if (p.dev_status) {
                    atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
                }
            }
            uint4 lo, hi;
            pfx_e4m3x4_to_f16x2x2(kb.x, lo.x, lo.y); pfx_e4m3x4_to_f16x2x2(kb.y, lo.z, lo.w);
            pfx_e4m3x4_to_f16x2x2(kb.z, hi.x, hi.y); pfx_e4m3x4_to_f16x2x2(kb.w, hi.z, hi.w);
            *(uint4*)(Ks + r * LD + 16 * c) = lo;
            *(uint4*)(Ks + r * LD + 16 * c + 8) = hi;
            pfx_e4m3x4_to_f16x2x2(vb.x, lo.x, lo.y); pfx_e4m3x4_to_f16x2x2(vb.y, lo.z, lo.w);
            pfx_e4m3x4_to_f16x2x2(vb.z, hi.x, hi.y); pfx_e4m3x4_to_f16x2x2(vb.w, hi.z, hi.w);
            *(uint4*)(Vs + r * LD + 16 * c) = lo;
            *(uint4*)(Vs + r * LD + 16 * c + 8) = hi;
        }
    } else {
        for (int x = tid; x < kPfxTile * D; x += nthreads) {
            const int r = x / D, d = x - r * D;
            float kx = 0.0f, vx = 0.0f;
            if (i0 + r < live) {
                const int64_t row = span_row(base, bt, i0 + r);
                if (row >= 0 && row < p.pool_rows) {
                    kx = load_as_float(p.k_pool, row * D + d, p.kv_dtype);
                    vx = load_as_float(p.v_pool, row * D + d, p.kv_dtype);
                } else if (p.dev_status) {
                    atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
                }
            }
            Ks[r * LD + d] = __float2half_rn(kx);
            Vs[r * LD + d] = __float2half_rn(vx);
        }
    }
}

// FP8 pools, software-pipelined: the bytes of the NEXT tile travel with asynchronous 16-byte copies into a raw
// staging area in shared memory (no registers held across the math) while the warps compute on the current tile.
// A thread converts exactly the vectors it copied itself, so waiting for its own copy group is enough.
__device__ __forceinline__ void pfx_cp_async16(void* smem_dst, const void* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}

template <int D>
__device__ __forceinline__ void pfx_fetch_tile(const PrefixParams& p, int base, const int32_t* bt, int live, int i0,
                                               uint8_t* Kraw, uint8_t* Vraw, int tid, int nthreads) {
    constexpr int VPR = D / 16;
    for (int x = tid; x < kPfxTile * VPR; x += nthreads) {
        const int r = x / VPR, c = x - r * VPR;
        bool have = false;
        if (i0 + r < live) {
            const int64_t row = span_row(base, bt, i0 + r);
            if (row >= 0 && row < p.pool_rows) {
                pfx_cp_async16(Kraw + 16 * x, (const uint8_t*)p.k_pool + row * D + 16 * c);
                pfx_cp_async16(Vraw + 16 * x, (const uint8_t*)p.v_pool + row * D + 16 * c);
                have = true;
            } else if (p.dev_status) {
                atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
            }
        }
        if (!have) {
            *(uint4*)(Kraw + 16 * x) = make_uint4(0u, 0u, 0u, 0u);
            *(uint4*)(Vraw + 16 * x) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int D>
__device__ __forceinline__ void pfx_commit_tile(const uint8_t* Kraw, const uint8_t* Vraw, __half* Ks, __half* Vs, int tid,
                                                int nthreads) {
    constexpr int LD = D + 8, VPR = D / 16;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    for (int x = tid; x < kPfxTile * VPR; x += nthreads) {
        const int r = x / VPR, c = x - r * VPR;
        const uint4 kb = *(const uint4*)(Kraw + 16 * x), vb = *(const uint4*)(Vraw + 16 * x);
        uint4 lo, hi;
        pfx_e4m3x4_to_f16x2x2(kb.x, lo.x, lo.y); pfx_e4m3x4_to_f16x2x2(kb.y, lo.z, lo.w);
        pfx_e4m3x4_to_f16x2x2(kb.z, hi.x, hi.y); pfx_e4m3x4_to_f16x2x2(kb.w, hi.z, hi.w);
        *(uint4*)(Ks + r * LD + 16 * c) = lo;
        *(uint4*)(Ks + r * LD + 16 * c + 8) = hi;
        pfx_e4m3x4_to_f16x2x2(vb.x, lo.x, lo.y); pfx_e4m3x4_to_f16x2x2(vb.y, lo.z, lo.w);
        pfx_e4m3x4_to_f16x2x2(vb.z, hi.x, hi.y); pfx_e4m3x4_to_f16x2x2(vb.w, hi.z, hi.w);
        *(uint4*)(Vs + r * LD + 16 * c) = lo;
        *(uint4*)(Vs + r * LD + 16 * c + 8) = hi;
    }
}

// The same look-ahead held in registers (head_dim 128, where the raw staging area would not fit the static
// shared-memory limit and the kernel has registers to spare): the bytes of the NEXT tile are fetched into registers (one 16-byte K
// and V vector per thread and pass) while the warps compute on the tile in shared memory.
template <int D>
struct PfxFetch {
    static constexpr int kPasses = (kPfxTile * (D / 16) + kPfxMaxWarps * 32 - 1) / (kPfxMaxWarps * 32);
    uint4 k[kPasses], v[kPasses];
};

template <int D>
__device__ __forceinline__ void pfx_fetch_tile_regs(const PrefixParams& p, int base, const int32_t* bt, int live, int i0,
                                               PfxFetch<D>& f, int tid, int nthreads) {
    constexpr int VPR = D / 16;
#pragma unroll
    for (int j = 0; j < PfxFetch<D>::kPasses; ++j) {
        const int x = tid + j * nthreads;
        f.k[j] = make_uint4(0u, 0u, 0u, 0u);
        f.v[j] = f.k[j];
        if (x >= kPfxTile * VPR) continue;
        const int r = x / VPR, c = x - r * VPR;
        if (i0 + r >= live) continue;
        const int64_t row = span_row(base, bt, i0 + r);
        if (row >= 0 && row < p.pool_rows) {
            f.k[j] = *(const uint4*)((const uint8_t*)p.k_pool + row * D + 16 * c);
            f.v[j] = *(const uint4*)((const uint8_t*)p.v_pool + row * D + 16 * c);
        } else if (p.dev_status) {
            atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
        }
    }
}

template <int D>
__device__ __forceinline__ void pfx_commit_tile_regs(const PfxFetch<D>& f, __half* Ks, __half* Vs, int tid, int nthreads) {
    constexpr int LD = D + 8, VPR = D / 16;
#pragma unroll
    for (int j = 0; j < PfxFetch<D>::kPasses; ++j) {
        const int x = tid + j * nthreads;
        if (x >= kPfxTile * VPR) continue;
        const int r = x / VPR, c = x - r * VPR;
        uint4 lo, hi;
        pfx_e4m3x4_to_f16x2x2(f.k[j].x, lo.x, lo.y); pfx_e4m3x4_to_f16x2x2(f.k[j].y, lo.z, lo.w);
        pfx_e4m3x4_to_f16x2x2(f.k[j].z, hi.x, hi.y); pfx_e4m3x4_to_f16x2x2(f.k[j].w, hi.z, hi.w);
        *(uint4*)(Ks + r * LD + 16 * c) = lo;
        *(uint4*)(Ks + r * LD + 16 * c + 8) = hi;
        pfx_e4m3x4_to_f16x2x2(f.v[j].x, lo.x, lo.y); pfx_e4m3x4_to_f16x2x2(f.v[j].y, lo.z, lo.w);
        pfx_e4m3x4_to_f16x2x2(f.v[j].z, hi.x, hi.y); pfx_e4m3x4_to_f16x2x2(f.v[j].w, hi.z, hi.w);
        *(uint4*)(Vs + r * LD + 16 * c) = lo;
        *(uint4*)(Vs + r * LD + 16 * c + 8) = hi;
    }
}

template <int D>
__global__ void __launch_bounds__(kPfxMaxWarps * 32, D == 64 ? 2 : 1) prefix_attention_kernel(PrefixParams p) {
    constexpr int LD = D + 8, KS = D / 16, NT = D / 8;
    __shared__ __align__(16) __half Ks[kPfxTile * LD];
    __shared__ __align__(16) __half Vs[kPfxTile * LD];
    constexpr bool kRawStage = D == 64;                         // next tile through shared memory (else registers)
    __shared__ __align__(16) uint8_t Kraw[kRawStage ? kPfxTile * D : 16];        // the next tile's FP8 bytes
    __shared__ __align__(16) uint8_t Vraw[kRawStage ? kPfxTile * D : 16];
    const int s = blockIdx.z, h = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int nthreads = blockDim.x;
    const int srow = p.seq_slots ? p.seq_slots[s] : s;
    const int live = p.live[(int64_t)srow * p.meta_ss + h];
    const int64_t tok0 = p.cu[s];
    const int T = p.cu[s + 1] - p.cu[s];
    const int q0 = blockIdx.x * 16 * p.tiles_per_cta;
    if (live <= 0 || q0 >= T) return;                    // uniform over the CTA: no prefix, or no queries here
    const int base = p.base ? p.base[(int64_t)srow * p.meta_ss + h] : 0;
    const int32_t* bt = p.bt ? p.bt + (int64_t)srow * p.bt_ss + (int64_t)h * p.bt_sh : nullptr;
    if (bt != nullptr && (live + 15) / 16 > p.bt_max_pages) {
        if (tid == 0 && p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
        return;
    }
    const int hq = h * p.group + warp % p.group;
    const int tq = q0 + (warp / p.group) * 16;            // first query token of this warp
    const bool active = warp < p.group * p.tiles_per_cta && tq < T;   // spare warps only help staging
    const int r0 = tq + g, r1 = tq + g + 8;               // the lane's two query rows
    const bool ok0 = active && r0 < T, ok1 = active && r1 < T;

    uint32_t qa[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const int64_t c = (int64_t)hq * p.q_sh + 16 * ks + 2 * t;
        qa[ks][0] = ok0 ? pfx_load2_f16(p.q, (tok0 + r0) * p.q_st + c, p.act_dtype) : 0u;
        qa[ks][1] = ok1 ? pfx_load2_f16(p.q, (tok0 + r1) * p.q_st + c, p.act_dtype) : 0u;
        qa[ks][2] = ok0 ? pfx_load2_f16(p.q, (tok0 + r0) * p.q_st + c + 8, p.act_dtype) : 0u;
        qa[ks][3] = ok1 ? pfx_load2_f16(p.q, (tok0 + r1) * p.q_st + c + 8, p.act_dtype) : 0u;
    }
    const float sl2 = p.scale * (p.k_scale ? p.k_scale[h] : 1.0f) * kPfxLog2eF;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    const int mat = lane >> 3, mrow = lane & 7;           // ldmatrix: this lane addresses row mrow of matrix mat

    const bool fp8 = p.kv_dtype == FDMS_E4M3;
    PfxFetch<D> nxt;
    if (fp8) {
        if constexpr (kRawStage) pfx_fetch_tile<D>(p, base, bt, live, 0, Kraw, Vraw, tid, nthreads);
        else pfx_fetch_tile_regs<D>(p, base, bt, live, 0, nxt, tid, nthreads);
    }
    for (int i0 = 0; i0 < live; i0 += kPfxTile) {
        __syncthreads();                                  // the previous tile has been consumed
        if (fp8) {
            if constexpr (kRawStage) pfx_commit_tile<D>(Kraw, Vraw, Ks, Vs, tid, nthreads);
            else pfx_commit_tile_regs<D>(nxt, Ks, Vs, tid, nthreads);
        } else {
            pfx_stage_tile<D>(p, base, bt, live, i0, Ks, Vs, tid, nthreads);
        }
        __syncthreads();
        if (fp8 && i0 + kPfxTile < live) {
            if constexpr (kRawStage) pfx_fetch_tile<D>(p, base, bt, live, i0 + kPfxTile, Kraw, Vraw, tid, nthreads);
            else pfx_fetch_tile_regs<D>(p, base, bt, live, i0 + kPfxTile, nxt, tid, nthreads);
        }
        if (!active) continue;
        // ---- S = Q K^T for 64 span rows ----
        float sc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                uint32_t b[4];
                pfx_ldmatrix_x4(b, Ks + (jp * 16 + (mat >> 1) * 8 + mrow) * LD + ks * 16 + (mat & 1) * 8);
                pfx_mma(sc[2 * jp], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[0], b[1]);
                pfx_mma(sc[2 * jp + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[2], b[3]);
            }
        }
        // ---- online softmax over the tile (rows g and g + 8 of the warp's 16 queries) ----
        const int valid = live - i0;                      // span rows of this tile that exist
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = 8 * j + 2 * t + (c & 1);
                sc[j][c] = col < valid ? sc[j][c] * sl2 : -INFINITY;
                mx[c >> 1] = fmaxf(mx[c >> 1], sc[j][c]);
            }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);   // finite: column 0 of every tile exists
            alpha[r] = pfx_ex2(m_run[r] - m_new);
            m_run[r] = m_new;
            l_run[r] *= alpha[r];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                sc[j][c] = pfx_ex2(sc[j][c] - m_run[c >> 1]);
                l_run[c >> 1] += sc[j][c];
            }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) { o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1]; }
        // ---- O += P V ----
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const uint32_t a0 = pfx_pack(sc[2 * kk][0], sc[2 * kk][1]), a1 = pfx_pack(sc[2 * kk][2], sc[2 * kk][3]);
            const uint32_t a2 = pfx_pack(sc[2 * kk + 1][0], sc[2 * kk + 1][1]), a3 = pfx_pack(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < NT / 2; ++dp) {
                uint32_t b[4];
                pfx_ldmatrix_x4_trans(b, Vs + (kk * 16 + (mat & 1) * 8 + mrow) * LD + dp * 16 + (mat >> 1) * 8);
                pfx_mma(o[2 * dp], a0, a1, a2, a3, b[0], b[1]);
                pfx_mma(o[2 * dp + 1], a0, a1, a2, a3, b[2], b[3]);
            }
        }
    }
    if (!active) return;

    // ---- normalise, merge with the chunk's own causal attention, write ----
    const float vs = p.v_scale ? p.v_scale[h] : 1.0f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = l_run[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = r == 0 ? r0 : r1;
        if (!(r == 0 ? ok0 : ok1)) continue;
        const float lse_p = (m_run[r] + log2f(l)) * kPfxLn2F;          // natural-log LSE of the prefix part
        float wp = vs / l, wd = 0.0f, lse = lse_p;
        if (p.dense_lse) {
            const float lse_d = p.dense_lse[(int64_t)hq * p.lse_sh + (tok0 + row) * p.lse_st];
            const float mm = fmaxf(lse_p, lse_d);
            const float ep = __expf(lse_p - mm), ed = __expf(lse_d - mm);
            const float inv = 1.0f / (ep + ed);
            wp *= ep * inv;
            wd = ed * inv;
            lse = mm + __logf(ep + ed);
        }
        if (p.lse_out && t == 0) p.lse_out[(int64_t)hq * p.lo_sh + (tok0 + row) * p.lo_st] = lse;
        const int64_t orow = (tok0 + row) * p.o_st + (int64_t)hq * p.o_sh;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int64_t at = orow + 8 * j + 2 * t;
            float y0 = o[j][2 * r] * wp, y1 = o[j][2 * r + 1] * wp;
            if (p.dense_lse) {
                y0 += wd * load_as_float(p.out, at, p.act_dtype);
                y1 += wd * load_as_float(p.out, at + 1, p.act_dtype);
            }
            store_from_float(p.out, at, p.act_dtype, y0);
            store_from_float(p.out, at + 1, p.act_dtype, y1);
        }
    }
}

}  // namespace fdms

using namespace fdms;

extern "C" int32_t fdms_prefix_attention(
    const void* q, int32_t act_dtype, int64_t q_stride_t, int64_t q_stride_h, const int32_t* cu_seqlens_q,
    int32_t max_q_len, const void* k_pool, const void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* base_offsets, const int32_t* live_counts, int64_t meta_stride_s,
    const int32_t* block_tables, int64_t bt_stride_s, int64_t bt_stride_h, int32_t bt_max_pages,
    const int32_t* seq_slots, const float* k_scale, const float* v_scale,
    void* out, int64_t out_stride_t, int64_t out_stride_h,
    const float* dense_lse, int64_t lse_stride_h, int64_t lse_stride_t,
    float* lse_out, int64_t lse_out_stride_h, int64_t lse_out_stride_t,
    int32_t num_seqs, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
    int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(q && cu_seqlens_q && k_pool && v_pool && live_counts && out, FDMS_E_ARG, "fdms_prefix_attention: null pointer");
    FDMS_REQUIRE(base_offsets || block_tables, FDMS_E_ARG, "fdms_prefix_attention: base_offsets or block_tables required");
    FDMS_REQUIRE(act_dtype == FDMS_F32 || act_dtype == FDMS_BF16 || act_dtype == FDMS_F16, FDMS_E_DTYPE,
                 "fdms_prefix_attention: activation dtype %d not supported", act_dtype);
    FDMS_REQUIRE(kv_dtype >= FDMS_F32 && kv_dtype <= FDMS_E4M3, FDMS_E_DTYPE, "fdms_prefix_attention: pool dtype %d not supported", kv_dtype);
    FDMS_REQUIRE(head_dim == 64 || head_dim == 128, FDMS_E_ARG, "fdms_prefix_attention: head_dim must be 64 or 128, got %d", head_dim);
    FDMS_REQUIRE(num_seqs >= 0 && num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0 && max_q_len >= 0,
                 FDMS_E_ARG, "fdms_prefix_attention: bad sizes");
    const int group = num_q_heads / num_kv_heads;
    FDMS_REQUIRE(group <= kPfxMaxWarps, FDMS_E_CAPACITY, "fdms_prefix_attention: at most %d q heads per KV head, got %d", kPfxMaxWarps, group);
    FDMS_REQUIRE(num_seqs <= 65535 && num_kv_heads <= 65535, FDMS_E_CAPACITY, "fdms_prefix_attention: grid too large");
    const int esz = act_dtype == FDMS_F32 ? 4 : 2;
    FDMS_REQUIRE(((uintptr_t)q % 4) == 0 && (q_stride_t * esz) % 4 == 0 && (q_stride_h * esz) % 4 == 0 &&
                     ((uintptr_t)out % 4) == 0 && (out_stride_t * esz) % 4 == 0 && (out_stride_h * esz) % 4 == 0,
                 FDMS_E_ARG, "fdms_prefix_attention: q / out rows must be 4-byte aligned");
    if (kv_dtype == FDMS_E4M3)
        FDMS_REQUIRE(((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0, FDMS_E_ARG,
                     "fdms_prefix_attention: FP8 pools must be 16-byte aligned");
    if (num_seqs == 0 || max_q_len == 0) return FDMS_OK;
    PrefixParams p;
    p.q = q; p.act_dtype = act_dtype; p.q_st = q_stride_t; p.q_sh = q_stride_h;
    p.cu = cu_seqlens_q; p.max_q = max_q_len;
    p.k_pool = k_pool; p.v_pool = v_pool; p.kv_dtype = kv_dtype; p.pool_rows = pool_rows;
    p.base = base_offsets; p.live = live_counts; p.meta_ss = meta_stride_s;
    p.bt = block_tables; p.bt_ss = bt_stride_s; p.bt_sh = bt_stride_h; p.bt_max_pages = bt_max_pages;
    p.seq_slots = seq_slots; p.k_scale = k_scale; p.v_scale = v_scale;
    p.out = out; p.o_st = out_stride_t; p.o_sh = out_stride_h;
    p.dense_lse = dense_lse; p.lse_sh = lse_stride_h; p.lse_st = lse_stride_t;
    p.lse_out = lse_out; p.lo_sh = lse_out_stride_h; p.lo_st = lse_out_stride_t;
    p.hq = num_q_heads; p.hk = num_kv_heads; p.group = group;
    p.tiles_per_cta = kPfxMaxWarps / group;
    p.scale = scale; p.dev_status = dev_status;
    const int q_per_cta = 16 * p.tiles_per_cta;
    dim3 grid((max_q_len + q_per_cta - 1) / q_per_cta, num_kv_heads, num_seqs);
    const int threads = kPfxMaxWarps * 32;              // always 8 warps: the staging passes are sized for them
    if (head_dim == 64) prefix_attention_kernel<64><<<grid, threads, 0, (cudaStream_t)stream>>>(p);
    else prefix_attention_kernel<128><<<grid, threads, 0, (cudaStream_t)stream>>>(p);
    FDMS_CHECK_LAUNCH("prefix_attention_kernel");
    return FDMS_OK;
}

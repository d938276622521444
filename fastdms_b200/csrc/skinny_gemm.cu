// y[M, N] = x[M, K] * W[N, K]^T (+ bias) for decode-sized M (<= 8 rows): the linear layers either side of
// the attention launch in a decoder block and the LM head, which at c = 8 are pure weight streaming
// (the reference calls cuBLAS through F.linear, fastdms/layers/linear.py:635-662, 1044-1048).
//
// One CTA = 8 warps on NT tiles of 16 output columns; the warps split K (K / 8 each, walked 256 at a
// time) so that even the narrowest projection fills the chip, and their 16 x 8 partial tiles are
// summed through shared memory.  Per step a lane streams 2 x 8 vectors of 16 bytes of W (8 KB per
// warp in flight) and holds the matching 16-byte vectors of x in registers across the CTA's tiles.
// Tensor cores: mma.sync.m16n8k16 with the weight rows on M and the <= 8 activation rows on N; the
// k-index of the MMA is a fixed permutation of the memory order (a lane's four MMA k-pairs are the
// four element pairs of its 16-byte vector, for A and B alike), so no shuffle or shared-memory
// staging is needed.  f32 accumulation, one rounding to the activation dtype at the end.
#include <stdlib.h>

#include "common.cuh"

namespace fdms {

constexpr int kSgWarps = 8;
constexpr int kSgStep = 256;          // k elements per warp and step (8 vectors of 32)

template <bool BF16>
__device__ __forceinline__ void sg_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight consecutive 16-bit elements <-> float.
template <bool BF16>
__device__ __forceinline__ void sg_unpack8(const uint4& v, float (&f)[8]) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (BF16) {
            f[2 * i] = __uint_as_float(u[i] << 16);
            f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        } else {
            const __half2 h = *(const __half2*)&u[i];
            f[2 * i] = __low2float(h);
            f[2 * i + 1] = __high2float(h);
        }
    }
}
template <bool BF16>
__device__ __forceinline__ uint4 sg_pack8(const float (&f)[8]) {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (BF16) { const __nv_bfloat162 b = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]); u[i] = *(const uint32_t*)&b; }
        else { const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]); u[i] = *(const uint32_t*)&h; }
    }
    return make_uint4(u[0], u[1], u[2], u[3]);
}

// Arguments of the fused RMSNorm (+ residual add) in front of the linear layer (NORM = true):
//   xf = float(x) (+ float(residual));  residual_out = round(xf) (written by CTA 0);
//   the GEMM's input row is round(round(xf * rsqrt(mean(xf^2) + eps)) * norm_weight),
// the arithmetic of rmsnorm_kernel; every CTA recomputes the 8 row statistics (the rows are small).
struct SgNorm {
    const uint16_t* residual; int64_t res_stride;
    const uint16_t* norm_weight; float eps;
    uint16_t* residual_out; int64_t res_out_stride;
};

// GATED = true (NT = 2) is the gate_up projection of a gated MLP with its activation: the CTA's two tiles are the
// gate columns n0 .. n0 + 15 and the up columns N/2 + n0 .. of W[N, K], and it writes
//   y[m, n0 + j] = round(round(silu(gate)) * up),  gate and up rounded to the activation dtype first,
// the arithmetic of the projection followed by silu_mul_kernel (fastdms/layers/activation.py: SiluAndMul), [M, N/2].
// WV = 16-byte weight vectors per lane, row and step (8: 256 k elements per warp and step, 8 KB of weights per warp in
// flight; 16: twice that, about 200 registers, for layers with at most one CTA per SM and a long K, where the number
// of dependent round trips is what the launch costs).
template <bool BF16, int NT, bool NORM, bool GATED = false, int WV = 8>
__global__ void __launch_bounds__(kSgWarps * 32) skinny_gemm_kernel(
    const uint16_t* __restrict__ x, int64_t x_stride, const uint16_t* __restrict__ w, int64_t w_stride,
    const uint16_t* __restrict__ bias, uint16_t* __restrict__ y, int64_t y_stride, int M, int N, int K, SgNorm nrm) {
    __shared__ float s_part[kSgWarps][NT][128];
    __shared__ float s_ss[kSgWarps][8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    static_assert(!GATED || NT == 2, "the gated form pairs one gate tile with one up tile");
    const int n0 = blockIdx.x * 16 * (GATED ? 1 : NT);
    const int kslice = K / kSgWarps, k_begin = warp * kslice;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f; }
    const uint16_t* xr = x + (int64_t)g * x_stride + k_begin + 8 * t;
    // The weights do not depend on the preceding kernel: the first tile's vectors are requested before
    // the dependency is resolved, so a chained launch streams them while that kernel still runs.
    pdl_trigger();
    static_assert(WV == 8 || (NT == 1 && !NORM && !GATED), "the wide step is for plain single-tile CTAs");
    uint4 wa[WV], wb[WV];
    {
        const uint16_t* w0 = w + (int64_t)(n0 + g) * w_stride + k_begin + 8 * t;
        const uint16_t* w1 = w0 + 8 * w_stride;
#pragma unroll
        for (int j = 0; j < WV; ++j) {
            wa[j] = __ldcs((const uint4*)(w0 + 32 * j));
            wb[j] = __ldcs((const uint4*)(w1 + 32 * j));
        }
    }
    pdl_wait();
    constexpr int DT = BF16 ? FDMS_BF16 : FDMS_F16;
    const uint16_t* rr = NORM && nrm.residual ? nrm.residual + (int64_t)g * nrm.res_stride + k_begin + 8 * t : nullptr;
    float inv = 0.0f;
    if (NORM) {
        // row statistics over the whole row: this warp's slice, then the 8 warps through shared memory
        float ss = 0.0f;
        if (g < M) {
            for (int ks = 0; ks < kslice; ks += kSgStep) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float f[8];
                    sg_unpack8<BF16>(*(const uint4*)(xr + ks + 32 * j), f);
                    if (rr) {
                        float r[8];
                        sg_unpack8<BF16>(*(const uint4*)(rr + ks + 32 * j), r);
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] += r[i];
                    }
                    if (blockIdx.x == 0 && nrm.residual_out)
                        *(uint4*)(nrm.residual_out + (int64_t)g * nrm.res_out_stride + k_begin + 8 * t + ks + 32 * j) = sg_pack8<BF16>(f);
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
                }
            }
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        if (t == 0) s_ss[warp][g] = ss;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kSgWarps; ++wv) tot += s_ss[wv][g];
        inv = rsqrtf(tot / (float)K + nrm.eps);
    }
    for (int ks = 0; ks < kslice; ks += 32 * WV) {
        uint4 xb[WV];
#pragma unroll
        for (int j = 0; j < WV; ++j) {
            if (g >= M) { xb[j] = make_uint4(0u, 0u, 0u, 0u); continue; }
            if (!NORM) { xb[j] = __ldg((const uint4*)(xr + ks + 32 * j)); continue; }
            float f[8], nw[8];
            sg_unpack8<BF16>(*(const uint4*)(xr + ks + 32 * j), f);
            if (rr) {
                float r[8];
                sg_unpack8<BF16>(*(const uint4*)(rr + ks + 32 * j), r);
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] += r[i];
            }
            sg_unpack8<BF16>(__ldg((const uint4*)(nrm.norm_weight + k_begin + 8 * t + ks + 32 * j)), nw);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = round_to_dtype(f[i] * inv, DT) * nw[i];
            xb[j] = sg_pack8<BF16>(f);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int row = (GATED ? n0 + nt * (N / 2) : n0 + nt * 16) + g;       // rows row and row + 8 of W
            if (!GATED && n0 + nt * 16 >= N) break;                 // uniform: the last CTA may own fewer tiles
            const uint16_t* w0 = w + (int64_t)row * w_stride + k_begin + ks + 8 * t;
            const uint16_t* w1 = w0 + 8 * w_stride;
            if (ks != 0 || nt != 0) {
#pragma unroll
                for (int j = 0; j < WV; ++j) {
                    wa[j] = __ldcs((const uint4*)(w0 + 32 * j));
                    wb[j] = __ldcs((const uint4*)(w1 + 32 * j));
                }
            }
#pragma unroll
            for (int j = 0; j < WV; ++j) {
                sg_mma<BF16>(acc[nt], wa[j].x, wb[j].x, wa[j].y, wb[j].y, xb[j].x, xb[j].y);
                sg_mma<BF16>(acc[nt], wa[j].z, wb[j].z, wa[j].w, wb[j].w, xb[j].z, xb[j].w);
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        *(float2*)&s_part[warp][nt][g * 8 + 2 * t] = make_float2(acc[nt][0], acc[nt][1]);
        *(float2*)&s_part[warp][nt][(g + 8) * 8 + 2 * t] = make_float2(acc[nt][2], acc[nt][3]);
    }
    __syncthreads();
    if constexpr (GATED) {
        for (int idx = tid; idx < 128; idx += kSgWarps * 32) {
            const int m = idx >> 4, nl = idx & 15;
            const int n = n0 + nl;
            if (m >= M || n >= N / 2) continue;
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int wv = 0; wv < kSgWarps; ++wv) { gate += s_part[wv][0][nl * 8 + m]; up += s_part[wv][NT - 1][nl * 8 + m]; }
            if (bias) {
                gate += BF16 ? __uint_as_float((uint32_t)bias[n] << 16) : __half2float(*(const __half*)&bias[n]);
                up += BF16 ? __uint_as_float((uint32_t)bias[N / 2 + n] << 16) : __half2float(*(const __half*)&bias[N / 2 + n]);
            }
            gate = round_to_dtype(gate, DT);
            up = round_to_dtype(up, DT);
            const float out = round_to_dtype(gate / (1.0f + __expf(-gate)), DT) * up;
            uint16_t o;
            if (BF16) { const __nv_bfloat16 b = __float2bfloat16_rn(out); o = *(const uint16_t*)&b; }
            else { const __half hh = __float2half_rn(out); o = *(const uint16_t*)&hh; }
            y[(int64_t)m * y_stride + n] = o;
        }
    } else {
    for (int idx = tid; idx < NT * 128; idx += kSgWarps * 32) {
        const int nt = idx >> 7, r = idx & 127, m = r >> 4, nl = r & 15;
        const int n = n0 + nt * 16 + nl;
        if (m >= M || n >= N) continue;
        float sum = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kSgWarps; ++wv) sum += s_part[wv][nt][nl * 8 + m];
        if (bias) sum += BF16 ? __uint_as_float((uint32_t)bias[n] << 16) : __half2float(*(const __half*)&bias[n]);
        uint16_t o;
        if (BF16) { const __nv_bfloat16 b = __float2bfloat16_rn(sum); o = *(const uint16_t*)&b; }
        else { const __half hh = __float2half_rn(sum); o = *(const uint16_t*)&hh; }
        y[(int64_t)m * y_stride + n] = o;
    }
    }
}

}  // namespace fdms

using namespace fdms;

static int32_t linear_decode_launch(const void* x, int64_t x_row_stride, const void* weight, int64_t w_row_stride,
                                    const void* bias, void* y, int64_t y_row_stride, int32_t dtype, int32_t rows,
                                    int32_t out_features, int32_t in_features, const SgNorm* norm, void* stream) {
    FDMS_REQUIRE(x && weight && y, FDMS_E_ARG, "fdms_linear_decode: null pointer");
    FDMS_REQUIRE(dtype == FDMS_BF16 || dtype == FDMS_F16, FDMS_E_DTYPE, "fdms_linear_decode: bf16 or f16 only");
    FDMS_REQUIRE(rows >= 0 && rows <= 8, FDMS_E_CAPACITY, "fdms_linear_decode: at most 8 rows, got %d", rows);
    FDMS_REQUIRE(out_features > 0 && out_features % 16 == 0 && in_features > 0 && in_features % (kSgWarps * kSgStep) == 0,
                 FDMS_E_ARG, "fdms_linear_decode: out_features %% 16 and in_features %% %d must be 0 (got %d, %d)",
                 kSgWarps * kSgStep, out_features, in_features);
    FDMS_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)weight & 15) == 0 && (x_row_stride * 2) % 16 == 0 &&
                     (w_row_stride * 2) % 16 == 0,
                 FDMS_E_ARG, "fdms_linear_decode: x and weight rows must be 16-byte aligned");
    if (norm) {
        FDMS_REQUIRE(norm->norm_weight && ((uintptr_t)norm->norm_weight & 15) == 0, FDMS_E_ARG,
                     "fdms_linear_decode_norm: norm weight missing or not 16-byte aligned");
        FDMS_REQUIRE((!norm->residual || (((uintptr_t)norm->residual & 15) == 0 && (norm->res_stride * 2) % 16 == 0)) &&
                         (!norm->residual_out || (((uintptr_t)norm->residual_out & 15) == 0 && (norm->res_out_stride * 2) % 16 == 0)),
                     FDMS_E_ARG, "fdms_linear_decode_norm: residual rows must be 16-byte aligned");
        FDMS_REQUIRE(!norm->residual_out || (norm->residual_out != x && norm->residual_out != norm->residual), FDMS_E_ARG,
                     "fdms_linear_decode_norm: residual_out must not alias x or residual (other CTAs still read them)");
    }
    if (rows == 0) return FDMS_OK;
    const int tiles = out_features / 16;
    const int nt = tiles >= 4096 ? 4 : (tiles >= 1024 ? 2 : 1);
    const unsigned grid = (unsigned)((tiles + nt - 1) / nt);
    const bool bf = dtype == FDMS_BF16;
    cudaStream_t st = (cudaStream_t)stream;
    const SgNorm nrm = norm ? *norm : SgNorm{nullptr, 0, nullptr, 0.0f, nullptr, 0};
    // Few CTAs (at most one per SM) and a long K: twice the weights per warp and step in flight (down_proj of the 1B
    // shape: four dependent round trips become two).  FDMS_LINEAR_WIDE=0 turns it off.
    static const bool wide_on = [] { const char* e = getenv("FDMS_LINEAR_WIDE"); return !(e && e[0] == '0'); }();
    if (!norm && nt == 1 && wide_on && grid <= 148 && in_features % (kSgWarps * 512) == 0) {
        if (bf)
            FDMS_CUDA_OK(launch_chained(skinny_gemm_kernel<true, 1, false, false, 16>, dim3(grid), dim3(kSgWarps * 32), st, chain_launches(),
                                        (const uint16_t*)x, x_row_stride, (const uint16_t*)weight, w_row_stride, (const uint16_t*)bias,
                                        (uint16_t*)y, y_row_stride, (int)rows, (int)out_features, (int)in_features, nrm));
        else
            FDMS_CUDA_OK(launch_chained(skinny_gemm_kernel<false, 1, false, false, 16>, dim3(grid), dim3(kSgWarps * 32), st, chain_launches(),
                                        (const uint16_t*)x, x_row_stride, (const uint16_t*)weight, w_row_stride, (const uint16_t*)bias,
                                        (uint16_t*)y, y_row_stride, (int)rows, (int)out_features, (int)in_features, nrm));
        FDMS_CHECK_LAUNCH("skinny_gemm_kernel (wide step)");
        return FDMS_OK;
    }
#define FDMS_SG_LAUNCH(B, T, NM)                                                                                \
    FDMS_CUDA_OK(launch_chained(skinny_gemm_kernel<B, T, NM>, dim3(grid), dim3(kSgWarps * 32), st, chain_launches(), \
                                (const uint16_t*)x, x_row_stride, (const uint16_t*)weight, w_row_stride,         \
                                (const uint16_t*)bias, (uint16_t*)y, y_row_stride, (int)rows, (int)out_features, \
                                (int)in_features, nrm))
#define FDMS_SG_PICK(B, NM)                                                                    \
    do {                                                                                       \
        if (nt == 4) FDMS_SG_LAUNCH(B, 4, NM); else if (nt == 2) FDMS_SG_LAUNCH(B, 2, NM); else FDMS_SG_LAUNCH(B, 1, NM); \
    } while (0)
    if (norm) { if (bf) FDMS_SG_PICK(true, true); else FDMS_SG_PICK(false, true); }
    else { if (bf) FDMS_SG_PICK(true, false); else FDMS_SG_PICK(false, false); }
#undef FDMS_SG_PICK
#undef FDMS_SG_LAUNCH
    FDMS_CHECK_LAUNCH("skinny_gemm_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_linear_decode(const void* x, int64_t x_row_stride, const void* weight, int64_t w_row_stride,
                                      const void* bias, void* y, int64_t y_row_stride, int32_t dtype, int32_t rows,
                                      int32_t out_features, int32_t in_features, void* stream) {
    clear_error();
    return linear_decode_launch(x, x_row_stride, weight, w_row_stride, bias, y, y_row_stride, dtype, rows, out_features,
                                in_features, nullptr, stream);
}

extern "C" int32_t fdms_linear_decode_gated(const void* x, int64_t x_row_stride, const void* weight, int64_t w_row_stride,
                                            const void* bias, void* y, int64_t y_row_stride, int32_t dtype, int32_t rows,
                                            int32_t out_features, int32_t in_features, void* stream) {
    clear_error();
    FDMS_REQUIRE(x && weight && y, FDMS_E_ARG, "fdms_linear_decode_gated: null pointer");
    FDMS_REQUIRE(dtype == FDMS_BF16 || dtype == FDMS_F16, FDMS_E_DTYPE, "fdms_linear_decode_gated: bf16 or f16 only");
    FDMS_REQUIRE(rows >= 0 && rows <= 8, FDMS_E_CAPACITY, "fdms_linear_decode_gated: at most 8 rows, got %d", rows);
    FDMS_REQUIRE(out_features > 0 && out_features % 32 == 0 && in_features > 0 && in_features % (kSgWarps * kSgStep) == 0,
                 FDMS_E_ARG, "fdms_linear_decode_gated: out_features %% 32 and in_features %% %d must be 0 (got %d, %d)",
                 kSgWarps * kSgStep, out_features, in_features);
    FDMS_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)weight & 15) == 0 && (x_row_stride * 2) % 16 == 0 &&
                     (w_row_stride * 2) % 16 == 0,
                 FDMS_E_ARG, "fdms_linear_decode_gated: x and weight rows must be 16-byte aligned");
    if (rows == 0) return FDMS_OK;
    const unsigned grid = (unsigned)(out_features / 32);
    cudaStream_t st = (cudaStream_t)stream;
    const SgNorm nrm{nullptr, 0, nullptr, 0.0f, nullptr, 0};
    if (dtype == FDMS_BF16)
        FDMS_CUDA_OK(launch_chained(skinny_gemm_kernel<true, 2, false, true>, dim3(grid), dim3(kSgWarps * 32), st, chain_launches(),
                                    (const uint16_t*)x, x_row_stride, (const uint16_t*)weight, w_row_stride, (const uint16_t*)bias,
                                    (uint16_t*)y, y_row_stride, (int)rows, (int)out_features, (int)in_features, nrm));
    else
        FDMS_CUDA_OK(launch_chained(skinny_gemm_kernel<false, 2, false, true>, dim3(grid), dim3(kSgWarps * 32), st, chain_launches(),
                                    (const uint16_t*)x, x_row_stride, (const uint16_t*)weight, w_row_stride, (const uint16_t*)bias,
                                    (uint16_t*)y, y_row_stride, (int)rows, (int)out_features, (int)in_features, nrm));
    FDMS_CHECK_LAUNCH("skinny_gemm_kernel (gated)");
    return FDMS_OK;
}

extern "C" int32_t fdms_linear_decode_norm(
    const void* x, int64_t x_row_stride, const void* residual, int64_t residual_row_stride, const void* norm_weight,
    float eps, void* residual_out, int64_t residual_out_row_stride, const void* weight, int64_t w_row_stride,
    const void* bias, void* y, int64_t y_row_stride, int32_t dtype, int32_t rows, int32_t out_features,
    int32_t in_features, void* stream) {
    clear_error();
    SgNorm n;
    n.residual = (const uint16_t*)residual; n.res_stride = residual_row_stride;
    n.norm_weight = (const uint16_t*)norm_weight; n.eps = eps;
    n.residual_out = (uint16_t*)residual_out; n.res_out_stride = residual_out_row_stride;
    return linear_decode_launch(x, x_row_stride, weight, w_row_stride, bias, y, y_row_stride, dtype, rows, out_features,
                                in_features, &n, stream);
}

// ------------------------------------------------------------------------------------------------
// FP8 (e4m3) weights with one float32 scale per output column: y = (x W8^T) * scale (+ bias).
// Half the weight bytes of the 16-bit kernel for the same layer (the reference's opt-in FP8 weight path,
// fastdms/layers/linear.py:548-662, quantises the activations as well and calls torch._scaled_mm; here
// the activations stay 16-bit and only the weights are stored in FP8).  Same decomposition as above:
// 8 warps split K, weight rows on the M side of mma.sync.m16n8k16.  A lane streams 16-byte vectors of
// 16 weights; the bytes are converted EXACTLY to f16 pairs in registers (cvt.rn.f16x2.e4m3x2) and the
// activations are converted to f16 once per CTA (exact for bf16 values inside the f16 range, which
// decode activations are), so the products are exact and the accumulation is float32.  The MMA's k
// index is again a fixed permutation of memory order shared by both operands: a lane's eight k-pairs
// are the eight byte pairs of its weight vector and the eight 32-bit words of the matching 32 bytes of x.
// ------------------------------------------------------------------------------------------------
namespace fdms {

// VECS = 16-byte weight vectors per lane, row and step: 64 * VECS k elements per warp and step.  With 4 a warp has
// 4 KB of weights in flight, half of what the 16-bit kernel keeps; layers with few tiles and a long K (down_proj)
// take 8, so that the halved bytes also halve the number of dependent round trips.

__device__ __forceinline__ void sg8_cvt(uint32_t w, uint32_t& lo, uint32_t& hi) {       // 4 e4m3 bytes -> 2 f16x2
    asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
        : "=r"(lo), "=r"(hi) : "r"(w));
}
__device__ __forceinline__ void sg8_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 8 consecutive 16-bit activations -> 4 f16x2 words
template <bool BF16>
__device__ __forceinline__ void sg8_x_to_f16(const uint4& v, uint32_t (&o)[4]) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (BF16) {
            const __half2 h = __floats2half2_rn(__uint_as_float(u[i] << 16), __uint_as_float(u[i] & 0xffff0000u));
            o[i] = *(const uint32_t*)&h;
        } else {
            o[i] = u[i];
        }
    }
}

template <bool BF16, int NT, int VECS>
__global__ void __launch_bounds__(kSgWarps * 32) skinny_gemm_fp8_kernel(
    const uint16_t* __restrict__ x, int64_t x_stride, const uint8_t* __restrict__ w, int64_t w_stride,
    const float* __restrict__ scale, const uint16_t* __restrict__ bias, uint16_t* __restrict__ y, int64_t y_stride,
    int M, int N, int K) {
    __shared__ float s_part[kSgWarps][NT][128];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16 * NT;
    const int kslice = K / kSgWarps, k_begin = warp * kslice;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f; }
    pdl_trigger();
    // first tile's weight vectors before the dependency is resolved (weights are written by nobody)
    uint4 wa[VECS], wb[VECS];
    {
        const uint8_t* w0 = w + (int64_t)(n0 + g) * w_stride + k_begin + 16 * t;
        const uint8_t* w1 = w0 + 8 * w_stride;
#pragma unroll
        for (int j = 0; j < VECS; ++j) {
            wa[j] = __ldcs((const uint4*)(w0 + 64 * j));
            wb[j] = __ldcs((const uint4*)(w1 + 64 * j));
        }
    }
    pdl_wait();
    const uint16_t* xr = x + (int64_t)g * x_stride + k_begin + 16 * t;
    for (int ks = 0; ks < kslice; ks += 64 * VECS) {
        uint32_t xb[VECS][8];
#pragma unroll
        for (int j = 0; j < VECS; ++j) {
            if (g >= M) {
#pragma unroll
                for (int i = 0; i < 8; ++i) xb[j][i] = 0u;
                continue;
            }
            uint32_t lo[4], hi[4];
            sg8_x_to_f16<BF16>(__ldg((const uint4*)(xr + ks + 64 * j)), lo);
            sg8_x_to_f16<BF16>(__ldg((const uint4*)(xr + ks + 64 * j + 8)), hi);
#pragma unroll
            for (int i = 0; i < 4; ++i) { xb[j][i] = lo[i]; xb[j][4 + i] = hi[i]; }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            if (n0 + nt * 16 >= N) break;                           // uniform: the last CTA may own fewer tiles
            const uint8_t* w0 = w + (int64_t)(n0 + nt * 16 + g) * w_stride + k_begin + ks + 16 * t;
            const uint8_t* w1 = w0 + 8 * w_stride;
            if (ks != 0 || nt != 0) {
#pragma unroll
                for (int j = 0; j < VECS; ++j) {
                    wa[j] = __ldcs((const uint4*)(w0 + 64 * j));
                    wb[j] = __ldcs((const uint4*)(w1 + 64 * j));
                }
            }
#pragma unroll
            for (int j = 0; j < VECS; ++j) {
                const uint32_t aw[4] = {wa[j].x, wa[j].y, wa[j].z, wa[j].w}, bw[4] = {wb[j].x, wb[j].y, wb[j].z, wb[j].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t a0, a2, a1, a3;
                    sg8_cvt(aw[i], a0, a2);                        // bytes 4i, 4i+1 | 4i+2, 4i+3 of row g
                    sg8_cvt(bw[i], a1, a3);                        // the same bytes of row g + 8
                    sg8_mma(acc[nt], a0, a1, a2, a3, xb[j][2 * i], xb[j][2 * i + 1]);
                }
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        *(float2*)&s_part[warp][nt][g * 8 + 2 * t] = make_float2(acc[nt][0], acc[nt][1]);
        *(float2*)&s_part[warp][nt][(g + 8) * 8 + 2 * t] = make_float2(acc[nt][2], acc[nt][3]);
    }
    __syncthreads();
    for (int idx = tid; idx < NT * 128; idx += kSgWarps * 32) {
        const int nt = idx >> 7, r = idx & 127, m = r & 7, nl = r >> 3;
        const int n = n0 + nt * 16 + nl;
        if (m >= M || n >= N) continue;
        float sum = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kSgWarps; ++wv) sum += s_part[wv][nt][nl * 8 + m];
        sum *= scale[n];
        if (bias) sum += BF16 ? __uint_as_float((uint32_t)bias[n] << 16) : __half2float(*(const __half*)&bias[n]);
        uint16_t o;
        if (BF16) { const __nv_bfloat16 b = __float2bfloat16_rn(sum); o = *(const uint16_t*)&b; }
        else { const __half hh = __float2half_rn(sum); o = *(const uint16_t*)&hh; }
        y[(int64_t)m * y_stride + n] = o;
    }
}

}  // namespace fdms

extern "C" int32_t fdms_linear_decode_fp8(const void* x, int64_t x_row_stride, const void* weight_e4m3, int64_t w_row_stride,
                                          const float* scale, const void* bias, void* y, int64_t y_row_stride, int32_t dtype,
                                          int32_t rows, int32_t out_features, int32_t in_features, void* stream) {
    clear_error();
    FDMS_REQUIRE(x && weight_e4m3 && scale && y, FDMS_E_ARG, "fdms_linear_decode_fp8: null pointer");
    FDMS_REQUIRE(dtype == FDMS_BF16 || dtype == FDMS_F16, FDMS_E_DTYPE, "fdms_linear_decode_fp8: bf16 or f16 activations only");
    FDMS_REQUIRE(rows >= 0 && rows <= 8, FDMS_E_CAPACITY, "fdms_linear_decode_fp8: at most 8 rows, got %d", rows);
    FDMS_REQUIRE(out_features > 0 && out_features % 16 == 0 && in_features > 0 && in_features % (kSgWarps * kSgStep) == 0,
                 FDMS_E_ARG, "fdms_linear_decode_fp8: out_features %% 16 and in_features %% %d must be 0 (got %d, %d)",
                 kSgWarps * kSgStep, out_features, in_features);
    FDMS_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)weight_e4m3 & 15) == 0 && (x_row_stride * 2) % 16 == 0 &&
                     w_row_stride % 16 == 0,
                 FDMS_E_ARG, "fdms_linear_decode_fp8: x and weight rows must be 16-byte aligned");
    if (rows == 0) return FDMS_OK;
    const int tiles = out_features / 16;
    const int nt = tiles >= 4096 ? 4 : (tiles >= 1024 ? 2 : 1);
    const unsigned grid = (unsigned)((tiles + nt - 1) / nt);
    const bool bf = dtype == FDMS_BF16;
    cudaStream_t st = (cudaStream_t)stream;
    // 8 vectors per step (8 KB of weights per warp in flight, about 150 registers: one CTA per SM) where a warp's K
    // range allows it and the layer has no more CTAs than that anyway: down_proj of the 1B shape 10.1 -> 8.4 us; with
    // 256 CTAs (the 8B shape's 4096-wide layers) the lost occupancy costs more, 16.3 -> 24.2 us.  FDMS_FP8_VECS=4 / 8
    // overrides.
    static const int vecs_env = [] { const char* e = getenv("FDMS_FP8_VECS"); return e ? atoi(e) : 0; }();
    const bool can8 = nt == 1 && in_features % (kSgWarps * 512) == 0;
    const bool vecs8 = can8 && (vecs_env == 8 || (vecs_env != 4 && grid <= 148));
#define FDMS_SG8_LAUNCH(B, T, V)                                                                                    \
    FDMS_CUDA_OK(launch_chained(skinny_gemm_fp8_kernel<B, T, V>, dim3(grid), dim3(kSgWarps * 32), st, chain_launches(), \
                                (const uint16_t*)x, x_row_stride, (const uint8_t*)weight_e4m3, w_row_stride, scale,      \
                                (const uint16_t*)bias, (uint16_t*)y, y_row_stride, (int)rows, (int)out_features,         \
                                (int)in_features))
#define FDMS_SG8_PICK(B)                                                                                  \
    do {                                                                                                  \
        if (vecs8) FDMS_SG8_LAUNCH(B, 1, 8);                                                              \
        else if (nt == 4) FDMS_SG8_LAUNCH(B, 4, 4); else if (nt == 2) FDMS_SG8_LAUNCH(B, 2, 4); else FDMS_SG8_LAUNCH(B, 1, 4); \
    } while (0)
    if (bf) FDMS_SG8_PICK(true); else FDMS_SG8_PICK(false);
#undef FDMS_SG8_PICK
#undef FDMS_SG8_LAUNCH
    FDMS_CHECK_LAUNCH("skinny_gemm_fp8_kernel");
    return FDMS_OK;
}

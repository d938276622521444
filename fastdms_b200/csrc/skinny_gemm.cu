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

template <bool BF16, int NT>
__global__ void __launch_bounds__(kSgWarps * 32) skinny_gemm_kernel(
    const uint16_t* __restrict__ x, int64_t x_stride, const uint16_t* __restrict__ w, int64_t w_stride,
    const uint16_t* __restrict__ bias, uint16_t* __restrict__ y, int64_t y_stride, int M, int N, int K) {
    __shared__ float s_part[kSgWarps][NT][128];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16 * NT;
    const int kslice = K / kSgWarps, k_begin = warp * kslice;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f; }
    const uint16_t* xr = x + (int64_t)g * x_stride + k_begin + 8 * t;
    // The weights do not depend on the preceding kernel: the first tile's vectors are requested before
    // the dependency is resolved, so a chained launch streams them while that kernel still runs.
    pdl_trigger();
    uint4 wa[8], wb[8];
    {
        const uint16_t* w0 = w + (int64_t)(n0 + g) * w_stride + k_begin + 8 * t;
        const uint16_t* w1 = w0 + 8 * w_stride;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            wa[j] = __ldcs((const uint4*)(w0 + 32 * j));
            wb[j] = __ldcs((const uint4*)(w1 + 32 * j));
        }
    }
    pdl_wait();
    for (int ks = 0; ks < kslice; ks += kSgStep) {
        uint4 xb[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            xb[j] = g < M ? __ldg((const uint4*)(xr + ks + 32 * j)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int row = n0 + nt * 16 + g;                       // rows row and row + 8 of W
            if (n0 + nt * 16 >= N) break;                           // uniform: the last CTA may own fewer tiles
            const uint16_t* w0 = w + (int64_t)row * w_stride + k_begin + ks + 8 * t;
            const uint16_t* w1 = w0 + 8 * w_stride;
            if (ks != 0 || nt != 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    wa[j] = __ldcs((const uint4*)(w0 + 32 * j));
                    wb[j] = __ldcs((const uint4*)(w1 + 32 * j));
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
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

}  // namespace fdms

using namespace fdms;

extern "C" int32_t fdms_linear_decode(const void* x, int64_t x_row_stride, const void* weight, int64_t w_row_stride,
                                      const void* bias, void* y, int64_t y_row_stride, int32_t dtype, int32_t rows,
                                      int32_t out_features, int32_t in_features, void* stream) {
    clear_error();
    FDMS_REQUIRE(x && weight && y, FDMS_E_ARG, "fdms_linear_decode: null pointer");
    FDMS_REQUIRE(dtype == FDMS_BF16 || dtype == FDMS_F16, FDMS_E_DTYPE, "fdms_linear_decode: bf16 or f16 only");
    FDMS_REQUIRE(rows >= 0 && rows <= 8, FDMS_E_CAPACITY, "fdms_linear_decode: at most 8 rows, got %d", rows);
    FDMS_REQUIRE(out_features > 0 && out_features % 16 == 0 && in_features > 0 && in_features % (kSgWarps * kSgStep) == 0,
                 FDMS_E_ARG, "fdms_linear_decode: out_features %% 16 and in_features %% %d must be 0 (got %d, %d)",
                 kSgWarps * kSgStep, out_features, in_features);
    FDMS_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)weight & 15) == 0 && (x_row_stride * 2) % 16 == 0 &&
                     (w_row_stride * 2) % 16 == 0,
                 FDMS_E_ARG, "fdms_linear_decode: x and weight rows must be 16-byte aligned");
    if (rows == 0) return FDMS_OK;
    const int tiles = out_features / 16;
    const int nt = tiles >= 4096 ? 4 : (tiles >= 1024 ? 2 : 1);
    const unsigned grid = (unsigned)((tiles + nt - 1) / nt);
    const bool bf = dtype == FDMS_BF16;
    cudaStream_t st = (cudaStream_t)stream;
#define FDMS_SG_LAUNCH(B, T)                                                                                   \
    FDMS_CUDA_OK(launch_chained(skinny_gemm_kernel<B, T>, dim3(grid), dim3(kSgWarps * 32), st, chain_launches(),   \
                                (const uint16_t*)x, x_row_stride, (const uint16_t*)weight, w_row_stride,            \
                                (const uint16_t*)bias, (uint16_t*)y, y_row_stride, (int)rows, (int)out_features,    \
                                (int)in_features))
    if (bf) { if (nt == 4) FDMS_SG_LAUNCH(true, 4); else if (nt == 2) FDMS_SG_LAUNCH(true, 2); else FDMS_SG_LAUNCH(true, 1); }
    else { if (nt == 4) FDMS_SG_LAUNCH(false, 4); else if (nt == 2) FDMS_SG_LAUNCH(false, 2); else FDMS_SG_LAUNCH(false, 1); }
#undef FDMS_SG_LAUNCH
    FDMS_CHECK_LAUNCH("skinny_gemm_kernel");
    return FDMS_OK;
}

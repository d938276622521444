// Row-wise helpers of the decoder block that sit between the attention launches of a decode step:
// RMSNorm with optional residual add, and SiLU(gate) * up.  16-bit activations (bf16 / f16), float32
// statistics, one 16-byte vector (8 elements) per load; results are rounded where the reference's
// torch ops round (fastdms/layers/layernorm.py:16-48, fastdms/layers/activation.py).
#include "common.cuh"

namespace fdms {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;        // 16-byte vectors per thread: hidden <= 8 * 4 * group size

__device__ __forceinline__ void unpack8(const uint4& v, int dt, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (dt == FDMS_BF16) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const __half2 h = *(const __half2*)&w[i];
            f[2 * i] = __low2float(h);
            f[2 * i + 1] = __high2float(h);
        }
    }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8], int dt) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (dt == FDMS_BF16) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *(const uint32_t*)&b;
        } else {
            const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *(const uint32_t*)&h;
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// A group of `T` threads (a power of two, 32..256) owns one row; a CTA holds 256 / T rows.
//   xf  = float(x) (+ float(residual))           residual_out = round(xf)
//   out = round(round(xf * rsqrt(mean(xf^2) + eps)) * weight)
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(
    const uint16_t* x, int64_t x_stride, const uint16_t* residual, int64_t res_stride, const uint16_t* weight,
    uint16_t* out, int64_t out_stride, uint16_t* residual_out, int64_t res_out_stride, int dt, int64_t rows, int hidden,
    float eps, int T) {
    __shared__ float s_part[kNormThreads / 32];
    pdl_trigger();                                         // the next kernel may start streaming its weights
    pdl_wait();                                            // x / residual come from the preceding kernel
    const int tid = threadIdx.x;
    const int grp = tid / T, lig = tid - grp * T;          // group index, lane in group
    const int64_t row = (int64_t)blockIdx.x * (kNormThreads / T) + grp;
    const int nvec = hidden >> 3;
    const bool live = row < rows;
    float v[kNormMaxVec][8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kNormMaxVec; ++j) {
        const int c = lig + j * T;
        if (live && c < nvec) {
            unpack8(*(const uint4*)(x + row * x_stride + 8 * c), dt, v[j]);
            if (residual) {
                float r[8];
                unpack8(*(const uint4*)(residual + row * res_stride + 8 * c), dt, r);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[j][i] += r[i];
            }
            if (residual_out) *(uint4*)(residual_out + row * res_out_stride + 8 * c) = pack8(v[j], dt);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += v[j][i] * v[j][i];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (T > 32) {
        if ((tid & 31) == 0) s_part[tid >> 5] = ss;
        __syncthreads();
        const int w0 = (grp * T) >> 5;
        ss = 0.0f;
        for (int w = 0; w < (T >> 5); ++w) ss += s_part[w0 + w];
    }
    const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int j = 0; j < kNormMaxVec; ++j) {
        const int c = lig + j * T;
        if (live && c < nvec) {
            float w[8], y[8];
            unpack8(*(const uint4*)(weight + 8 * c), dt, w);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = round_to_dtype(v[j][i] * inv, dt) * w[i];
            *(uint4*)(out + row * out_stride + 8 * c) = pack8(y, dt);
        }
    }
}

// Per-head RMSNorm of the q and k heads of a fused projection output, in place, one launch: a warp owns one
// (row, head) of head_dim <= 256 elements (one 16-byte vector per lane).  Same arithmetic as rmsnorm_kernel.
__global__ void __launch_bounds__(kNormThreads) qk_rmsnorm_kernel(
    uint16_t* q, int64_t q_sb, int64_t q_sh, int q_heads, const uint16_t* q_weight,
    uint16_t* k, int64_t k_sb, int64_t k_sh, int k_heads, const uint16_t* k_weight,
    int dt, int64_t rows, int head_dim, float eps) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int heads = q_heads + k_heads;
    const int64_t unit = (int64_t)blockIdx.x * (kNormThreads / 32) + (threadIdx.x >> 5);
    if (unit >= rows * heads) return;
    const int64_t row = unit / heads;
    const int head = (int)(unit - row * heads);
    const bool isq = head < q_heads;
    uint16_t* x = isq ? q + row * q_sb + (int64_t)head * q_sh : k + row * k_sb + (int64_t)(head - q_heads) * k_sh;
    const uint16_t* weight = isq ? q_weight : k_weight;
    const bool have = lane < (head_dim >> 3);
    float v[8], ss = 0.0f;
    if (have) {
        unpack8(*(const uint4*)(x + 8 * lane), dt, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / (float)head_dim + eps);
    if (have) {
        float w[8], y[8];
        unpack8(*(const uint4*)(weight + 8 * lane), dt, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = round_to_dtype(v[i] * inv, dt) * w[i];
        *(uint4*)(x + 8 * lane) = pack8(y, dt);
    }
}

// out[r, c] = round(round(silu(x[r, c])) * x[r, n + c]), 8 elements per thread.
__global__ void silu_mul_kernel(const uint16_t* x, int64_t x_stride, uint16_t* out, int64_t out_stride, int dt,
                                int64_t rows, int n) {
    const int nvec = n >> 3;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i >= rows * nvec) return;
    const int64_t r = i / nvec;
    const int c = (int)(i - r * nvec);
    float a[8], b[8], y[8];
    unpack8(*(const uint4*)(x + r * x_stride + 8 * c), dt, a);
    unpack8(*(const uint4*)(x + r * x_stride + n + 8 * c), dt, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) y[k] = round_to_dtype(a[k] / (1.0f + __expf(-a[k])), dt) * b[k];
    *(uint4*)(out + r * out_stride + 8 * c) = pack8(y, dt);
}

}  // namespace fdms

using namespace fdms;

static bool aligned16(const void* p, int64_t stride_elems) {
    return ((uintptr_t)p & 15) == 0 && ((stride_elems * 2) & 15) == 0;
}

extern "C" int32_t fdms_rmsnorm(
    const void* x, int64_t x_row_stride, const void* residual, int64_t residual_row_stride, const void* weight,
    void* out, int64_t out_row_stride, void* residual_out, int64_t residual_out_row_stride,
    int32_t dtype, int64_t rows, int32_t hidden, float eps, void* stream) {
    clear_error();
    FDMS_REQUIRE(x && weight && out, FDMS_E_ARG, "fdms_rmsnorm: null pointer");
    FDMS_REQUIRE(dtype == FDMS_BF16 || dtype == FDMS_F16, FDMS_E_DTYPE, "fdms_rmsnorm: bf16 or f16 activations only");
    FDMS_REQUIRE(rows >= 0 && hidden > 0 && hidden % 8 == 0, FDMS_E_ARG, "fdms_rmsnorm: hidden must be a positive multiple of 8");
    FDMS_REQUIRE(aligned16(x, x_row_stride) && aligned16(out, out_row_stride) && aligned16(weight, 0) &&
                     (!residual || aligned16(residual, residual_row_stride)) &&
                     (!residual_out || aligned16(residual_out, residual_out_row_stride)),
                 FDMS_E_ARG, "fdms_rmsnorm: pointers and row strides must be 16-byte aligned");
    if (rows == 0) return FDMS_OK;
    const int nvec = hidden / 8;
    int T = 32;
    while (T < kNormThreads && T * 2 <= nvec) T *= 2;          // about one vector per thread
    while (T < kNormThreads && T * kNormMaxVec < nvec) T *= 2;
    FDMS_REQUIRE(T * kNormMaxVec >= nvec, FDMS_E_CAPACITY, "fdms_rmsnorm: hidden=%d is larger than %d", hidden,
                 kNormThreads * kNormMaxVec * 8);
    const int rows_per_block = kNormThreads / T;
    const int64_t blocks = (rows + rows_per_block - 1) / rows_per_block;
    FDMS_REQUIRE(blocks < (1ll << 31), FDMS_E_CAPACITY, "fdms_rmsnorm: too many rows");
    FDMS_CUDA_OK(launch_chained(
        rmsnorm_kernel, dim3((unsigned)blocks), dim3(kNormThreads), (cudaStream_t)stream, chain_launches(),
        (const uint16_t*)x, x_row_stride, (const uint16_t*)residual, residual_row_stride, (const uint16_t*)weight,
        (uint16_t*)out, out_row_stride, (uint16_t*)residual_out, residual_out_row_stride, (int)dtype, rows, (int)hidden, eps, T));
    FDMS_CHECK_LAUNCH("rmsnorm_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_qk_rmsnorm(
    void* q, int64_t q_stride_row, int64_t q_stride_head, int32_t q_heads, const void* q_weight,
    void* k, int64_t k_stride_row, int64_t k_stride_head, int32_t k_heads, const void* k_weight,
    int32_t dtype, int64_t rows, int32_t head_dim, float eps, void* stream) {
    clear_error();
    FDMS_REQUIRE(q && k && q_weight && k_weight, FDMS_E_ARG, "fdms_qk_rmsnorm: null pointer");
    FDMS_REQUIRE(dtype == FDMS_BF16 || dtype == FDMS_F16, FDMS_E_DTYPE, "fdms_qk_rmsnorm: bf16 or f16 activations only");
    FDMS_REQUIRE(rows >= 0 && q_heads > 0 && k_heads > 0 && head_dim > 0 && head_dim % 8 == 0 && head_dim <= 256, FDMS_E_ARG,
                 "fdms_qk_rmsnorm: head_dim must be a multiple of 8 up to 256, got %d", head_dim);
    FDMS_REQUIRE(aligned16(q, q_stride_row) && aligned16(q, q_stride_head) && aligned16(k, k_stride_row) &&
                     aligned16(k, k_stride_head) && aligned16(q_weight, 0) && aligned16(k_weight, 0),
                 FDMS_E_ARG, "fdms_qk_rmsnorm: pointers and strides must be 16-byte aligned");
    if (rows == 0) return FDMS_OK;
    const int64_t units = rows * (q_heads + k_heads);
    const int64_t blocks = (units + kNormThreads / 32 - 1) / (kNormThreads / 32);
    FDMS_REQUIRE(blocks < (1ll << 31), FDMS_E_CAPACITY, "fdms_qk_rmsnorm: too many rows");
    FDMS_CUDA_OK(launch_chained(
        qk_rmsnorm_kernel, dim3((unsigned)blocks), dim3(kNormThreads), (cudaStream_t)stream, chain_launches(),
        (uint16_t*)q, q_stride_row, q_stride_head, (int)q_heads, (const uint16_t*)q_weight,
        (uint16_t*)k, k_stride_row, k_stride_head, (int)k_heads, (const uint16_t*)k_weight,
        (int)dtype, rows, (int)head_dim, eps));
    FDMS_CHECK_LAUNCH("qk_rmsnorm_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_silu_and_mul(const void* x, int64_t x_row_stride, void* out, int64_t out_row_stride,
                                     int32_t dtype, int64_t rows, int32_t n, void* stream) {
    clear_error();
    FDMS_REQUIRE(x && out, FDMS_E_ARG, "fdms_silu_and_mul: null pointer");
    FDMS_REQUIRE(dtype == FDMS_BF16 || dtype == FDMS_F16, FDMS_E_DTYPE, "fdms_silu_and_mul: bf16 or f16 activations only");
    FDMS_REQUIRE(rows >= 0 && n > 0 && n % 8 == 0, FDMS_E_ARG, "fdms_silu_and_mul: n must be a positive multiple of 8");
    FDMS_REQUIRE(aligned16(x, x_row_stride) && aligned16(out, out_row_stride), FDMS_E_ARG,
                 "fdms_silu_and_mul: pointers and row strides must be 16-byte aligned");
    if (rows == 0) return FDMS_OK;
    const int64_t total = rows * (n / 8);
    const int64_t blocks = (total + 255) / 256;
    FDMS_REQUIRE(blocks < (1ll << 31), FDMS_E_CAPACITY, "fdms_silu_and_mul: too many elements");
    FDMS_CUDA_OK(launch_chained(silu_mul_kernel, dim3((unsigned)blocks), dim3(256), (cudaStream_t)stream, chain_launches(),
                                (const uint16_t*)x, x_row_stride, (uint16_t*)out, out_row_stride, (int)dtype, rows, (int)n));
    FDMS_CHECK_LAUNCH("silu_mul_kernel");
    return FDMS_OK;
}

// ---------------------------------------------------------------------------------------------------
// Greedy head: index of the largest logit of every row (the reference takes `logits.argmax(dim=-1)`
// for temperature-0 requests, fastdms/engine/model_runner.py:1147-1151).  Ties go to the lowest
// index and a NaN counts as the largest value, as torch's argmax does.  One launch: every CTA
// reduces a slice of a row to a 64-bit key (ordered value bits | inverted index), merges it into the
// row's key with an atomic max, and the last CTA of a row to finish decodes the key and clears the
// row's two scratch words again (the scratch must be zero before the first call only).
namespace fdms {

constexpr int kArgmaxThreads = 256;
constexpr int kArgmaxVecPerThread = 4;                 // 8 x 16-bit or 4 x 32-bit elements per vector

__device__ __forceinline__ uint32_t ordered_bits(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long argmax_key(float f, uint32_t idx) {
    if (f != f) f = __uint_as_float(0x7fc00000u);      // any NaN -> the canonical positive one (above +inf)
    return ((unsigned long long)ordered_bits(f) << 32) | (unsigned long long)(0xffffffffu - idx);
}

__global__ void __launch_bounds__(kArgmaxThreads) argmax_rows_kernel(
    const void* x, int64_t row_stride, int dt, int64_t n, int per_cta, int ctas_per_row, int vec_ok,
    unsigned long long* keys, unsigned int* done, int64_t* out) {
    __shared__ unsigned long long s_key[kArgmaxThreads / 32];
    const int row = blockIdx.y, tid = threadIdx.x;
    const int64_t lo = (int64_t)blockIdx.x * per_cta;
    const int64_t hi = lo + per_cta < n ? lo + per_cta : n;
    const char* base = (const char*)x + row * row_stride * (dt == FDMS_F32 ? 4 : 2);
    unsigned long long best = 0ull;
    if (vec_ok) {
        const int epv = dt == FDMS_F32 ? 4 : 8;        // elements per 16-byte vector
        uint4 v[kArgmaxVecPerThread];
        int64_t at[kArgmaxVecPerThread];
#pragma unroll
        for (int j = 0; j < kArgmaxVecPerThread; ++j) {
            at[j] = lo + ((int64_t)j * kArgmaxThreads + tid) * epv;
            v[j] = at[j] < hi ? __ldcs((const uint4*)(base + at[j] * (16 / epv))) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < kArgmaxVecPerThread; ++j) {
            if (at[j] >= hi) continue;
            if (dt == FDMS_F32) {
                const float f[4] = {__uint_as_float(v[j].x), __uint_as_float(v[j].y), __uint_as_float(v[j].z), __uint_as_float(v[j].w)};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const unsigned long long k = argmax_key(f[i], (uint32_t)(at[j] + i));
                    best = k > best ? k : best;
                }
            } else {
                float f[8];
                unpack8(v[j], dt, f);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const unsigned long long k = argmax_key(f[i], (uint32_t)(at[j] + i));
                    best = k > best ? k : best;
                }
            }
        }
    } else {
        for (int64_t i = lo + tid; i < hi; i += kArgmaxThreads) {
            const unsigned long long k = argmax_key(load_as_float(base, i, dt), (uint32_t)i);
            best = k > best ? k : best;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((tid & 31) == 0) s_key[tid >> 5] = best;
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int w = 1; w < kArgmaxThreads / 32; ++w) best = s_key[w] > best ? s_key[w] : best;
        atomicMax(&keys[row], best);
        __threadfence();
        if (atomicAdd(&done[row], 1u) == (unsigned)ctas_per_row - 1u) {
            __threadfence();
            const unsigned long long k = atomicExch(&keys[row], 0ull);
            out[row] = (int64_t)(0xffffffffu - (uint32_t)(k & 0xffffffffull));
            done[row] = 0u;
        }
    }
}

}  // namespace fdms

extern "C" int64_t fdms_argmax_workspace_bytes(int64_t rows) { return rows > 0 ? rows * 16 : 0; }

extern "C" int32_t fdms_argmax_rows(const void* x, int64_t row_stride, int32_t dtype, int64_t rows, int64_t n,
                                    int64_t* out, void* workspace, int64_t workspace_bytes, void* stream) {
    clear_error();
    FDMS_REQUIRE(x && out && workspace, FDMS_E_ARG, "fdms_argmax_rows: null pointer");
    FDMS_REQUIRE(dtype == FDMS_BF16 || dtype == FDMS_F16 || dtype == FDMS_F32, FDMS_E_DTYPE,
                 "fdms_argmax_rows: bf16, f16 or f32 logits only");
    FDMS_REQUIRE(rows >= 0 && rows < 65536 && n > 0 && n < (1ll << 32) - 1, FDMS_E_ARG,
                 "fdms_argmax_rows: rows must be below 65536 and 0 < n < 2^32 - 1");
    FDMS_REQUIRE(workspace_bytes >= fdms_argmax_workspace_bytes(rows) && ((uintptr_t)workspace & 7) == 0, FDMS_E_CAPACITY,
                 "fdms_argmax_rows: workspace of %lld bytes needed (8-byte aligned, zeroed before the first call)",
                 (long long)fdms_argmax_workspace_bytes(rows));
    if (rows == 0) return FDMS_OK;
    const int esz = dtype == FDMS_F32 ? 4 : 2, epv = 16 / esz;
    const int vec_ok = ((uintptr_t)x & 15) == 0 && (row_stride * esz) % 16 == 0 && n % epv == 0;
    const int per_cta = fdms::kArgmaxThreads * fdms::kArgmaxVecPerThread * epv;
    const int64_t ctas = (n + per_cta - 1) / per_cta;
    FDMS_REQUIRE(ctas < (1ll << 31), FDMS_E_CAPACITY, "fdms_argmax_rows: row too long");
    unsigned long long* keys = (unsigned long long*)workspace;
    unsigned int* done = (unsigned int*)(keys + rows);
    fdms::argmax_rows_kernel<<<dim3((unsigned)ctas, (unsigned)rows), fdms::kArgmaxThreads, 0, (cudaStream_t)stream>>>(
        x, row_stride, dtype, n, per_cta, (int)ctas, vec_ok, keys, done, out);
    FDMS_CHECK_LAUNCH("argmax_rows_kernel");
    return FDMS_OK;
}

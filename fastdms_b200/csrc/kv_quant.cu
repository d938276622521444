// FP8 e4m3 KV quantise / dequantise with a per-KV-head scale.  Pure streaming kernels: each
// thread converts 16 consecutive elements of one head row (one 16-byte FP8 vector), so HBM
// accesses are 128-bit wide on the FP8 side and 2-4 x 128-bit on the activation side.
#include "common.cuh"

namespace fdms {

constexpr int kQuantVec = 16;

__global__ void kv_quant_kernel(const void* x, int x_dtype, uint8_t* out, const float* scale,
                                int64_t total_vecs, int hk, int dim) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_vecs) return;
    const int64_t e0 = i * kQuantVec;
    const int h = (int)((e0 / dim) % hk);
    const float s = scale ? scale[h] : 1.0f;
    union { uint4 v; uint8_t b[16]; } o;
    float f[kQuantVec];
    if (x_dtype == FDMS_F32) {
        const float4* p = (const float4*)((const float*)x + e0);
#pragma unroll
        for (int j = 0; j < 4; ++j) { float4 t = p[j]; f[4 * j] = t.x; f[4 * j + 1] = t.y; f[4 * j + 2] = t.z; f[4 * j + 3] = t.w; }
    } else {
        union { uint4 v[2]; uint16_t u[16]; } in;
        const uint4* p = (const uint4*)((const uint16_t*)x + e0);
        in.v[0] = p[0]; in.v[1] = p[1];
#pragma unroll
        for (int j = 0; j < 16; ++j)
            f[j] = x_dtype == FDMS_BF16 ? __bfloat162float(__ushort_as_bfloat16(in.u[j]))
                                        : __half2float(__ushort_as_half(in.u[j]));
    }
#pragma unroll
    for (int j = 0; j < kQuantVec; ++j) o.b[j] = float_to_e4m3(scale ? __fdiv_rn(f[j], s) : f[j]);
    *(uint4*)(out + e0) = o.v;
}

__global__ void kv_dequant_kernel(const uint8_t* x, void* out, int out_dtype, const float* scale,
                                  int64_t total_vecs, int hk, int dim) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_vecs) return;
    const int64_t e0 = i * kQuantVec;
    const int h = (int)((e0 / dim) % hk);
    const float s = scale ? scale[h] : 1.0f;
    union { uint4 v; uint8_t b[16]; } in;
    in.v = *(const uint4*)(x + e0);
    float f[kQuantVec];
#pragma unroll
    for (int j = 0; j < kQuantVec; ++j) f[j] = __fmul_rn(e4m3_to_float(in.b[j]), s);
    if (out_dtype == FDMS_F32) {
        float4* p = (float4*)((float*)out + e0);
#pragma unroll
        for (int j = 0; j < 4; ++j) p[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
    } else {
        union { uint4 v[2]; uint16_t u[16]; } o;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            o.u[j] = out_dtype == FDMS_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(f[j]))
                                            : __half_as_ushort(__float2half_rn(f[j]));
        uint4* p = (uint4*)((uint16_t*)out + e0);
        p[0] = o.v[0]; p[1] = o.v[1];
    }
}

static int32_t check_quant_args(const char* who, const void* a, const void* b, int dt, int64_t n, int hk, int dim) {
    FDMS_REQUIRE(a && b, FDMS_E_ARG, "%s: null pointer", who);
    FDMS_REQUIRE(dt == FDMS_F32 || dt == FDMS_BF16 || dt == FDMS_F16, FDMS_E_DTYPE, "%s: dtype %d not supported", who, dt);
    FDMS_REQUIRE(n >= 0 && hk > 0 && dim > 0 && dim % kQuantVec == 0, FDMS_E_ARG,
                 "%s: head_dim=%d must be a positive multiple of %d", who, dim, kQuantVec);
    FDMS_REQUIRE((uintptr_t)a % 16 == 0 && (uintptr_t)b % 16 == 0, FDMS_E_ARG, "%s: pointers must be 16-byte aligned", who);
    return FDMS_OK;
}

}  // namespace fdms

using namespace fdms;

extern "C" int32_t fdms_kv_quant(const void* x, int32_t x_dtype, uint8_t* out, const float* scale,
                                 int64_t n, int32_t num_kv_heads, int32_t head_dim, void* stream) {
    clear_error();
    int32_t rc = check_quant_args("fdms_kv_quant", x, out, x_dtype, n, num_kv_heads, head_dim);
    if (rc != FDMS_OK) return rc;
    const int64_t vecs = n * num_kv_heads * head_dim / kQuantVec;
    if (vecs == 0) return FDMS_OK;
    kv_quant_kernel<<<(unsigned)((vecs + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        x, x_dtype, out, scale, vecs, num_kv_heads, head_dim);
    FDMS_CHECK_LAUNCH("kv_quant_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_kv_dequant(const uint8_t* x, void* out, int32_t out_dtype, const float* scale,
                                   int64_t n, int32_t num_kv_heads, int32_t head_dim, void* stream) {
    clear_error();
    int32_t rc = check_quant_args("fdms_kv_dequant", x, out, out_dtype, n, num_kv_heads, head_dim);
    if (rc != FDMS_OK) return rc;
    const int64_t vecs = n * num_kv_heads * head_dim / kQuantVec;
    if (vecs == 0) return FDMS_OK;
    kv_dequant_kernel<<<(unsigned)((vecs + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        x, out, out_dtype, scale, vecs, num_kv_heads, head_dim);
    FDMS_CHECK_LAUNCH("kv_dequant_kernel");
    return FDMS_OK;
}

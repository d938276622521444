// Shared helpers for the fastdms_b200 kernels: status reporting, dtype load/store, FP8 conversion.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fastdms_b200.h"

namespace fdms {

// Records the message returned by fdms_last_error() for this host thread and returns `code`.
int32_t fail(int32_t code, const char* fmt, ...);
void clear_error();

#define FDMS_REQUIRE(cond, code, ...)                  \
    do {                                               \
        if (!(cond)) return ::fdms::fail((code), __VA_ARGS__); \
    } while (0)

// Call after a kernel launch: converts a launch error into FDMS_E_CUDA.
#define FDMS_CHECK_LAUNCH(name)                                                              \
    do {                                                                                     \
        cudaError_t e__ = cudaGetLastError();                                                \
        if (e__ != cudaSuccess)                                                              \
            return ::fdms::fail(FDMS_E_CUDA, "%s launch failed: %s", (name), cudaGetErrorString(e__)); \
    } while (0)

// Wraps a runtime call that returns cudaError_t.
#define FDMS_CUDA_OK(expr)                                                                   \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess)                                                              \
            return ::fdms::fail(FDMS_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

__host__ __device__ inline int dtype_size(int dt) {
    return dt == FDMS_F32 ? 4 : (dt == FDMS_E4M3 ? 1 : 2);
}

// ---- scalar load/store by runtime dtype (used by the non-hot helper kernels) ------------------
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
    return __half2float(__half(h));
}

// Round-to-nearest-even, saturating to +-448 (the behaviour of the reference's GPU store).
__device__ __forceinline__ uint8_t float_to_e4m3(float x) {
    return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float load_as_float(const void* p, int64_t i, int dt) {
    switch (dt) {
        case FDMS_F32: return ((const float*)p)[i];
        case FDMS_BF16: return __bfloat162float(((const __nv_bfloat16*)p)[i]);
        case FDMS_F16: return __half2float(((const __half*)p)[i]);
        default: return e4m3_to_float(((const uint8_t*)p)[i]);
    }
}

__device__ __forceinline__ void store_from_float(void* p, int64_t i, int dt, float x) {
    switch (dt) {
        case FDMS_F32: ((float*)p)[i] = x; break;
        case FDMS_BF16: ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(x); break;
        case FDMS_F16: ((__half*)p)[i] = __float2half_rn(x); break;
        default: ((uint8_t*)p)[i] = float_to_e4m3(x); break;
    }
}

// Value of `x` after rounding to the activation dtype (what a store followed by a load would give).
__device__ __forceinline__ float round_to_dtype(float x, int dt) {
    switch (dt) {
        case FDMS_BF16: return __bfloat162float(__float2bfloat16_rn(x));
        case FDMS_F16: return __half2float(__float2half_rn(x));
        default: return x;
    }
}

// The DMS decision rule, fastdms/engine/dms.py:225-228: one float32 compare against a host-rounded
// threshold when alpha_scale > 0, else two separately rounded float32 operations.
struct DecisionRule {
    float threshold;   // float32(alpha_offset / alpha_scale) computed in double on the host
    float alpha_scale;
    float alpha_offset;
    int positive;
    __device__ __forceinline__ bool evict(float v) const {
        if (positive) return v > threshold;
        return __fsub_rn(__fmul_rn(v, alpha_scale), alpha_offset) > 0.0f;
    }
};

inline DecisionRule make_rule(double alpha_scale, double alpha_offset) {
    DecisionRule r;
    r.alpha_scale = (float)alpha_scale;
    r.alpha_offset = (float)alpha_offset;
    r.positive = alpha_scale > 0.0 ? 1 : 0;
    r.threshold = r.positive ? (float)(alpha_offset / alpha_scale) : 0.0f;
    return r;
}

// Physical pool row of logical row `i` of a span: contiguous from `base`, or through 16-row pages.
__device__ __forceinline__ int64_t span_row(int32_t base, const int32_t* bt, int32_t i) {
    if (bt == nullptr) return (int64_t)base + i;
    return (int64_t)bt[i >> 4] * 16 + (i & 15);
}


// Programmatic dependent launch for chains of small kernels.  `pdl_trigger` lets the next kernel of the
// stream (if it was launched with `launch_chained`) start its preamble while this one runs;
// `pdl_wait` returns once the preceding kernel has completed and its writes are visible (at once when
// the launch was an ordinary one).  Code before `pdl_wait` may only touch memory that no kernel of
// the stream writes (weights).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, bool chained,
                                  Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = chained ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// FDMS_PDL_CHAIN=0 launches the decoder-block helpers (norm, activation, decode-sized linear) as ordinary kernels.
inline bool chain_launches() {
    static const bool on = [] { const char* e = getenv("FDMS_PDL_CHAIN"); return !(e && e[0] == '0'); }();
    return on;
}

}  // namespace fdms

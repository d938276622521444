// Decode-step preprocess: DMS decision + neox RoPE + FP8 quantise + append store, one launch per
// layer; and the prefill-side decision extraction.
//
// Work per layer is tiny (batch * kv_heads rows of head_dim elements), so the kernel is launch
// bound: one warp owns one (sequence, KV head) pair, lanes stride over the half head dimension.
// All float32 arithmetic is written with explicitly rounded intrinsics so that the compiler cannot
// contract a*b-c*d into fused multiply-adds: results are bit-identical to an unfused float32
// evaluation followed by a rounding to the activation dtype.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace fdms {

namespace {
thread_local char g_error[512] = {0};
}

int32_t fail(int32_t code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}
void clear_error() { g_error[0] = 0; }

struct StoreParams {
    void* q; int64_t q_sb, q_sh;
    void* k; int64_t k_sb, k_sh;
    const void* v; int64_t v_sb, v_sh;
    int act_dtype;
    const float* cos_sin; int64_t cs_stride; int64_t cs_rows;
    const int64_t* positions;
    void* k_pool; void* v_pool; int kv_dtype; int64_t pool_rows;
    const int32_t* slot; int64_t slot_sb;
    uint8_t* evict; int64_t evict_sb;
    const float* k_scale; const float* v_scale;
    int batch, hq, hk, dim;
    DecisionRule rule;
    int do_decision, do_rope, store_q, store_k;
    int32_t* dev_status;
};

// Latency matters more than bandwidth here (a few KB per launch), so the kernel is written as two
// dependent rounds of global loads: [positions, slot, every q/k/v element this lane owns] and then
// [cos/sin of the position]; everything is in registers before the first store.
// NP = pairs (i, i + half) per lane, i.e. head_dim <= 64 * NP; MAXG = q heads per KV head.
template <int NP, int MAXG>
__global__ void store_decode_kernel(StoreParams p) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= p.batch * p.hk) return;
    const int b = warp / p.hk;
    const int h = warp - b * p.hk;
    const int group = p.hq / p.hk;
    const int half = p.dim >> 1;
    const int adt = p.act_dtype;

    const int64_t q0 = (int64_t)b * p.q_sb + (int64_t)(h * group) * p.q_sh;
    const int64_t k0 = (int64_t)b * p.k_sb + (int64_t)h * p.k_sh;
    const int64_t v0 = (int64_t)b * p.v_sb + (int64_t)h * p.v_sh;
    const bool rot_q = p.do_rope && p.store_q;

    // ---- phase 1: independent loads ----
    int64_t pos = p.do_rope ? p.positions[b] : 0;
    if (pos < 0 || (p.do_rope && pos >= p.cs_rows)) {           // positions index the cos/sin table: checked, not trusted
        if (lane == 0 && p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
        pos = 0;
    }
    const int32_t slot = p.slot ? p.slot[(int64_t)b * p.slot_sb + h] : -1;
    const float dv = p.do_decision ? load_as_float(p.q, q0 + p.dim - 1, adt) : 0.0f;
    const float ks = p.k_scale ? p.k_scale[h] : 1.0f;
    const float vs = p.v_scale ? p.v_scale[h] : 1.0f;
    float kx[NP][2], vx[NP][2], qx[MAXG][NP][2];
#pragma unroll
    for (int n = 0; n < NP; ++n) {
        const int i = lane + 32 * n;
        const bool in = i < half;
        kx[n][0] = in ? load_as_float(p.k, k0 + i, adt) : 0.0f;
        kx[n][1] = in ? load_as_float(p.k, k0 + half + i, adt) : 0.0f;
        vx[n][0] = in ? load_as_float(p.v, v0 + i, adt) : 0.0f;
        vx[n][1] = in ? load_as_float(p.v, v0 + half + i, adt) : 0.0f;
#pragma unroll
        for (int g = 0; g < MAXG; ++g) {
            const bool qin = in && rot_q && g < group;
            qx[g][n][0] = qin ? load_as_float(p.q, q0 + (int64_t)g * p.q_sh + i, adt) : 0.0f;
            qx[g][n][1] = qin ? load_as_float(p.q, q0 + (int64_t)g * p.q_sh + half + i, adt) : 0.0f;
        }
    }
    // ---- phase 2: cos / sin of this sequence's position ----
    float cs[NP][2];
#pragma unroll
    for (int n = 0; n < NP; ++n) {
        const int i = lane + 32 * n;
        const bool in = p.do_rope && i < half;
        cs[n][0] = in ? p.cos_sin[pos * p.cs_stride + i] : 1.0f;
        cs[n][1] = in ? p.cos_sin[pos * p.cs_stride + half + i] : 0.0f;
    }

    if (p.do_decision && lane == 0) {
        if (p.evict) p.evict[(int64_t)b * p.evict_sb + h] = p.rule.evict(dv) ? 1 : 0;
        // Without RoPE write-back of q the lane is cleared in place only for plain extraction.
        if (!p.do_rope) store_from_float(p.q, q0 + p.dim - 1, adt, 0.0f);
    }
    bool do_store = slot >= 0;
    if (do_store && (int64_t)slot >= p.pool_rows) {
        if (lane == 0 && p.dev_status) atomicOr(p.dev_status, FDMS_DEV_BAD_INDEX);
        do_store = false;
    }
    const int64_t row = (int64_t)slot * p.dim;
#pragma unroll
    for (int n = 0; n < NP; ++n) {
        const int i = lane + 32 * n;
        if (i >= half) continue;
        const float c = cs[n][0], sn = cs[n][1];
        if (rot_q) {
#pragma unroll
            for (int g = 0; g < MAXG; ++g) {
                if (g >= group) break;
                const float x1 = qx[g][n][0];
                float x2 = qx[g][n][1];
                if (p.do_decision && g == 0 && i == half - 1) x2 = 0.0f;     // the borrowed decision channel
                const int64_t qo = q0 + (int64_t)g * p.q_sh;
                store_from_float(p.q, qo + i, adt, __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn)));
                store_from_float(p.q, qo + half + i, adt, __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn)));
            }
        }
        float y1 = kx[n][0], y2 = kx[n][1];
        if (p.do_rope) {
            y1 = round_to_dtype(__fsub_rn(__fmul_rn(kx[n][0], c), __fmul_rn(kx[n][1], sn)), adt);
            y2 = round_to_dtype(__fadd_rn(__fmul_rn(kx[n][1], c), __fmul_rn(kx[n][0], sn)), adt);
            if (p.store_k) {
                store_from_float(p.k, k0 + i, adt, y1);
                store_from_float(p.k, k0 + half + i, adt, y2);
            }
        }
        if (do_store) {
            if (p.k_scale) { y1 = __fdiv_rn(y1, ks); y2 = __fdiv_rn(y2, ks); }
            store_from_float(p.k_pool, row + i, p.kv_dtype, y1);
            store_from_float(p.k_pool, row + half + i, p.kv_dtype, y2);
            store_from_float(p.v_pool, row + i, p.kv_dtype, p.v_scale ? __fdiv_rn(vx[n][0], vs) : vx[n][0]);
            store_from_float(p.v_pool, row + half + i, p.kv_dtype, p.v_scale ? __fdiv_rn(vx[n][1], vs) : vx[n][1]);
        }
    }
}

__global__ void extract_decisions_kernel(void* q, int q_dtype, int64_t q_st, int64_t q_sh,
                                         uint8_t* evict, int64_t ev_st, int64_t total, int hk, int group,
                                         int dim, DecisionRule rule) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int64_t t = i / hk;
    const int h = (int)(i - t * hk);
    const int64_t off = t * q_st + (int64_t)(h * group) * q_sh + (dim - 1);
    const float v = load_as_float(q, off, q_dtype);
    evict[t * ev_st + h] = rule.evict(v) ? 1 : 0;
    store_from_float(q, off, q_dtype, 0.0f);
}

}  // namespace fdms

using namespace fdms;

extern "C" int32_t fdms_abi_version(void) { return FDMS_ABI_VERSION; }
extern "C" const char* fdms_last_error(void) { return g_error; }

extern "C" int32_t fdms_store_decode(
    void* q, int64_t q_stride_b, int64_t q_stride_h,
    void* k, int64_t k_stride_b, int64_t k_stride_h,
    const void* v, int64_t v_stride_b, int64_t v_stride_h, int32_t act_dtype,
    const float* cos_sin, int64_t cos_sin_stride, int64_t cos_sin_rows, const int64_t* positions,
    void* k_pool, void* v_pool, int32_t kv_dtype, int64_t pool_rows,
    const int32_t* slot_mapping, int64_t slot_stride_b,
    uint8_t* evict_out, int64_t evict_stride_b,
    const float* k_scale, const float* v_scale,
    int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
    double alpha_scale, double alpha_offset,
    int32_t do_decision, int32_t do_rope, int32_t store_q, int32_t store_k,
    int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(batch >= 0 && num_q_heads > 0 && num_kv_heads > 0 && head_dim > 0, FDMS_E_ARG,
                 "fdms_store_decode: bad sizes batch=%d q_heads=%d kv_heads=%d head_dim=%d", batch,
                 num_q_heads, num_kv_heads, head_dim);
    FDMS_REQUIRE(num_q_heads % num_kv_heads == 0, FDMS_E_ARG,
                 "q_heads=%d must be divisible by kv_heads=%d", num_q_heads, num_kv_heads);
    FDMS_REQUIRE(head_dim % 2 == 0, FDMS_E_ARG, "RoPE head_dim must be even, got %d", head_dim);
    FDMS_REQUIRE(act_dtype == FDMS_F32 || act_dtype == FDMS_BF16 || act_dtype == FDMS_F16, FDMS_E_DTYPE,
                 "fdms_store_decode: activation dtype %d not supported", act_dtype);
    FDMS_REQUIRE(kv_dtype >= FDMS_F32 && kv_dtype <= FDMS_E4M3, FDMS_E_DTYPE,
                 "fdms_store_decode: pool dtype %d not supported", kv_dtype);
    FDMS_REQUIRE(k && v, FDMS_E_ARG, "fdms_store_decode: k and v are required");
    FDMS_REQUIRE(!(do_decision || (do_rope && store_q)) || q, FDMS_E_ARG, "fdms_store_decode: q is required");
    FDMS_REQUIRE(!do_rope || cos_sin_rows > 0, FDMS_E_ARG, "fdms_store_decode: cos_sin_rows must be positive");
    FDMS_REQUIRE(!do_rope || (cos_sin && positions), FDMS_E_ARG,
                 "fdms_store_decode: RoPE needs cos_sin and positions");
    FDMS_REQUIRE(!slot_mapping || (k_pool && v_pool), FDMS_E_ARG, "fdms_store_decode: pools are required");
    FDMS_REQUIRE(alpha_scale != 0.0 || !do_decision, FDMS_E_ARG, "alpha_scale must be non-zero");
    if (batch == 0) return FDMS_OK;
    StoreParams p;
    p.q = q; p.q_sb = q_stride_b; p.q_sh = q_stride_h;
    p.k = k; p.k_sb = k_stride_b; p.k_sh = k_stride_h;
    p.v = v; p.v_sb = v_stride_b; p.v_sh = v_stride_h;
    p.act_dtype = act_dtype;
    p.cos_sin = cos_sin; p.cs_stride = cos_sin_stride; p.cs_rows = cos_sin_rows; p.positions = positions;
    p.k_pool = k_pool; p.v_pool = v_pool; p.kv_dtype = kv_dtype; p.pool_rows = pool_rows;
    p.slot = slot_mapping; p.slot_sb = slot_stride_b;
    p.evict = evict_out; p.evict_sb = evict_stride_b;
    p.k_scale = k_scale; p.v_scale = v_scale;
    p.batch = batch; p.hq = num_q_heads; p.hk = num_kv_heads; p.dim = head_dim;
    p.rule = make_rule(do_decision ? alpha_scale : 1.0, alpha_offset);
    p.do_decision = do_decision; p.do_rope = do_rope; p.store_q = store_q; p.store_k = store_k;
    p.dev_status = dev_status;
    const int warps = batch * num_kv_heads;
    const int threads = 128;
    const int blocks = (warps * 32 + threads - 1) / threads;
    const int group = num_q_heads / num_kv_heads;
    FDMS_REQUIRE(head_dim <= 256, FDMS_E_CAPACITY, "head_dim=%d is above the fused decode preprocess kernel limit", head_dim);
    FDMS_REQUIRE(group <= 16 || !(do_rope && store_q), FDMS_E_CAPACITY,
                 "group_size=%d is above the fused decode preprocess limit of 16", group);
    if (head_dim <= 128 && group <= 4)
        store_decode_kernel<2, 4><<<blocks, threads, 0, (cudaStream_t)stream>>>(p);
    else if (head_dim <= 128 && group <= 8)
        store_decode_kernel<2, 8><<<blocks, threads, 0, (cudaStream_t)stream>>>(p);
    else
        store_decode_kernel<4, 16><<<blocks, threads, 0, (cudaStream_t)stream>>>(p);
    FDMS_CHECK_LAUNCH("store_decode_kernel");
    return FDMS_OK;
}

extern "C" int32_t fdms_extract_decisions(
    void* q, int32_t q_dtype, int64_t q_stride_t, int64_t q_stride_h,
    uint8_t* evict_out, int64_t evict_stride_t,
    int64_t tokens, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
    double alpha_scale, double alpha_offset, void* stream) {
    clear_error();
    FDMS_REQUIRE(q && evict_out, FDMS_E_ARG, "fdms_extract_decisions: null pointer");
    FDMS_REQUIRE(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, FDMS_E_ARG,
                 "num_qo_heads=%d must be divisible by num_kv_heads=%d", num_q_heads, num_kv_heads);
    FDMS_REQUIRE(q_dtype == FDMS_F32 || q_dtype == FDMS_BF16 || q_dtype == FDMS_F16, FDMS_E_DTYPE,
                 "fdms_extract_decisions: dtype %d not supported", q_dtype);
    FDMS_REQUIRE(alpha_scale != 0.0, FDMS_E_ARG, "alpha_scale must be non-zero");
    const int64_t total = tokens * num_kv_heads;
    if (total <= 0) return FDMS_OK;
    const int threads = 256;
    const int64_t blocks = (total + threads - 1) / threads;
    extract_decisions_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
        q, q_dtype, q_stride_t, q_stride_h, evict_out, evict_stride_t, total, num_kv_heads,
        num_q_heads / num_kv_heads, head_dim, make_rule(alpha_scale, alpha_offset));
    FDMS_CHECK_LAUNCH("extract_decisions_kernel");
    return FDMS_OK;
}

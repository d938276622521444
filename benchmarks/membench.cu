// Memory-path microbenchmarks behind the design of the decode attention kernels: what one B200 delivers for
// the access patterns the kernels can choose between, with no math in the way.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o membench benchmarks/membench.cu && ./membench
//
// A  streaming read of 1 GiB, 16 bytes per lane
// B  random 16-row pages read straight into registers (1 KiB, 2 KiB, 4 KiB and 512-byte chunks; a 1 KiB K
//    page plus a 1 KiB V page from two pools, as the compact pool is laid out)
// C  the same pages brought into a per-warp shared-memory ring with bulk asynchronous copies
// D  sixteen 10.5 MB regions read by sixteen chained launches (ordinary / programmatic dependent launch,
//    with and without prefetching the next region into L2)
// E  the period of a chain of minimal dependent launches
// F  chained launches whose CTAs bring their whole slice into shared memory before the dependency on the
//    preceding launch is resolved
// Every mbarrier wait is bounded; a wait that runs out sets the error flag printed at the end.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#include <algorithm>
#include <random>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(1); } } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(20000) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < 20000; ++i) if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- A: streaming read
__global__ void __launch_bounds__(256) stream_read(const uint4* __restrict__ p, size_t n16, uint32_t* sink) {
    uint32_t acc = 0;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i + 3 * stride < n16; i += 4 * stride) {
        uint4 a = __ldcs(p + i), b = __ldcs(p + i + stride), c = __ldcs(p + i + 2 * stride), d = __ldcs(p + i + 3 * stride);
        acc ^= a.x ^ b.y ^ c.z ^ d.w;
    }
    for (; i < n16; i += stride) acc ^= __ldcs(p + i).x;
    if (acc == 0x12345678u) *sink = acc;
}

// ---------------------------------------------------------------- B: random chunks, direct loads
// mode 0: chunk = CH bytes contiguous at perm[i]*CH in pool K.  mode 1: CH/2 from K and CH/2 from V at perm[i]*(CH/2).
template <int CH, int U>
__global__ void __launch_bounds__(256, 2) chunk_read_direct(const uint8_t* __restrict__ K, const uint8_t* __restrict__ V,
                                                            const int32_t* __restrict__ perm, int nchunks, int mode, uint32_t* sink) {
    const int lane = threadIdx.x & 31;
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int nw = (gridDim.x * blockDim.x) >> 5;
    constexpr int V16 = CH / 512;          // uint4 per lane per chunk
    uint32_t acc = 0;
    for (int c0 = gw; c0 < nchunks; c0 += nw * U) {
        uint4 buf[U][V16];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + u * nw;
            if (c < nchunks) {
                const int64_t id = perm[c];
#pragma unroll
                for (int j = 0; j < V16; ++j) {
                    const uint8_t* src;
                    if (mode == 0) src = K + id * CH + j * 512 + lane * 16;
                    else src = (j < V16 / 2 ? K + id * (CH / 2) + j * 512 : V + id * (CH / 2) + (j - V16 / 2) * 512) + lane * 16;
                    buf[u][j] = __ldcs((const uint4*)src);
                }
            } else {
#pragma unroll
                for (int j = 0; j < V16; ++j) buf[u][j] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int j = 0; j < V16; ++j) acc ^= buf[u][j].x ^ buf[u][j].w;
    }
    if (acc == 0x12345678u) *sink = acc;
}

// ---------------------------------------------------------------- C: random chunks, bulk copies into a per-warp ring
// Each warp owns R slots of CH bytes.  issue_mode 0: lane 0 issues; 1: lane (slot) issues its own slot.
template <int CH>
__global__ void __launch_bounds__(256, 2) chunk_read_bulk(const uint8_t* __restrict__ K, const uint8_t* __restrict__ V,
                                                          const int32_t* __restrict__ perm, int nchunks, int mode, int R,
                                                          int issue_mode, uint32_t* sink, int* err) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int nw = (gridDim.x * blockDim.x) >> 5;
    uint8_t* ring = smem + (size_t)warp * R * CH;
    uint64_t* bars = (uint64_t*)(smem + (size_t)8 * R * CH) + warp * R;
    if (lane < R) mbar_init(&bars[lane], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
    const int mine = gw < nchunks ? (nchunks - gw + nw - 1) / nw : 0;
    auto issue = [&](int i) {          // i-th chunk of this warp into slot i % R (called by one lane)
        const int s = i % R;
        const int64_t id = perm[gw + i * nw];
        mbar_expect_tx(&bars[s], CH);
        if (mode == 0) bulk_g2s(ring + s * CH, K + id * CH, CH, &bars[s]);
        else {
            bulk_g2s(ring + s * CH, K + id * (CH / 2), CH / 2, &bars[s]);
            bulk_g2s(ring + s * CH + CH / 2, V + id * (CH / 2), CH / 2, &bars[s]);
        }
    };
    if (issue_mode == 0) { if (lane == 0) for (int i = 0; i < R && i < mine; ++i) issue(i); }
    else { if (lane < R && lane < mine) issue(lane); }
    uint32_t acc = 0;
    for (int i = 0; i < mine; ++i) {
        const int s = i % R;
        if (!mbar_wait(&bars[s], (i / R) & 1)) { if (lane == 0) atomicExch(err, 1); break; }
        acc ^= *(const uint32_t*)(ring + s * CH + lane * 16);
        __syncwarp();
        if (i + R < mine && lane == 0) issue(i + R);
    }
    if (acc == 0x12345678u) *sink = acc;
}

// ---------------------------------------------------------------- D: read region (direct) + prefetch next region into L2
template <int U>
__global__ void __launch_bounds__(256, 2) read_prefetch(const uint8_t* __restrict__ K, const uint8_t* __restrict__ V,
                                                        const int32_t* __restrict__ perm, int nchunks,
                                                        const uint8_t* __restrict__ Kn, const uint8_t* __restrict__ Vn,
                                                        const int32_t* __restrict__ permn, int do_prefetch, int pdl,
                                                        const uint32_t* dep, uint32_t* sink) {
    const int lane = threadIdx.x & 31;
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int nw = (gridDim.x * blockDim.x) >> 5;
    if (pdl) pdl_trigger();
    if (do_prefetch) {
        // one lane per chunk: 1 KiB of K and 1 KiB of V
        for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < nchunks; c += gridDim.x * blockDim.x) {
            const int64_t id = permn[c];
            bulk_prefetch_l2(Kn + id * 1024, 1024);
            bulk_prefetch_l2(Vn + id * 1024, 1024);
        }
    }
    uint32_t acc = 0;
    for (int c0 = gw; c0 < nchunks; c0 += nw * U) {
        uint4 buf[U][4];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + u * nw;
            if (c < nchunks) {
                const int64_t id = perm[c];
                buf[u][0] = __ldcs((const uint4*)(K + id * 1024 + lane * 16));
                buf[u][1] = __ldcs((const uint4*)(K + id * 1024 + 512 + lane * 16));
                buf[u][2] = __ldcs((const uint4*)(V + id * 1024 + lane * 16));
                buf[u][3] = __ldcs((const uint4*)(V + id * 1024 + 512 + lane * 16));
            } else {
                buf[u][0] = buf[u][1] = buf[u][2] = buf[u][3] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) acc ^= buf[u][0].x ^ buf[u][1].y ^ buf[u][2].z ^ buf[u][3].w;
    }
    if (pdl) pdl_wait();
    if (threadIdx.x == 0) acc ^= dep[blockIdx.x & 63];
    if (acc == 0x12345678u) *sink = acc;
    if (threadIdx.x == 0) sink[1 + (blockIdx.x & 63)] = acc | 1u;
}

// ---------------------------------------------------------------- E: minimal dependent kernel
__global__ void __launch_bounds__(256) pdl_min(const uint32_t* in, uint32_t* out, int pdl) {
    if (pdl) { pdl_trigger(); pdl_wait(); }
    if (threadIdx.x == 0) out[blockIdx.x] = in[blockIdx.x] + 1;
}

// ---------------------------------------------------------------- F: pre-wait bulk load of the CTA's whole slice into smem
// CTA b of a launch owns chunks [b*per, (b+1)*per) of the launch's permutation; chunk = 1 KiB K + 1 KiB V (mode 1) or 2 KiB (mode 0).
__global__ void __launch_bounds__(256, 2) pdl_slice(const uint8_t* __restrict__ K, const uint8_t* __restrict__ V,
                                                    const int32_t* __restrict__ perm, int per, int mode, int pdl,
                                                    const uint32_t* dep_in, uint32_t* dep_out, int* err) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint64_t* bars = (uint64_t*)(smem + (size_t)per * 2048);
    if (pdl) pdl_trigger();
    if (threadIdx.x < 8) mbar_init(&bars[threadIdx.x], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    // warp w owns chunks w, w+8, ...; lane i issues chunk w + 8 i
    const int nmine = warp < per ? (per - warp + 7) / 8 : 0;
    if (lane == 0 && nmine > 0) mbar_expect_tx(&bars[warp], (uint32_t)nmine * 2048);
    __syncwarp();
    for (int i = lane; i < nmine; i += 32) {
        const int c = warp + 8 * i;
        const int64_t id = perm[(size_t)blockIdx.x * per + c];
        if (mode == 0) bulk_g2s(smem + (size_t)c * 2048, K + id * 2048, 2048, &bars[warp]);
        else {
            bulk_g2s(smem + (size_t)c * 2048, K + id * 1024, 1024, &bars[warp]);
            bulk_g2s(smem + (size_t)c * 2048 + 1024, V + id * 1024, 1024, &bars[warp]);
        }
    }
    if (pdl) pdl_wait();
    uint32_t acc = dep_in[blockIdx.x];
    if (nmine > 0 && !mbar_wait(&bars[warp], 0)) { if (lane == 0) atomicExch(err, 2); }
    for (int i = 0; i < nmine; ++i) acc ^= *(const uint32_t*)(smem + (size_t)(warp + 8 * i) * 2048 + lane * 16);
    acc = __reduce_xor_sync(0xffffffffu, acc);
    if (threadIdx.x == 0) dep_out[blockIdx.x] = acc;
}

// ================================================================ host
static float time_graph(cudaGraphExec_t g, cudaStream_t s, int reps) {
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int i = 0; i < 3; ++i) CK(cudaGraphLaunch(g, s));
    CK(cudaStreamSynchronize(s));
    CK(cudaEventRecord(e0, s));
    for (int i = 0; i < reps; ++i) CK(cudaGraphLaunch(g, s));
    CK(cudaEventRecord(e1, s));
    CK(cudaStreamSynchronize(s));
    float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
    return ms / reps;
}

template <typename F>
static float capture_and_time(cudaStream_t s, int reps, F enqueue) {
    cudaGraph_t g; cudaGraphExec_t ge;
    CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    enqueue();
    CK(cudaStreamEndCapture(s, &g));
    CK(cudaGraphInstantiate(&ge, g, 0));
    float ms = time_graph(ge, s, reps);
    CK(cudaGraphExecDestroy(ge)); CK(cudaGraphDestroy(g));
    return ms;
}

template <typename K, typename... A>
static void launch(K kern, dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl, A... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;
    CK(cudaLaunchKernelEx(&cfg, kern, args...));
}

int main() {
    CK(cudaSetDevice(0));
    cudaStream_t s; CK(cudaStreamCreate(&s));
    const size_t POOL = (size_t)1 << 30;            // 1 GiB K, 1 GiB V
    uint8_t *K, *V; CK(cudaMalloc(&K, POOL)); CK(cudaMalloc(&V, POOL));
    CK(cudaMemset(K, 1, POOL)); CK(cudaMemset(V, 2, POOL));
    uint32_t* sink; CK(cudaMalloc(&sink, 4096)); CK(cudaMemset(sink, 0, 4096));
    int* err; CK(cudaMalloc(&err, 4)); CK(cudaMemset(err, 0, 4));
    std::mt19937 rng(1);

    // ---- A
    {
        float ms = capture_and_time(s, 10, [&] { stream_read<<<148 * 8, 256, 0, s>>>((const uint4*)K, POOL / 16, sink); });
        printf("A stream_read 1GiB: %.1f GB/s\n", POOL / ms / 1e6);
    }
    // permutations of chunk ids for several chunk sizes (over the 1 GiB pool)
    auto make_perm = [&](size_t n) {
        std::vector<int32_t> p(n);
        for (size_t i = 0; i < n; ++i) p[i] = (int32_t)i;
        std::shuffle(p.begin(), p.end(), rng);
        int32_t* d; CK(cudaMalloc(&d, n * 4));
        CK(cudaMemcpy(d, p.data(), n * 4, cudaMemcpyHostToDevice));
        return d;
    };
    int32_t* perm512 = make_perm(POOL / 512);
    int32_t* perm1k = make_perm(POOL / 1024);
    int32_t* perm2k = make_perm(POOL / 2048);
    int32_t* perm4k = make_perm(POOL / 4096);
    // ---- B: direct, total bytes read 1 GiB each
    {
        const int grid = 148 * 2;
        float ms;
        ms = capture_and_time(s, 10, [&] { chunk_read_direct<1024, 6><<<grid, 256, 0, s>>>(K, V, perm1k, (int)(POOL / 1024), 0, sink); });
        printf("B direct 1KiB contiguous U=6: %.1f GB/s\n", POOL / ms / 1e6);
        ms = capture_and_time(s, 10, [&] { chunk_read_direct<2048, 3><<<grid, 256, 0, s>>>(K, V, perm2k, (int)(POOL / 2048), 0, sink); });
        printf("B direct 2KiB contiguous U=3: %.1f GB/s\n", POOL / ms / 1e6);
        ms = capture_and_time(s, 10, [&] { chunk_read_direct<2048, 3><<<grid, 256, 0, s>>>(K, V, perm1k, (int)(POOL / 2048), 1, sink); });
        printf("B direct 1KiB K + 1KiB V (same id) U=3: %.1f GB/s\n", POOL / ms / 1e6);
        ms = capture_and_time(s, 10, [&] { chunk_read_direct<4096, 2><<<grid, 256, 0, s>>>(K, V, perm4k, (int)(POOL / 4096), 0, sink); });
        printf("B direct 4KiB contiguous U=2: %.1f GB/s\n", POOL / ms / 1e6);
        ms = capture_and_time(s, 10, [&] { chunk_read_direct<2048, 6><<<148, 256, 0, s>>>(K, V, perm1k, (int)(POOL / 2048), 1, sink); });
        printf("B direct 1KiB K + 1KiB V U=6, 1 CTA/SM: %.1f GB/s\n", POOL / ms / 1e6);
        ms = capture_and_time(s, 10, [&] { chunk_read_direct<512, 8><<<grid, 256, 0, s>>>(K, V, perm512, (int)(POOL / 512), 0, sink); });
        printf("B direct 512B contiguous U=8: %.1f GB/s\n", POOL / ms / 1e6);
    }
    // ---- C: bulk ring
    {
        const int grid = 148 * 2;
        for (int issue_mode = 0; issue_mode < 2; ++issue_mode) {
            for (int R : {4, 6}) {
                size_t smem2k = (size_t)8 * R * 2048 + 8 * R * 8 + 64;
                CK(cudaFuncSetAttribute(chunk_read_bulk<2048>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2k));
                float ms = capture_and_time(s, 10, [&] { chunk_read_bulk<2048><<<grid, 256, smem2k, s>>>(K, V, perm2k, (int)(POOL / 2048), 0, R, issue_mode, sink, err); });
                printf("C bulk 2KiB contiguous R=%d issue=%d: %.1f GB/s\n", R, issue_mode, POOL / ms / 1e6);
                ms = capture_and_time(s, 10, [&] { chunk_read_bulk<2048><<<grid, 256, smem2k, s>>>(K, V, perm1k, (int)(POOL / 2048), 1, R, issue_mode, sink, err); });
                printf("C bulk 1KiB K + 1KiB V R=%d issue=%d: %.1f GB/s\n", R, issue_mode, POOL / ms / 1e6);
            }
            int R = 3;
            size_t smem4k = (size_t)8 * R * 4096 + 8 * R * 8 + 64;
            CK(cudaFuncSetAttribute(chunk_read_bulk<4096>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4k));
            float ms = capture_and_time(s, 10, [&] { chunk_read_bulk<4096><<<grid, 256, smem4k, s>>>(K, V, perm4k, (int)(POOL / 4096), 0, R, issue_mode, sink, err); });
            printf("C bulk 4KiB contiguous R=%d issue=%d: %.1f GB/s\n", R, issue_mode, POOL / ms / 1e6);
        }
    }
    // ---- D: 16 regions of 5120 chunk pairs (10.5 MB) each, chained
    const int NL = 16, NCH = 5120;
    {
        // region l uses chunk ids perm1k[l*NCH .. ) (random places in the 1 GiB pools)
        for (int pdl = 0; pdl < 2; ++pdl)
            for (int pf = 0; pf < 2; ++pf)
                for (int grid : {128, 256}) {
                    float ms = capture_and_time(s, 30, [&] {
                        for (int l = 0; l < NL; ++l) {
                            const int ln = (l + 1) % NL;
                            launch(read_prefetch<3>, dim3(grid), dim3(256), 0, s, pdl && l > 0, (const uint8_t*)K, (const uint8_t*)V,
                                   (const int32_t*)(perm1k + (size_t)l * NCH), NCH, (const uint8_t*)K, (const uint8_t*)V,
                                   (const int32_t*)(perm1k + (size_t)ln * NCH), pf, pdl, (const uint32_t*)(sink + 1), sink + 128);
                        }
                    });
                    const double bytes = (double)NCH * 2048;
                    printf("D read 10.5MB region direct, grid=%d prefetch_next=%d pdl=%d: %.2f us/launch -> %.1f GB/s\n", grid, pf, pdl,
                           ms * 1e3 / NL, bytes / (ms * 1e-3 / NL) / 1e9);
                }
    }
    // ---- E: PDL floor
    {
        uint32_t* buf; CK(cudaMalloc(&buf, 17 * 1024 * 4)); CK(cudaMemset(buf, 0, 17 * 1024 * 4));
        for (int pdl = 0; pdl < 2; ++pdl) {
            float ms = capture_and_time(s, 50, [&] {
                for (int l = 0; l < NL; ++l)
                    launch(pdl_min, dim3(128), dim3(256), 0, s, pdl && l > 0, (const uint32_t*)(buf + l * 1024), buf + (l + 1) * 1024, pdl);
            });
            printf("E minimal dependent kernel chain, pdl=%d: %.2f us/launch\n", pdl, ms * 1e3 / NL);
        }
    }
    // ---- F: pre-wait whole-slice bulk load
    {
        uint32_t* dep; CK(cudaMalloc(&dep, 17 * 1024 * 4)); CK(cudaMemset(dep, 0, 17 * 1024 * 4));
        CK(cudaFuncSetAttribute(pdl_slice, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        for (int pdl = 0; pdl < 2; ++pdl)
            for (int mode = 0; mode < 2; ++mode)
                for (int grid : {128, 256}) {
                    const int per = NCH / grid;
                    const size_t smem = (size_t)per * 2048 + 64;
                    float ms = capture_and_time(s, 30, [&] {
                        for (int l = 0; l < NL; ++l)
                            launch(pdl_slice, dim3(grid), dim3(256), smem, s, pdl && l > 0, (const uint8_t*)K, (const uint8_t*)V,
                                   (const int32_t*)((mode == 0 ? perm2k : perm1k) + (size_t)l * NCH), per, mode, pdl,
                                   (const uint32_t*)(dep + l * 1024), dep + (l + 1) * 1024, err);
                    });
                    const double bytes = (double)NCH * 2048;
                    printf("F whole-slice bulk into smem, grid=%d (%d KB/CTA) %s pdl=%d: %.2f us/launch -> %.1f GB/s\n", grid, per * 2,
                           mode == 0 ? "2KiB pages" : "1KiB K + 1KiB V", pdl, ms * 1e3 / NL, bytes / (ms * 1e-3 / NL) / 1e9);
                }
    }
    int herr = 0; CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
    printf("err flag: %d\n", herr);
    CK(cudaDeviceSynchronize());
    return 0;
}

// One-shot all-reduce over NVLink peer memory for the small tensors of tensor-parallel decode
// ([batch, hidden] after o_proj and down_proj: 64 KB at batch 8, hidden 4096; the reference calls
// NCCL's all_reduce there, fastdms/layers/linear.py:1044-1048).  At this size an all-reduce is pure
// latency, so the exchange is one NVLink traversal: every rank PUSHES its input into a slot of every
// peer's region, each 32-bit word next to the call's epoch (16-byte stores {word, epoch, word, epoch} whose
// 8-byte halves arrive whole), then reads the slots the peers pushed into its OWN memory, waiting (bounded)
// for the words whose epoch does not match yet, and adds all inputs in rank order (the same order on every
// rank: all ranks get identical bits).  No fence, no flag, no load from a peer.
//
// Memory, per rank, all in one peer-mapped allocation:
//   slots[2][world][2 * max_bytes]   two halves used alternately by consecutive calls; slot (half, r) holds
//                                    what rank r pushed, as (word, epoch) pairs
//   epoch[kArCtas]                   this rank's call counter, one per CTA (kept on the device so that a
//                                    captured CUDA graph can replay the call); the region starts zeroed
// A rank can be at most one call ahead of a peer (to start call e + 2 it has finished call e + 1, for which it
// needed the peer's words of call e + 1, which the peer pushes only after it has finished reading call e), so
// two halves are enough and a stale slot carries epoch e - 2.
// Every wait is bounded: after kArSpinLimit polls of a word the CTA raises FDMS_DEV_WAIT_TIMEOUT in the status
// word, leaves the silent peer out and returns, so a missing peer costs seconds, not a hang.  After a timeout
// the ranks' epochs may disagree: the bit is fatal for the region, which must be re-created collectively.
#include <string.h>

#include "common.cuh"

namespace fdms {

constexpr int kArCtas = 8;                 // CTAs per call, fixed: part of the epoch layout
constexpr int kArThreads = 256;
constexpr int kArMaxWorld = 8;
constexpr unsigned kArSpinLimit = 1u << 20;       // polls of one word: about a second

struct ArParams {
    uint8_t* slots[kArMaxWorld];           // peers' regions (index = rank)
    uint32_t* epoch;                       // local, [kArCtas]
    const void* in; void* out;
    int64_t n; int dtype; int rank, world; int64_t max_bytes;     // max_bytes rounded up to 256
    int32_t* dev_status;
};

__device__ __forceinline__ void st_pair16(void* p, uint32_t a, uint32_t b, uint32_t e) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(e), "r"(b), "r"(e) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void accumulate16(const uint4& v, int dt, float (&acc)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    if (dt == FDMS_F32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] += __uint_as_float(w[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (dt == FDMS_BF16) {
                acc[2 * i] += __uint_as_float(w[i] << 16);
                acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            } else {
                const __half2 h = *(const __half2*)&w[i];
                acc[2 * i] += __low2float(h);
                acc[2 * i + 1] += __high2float(h);
            }
        }
    }
}

// Byte offset of slot (half, source rank) inside a region.
__device__ __forceinline__ int64_t ar_slot(int half, int src, int world, int64_t max_bytes) {
    return ((int64_t)half * world + src) * 2 * max_bytes;
}

__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(ArParams p) {
    __shared__ volatile int s_missing[kArMaxWorld];
    const int c = blockIdx.x, tid = threadIdx.x;
    const int esz = p.dtype == FDMS_F32 ? 4 : 2;
    const int64_t bytes = p.n * esz;
    const int64_t vecs = bytes >> 4;                                   // 16-byte vectors in the tensor
    const int64_t per = (vecs + kArCtas - 1) / kArCtas;
    const int64_t v0 = (int64_t)c * per, v1 = min(vecs, v0 + per);
    const uint32_t e = p.epoch[c] + 1;
    const int half = (int)(e & 1u);
    if (tid < kArMaxWorld) s_missing[tid] = 0;
    __syncthreads();
    // push this rank's chunk to every peer: vector i becomes two 16-byte (word, epoch) stores at 32 * i
    for (int64_t i = v0 + tid; i < v1; i += kArThreads) {
        const uint4 v = ((const uint4*)p.in)[i];
        for (int r = 0; r < p.world; ++r) {
            if (r == p.rank) continue;
            uint8_t* dst = p.slots[r] + ar_slot(half, p.rank, p.world, p.max_bytes) + (i << 5);
            st_pair16(dst, v.x, v.y, e);
            st_pair16(dst + 16, v.z, v.w, e);
        }
    }
    // sum in rank order: own input from `in`, the peers' from this rank's region
    const uint8_t* mine = p.slots[p.rank];
    for (int64_t i = v0 + tid; i < v1; i += kArThreads) {
        uint4 lo[kArMaxWorld], hi[kArMaxWorld];
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r) {
            if (r < p.world && r != p.rank) {
                const uint8_t* src = mine + ar_slot(half, r, p.world, p.max_bytes) + (i << 5);
                lo[r] = ld_volatile16(src);
                hi[r] = ld_volatile16(src + 16);
            }
        }
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r) {
            if (r >= p.world) continue;
            if (r == p.rank) {
                accumulate16(((const uint4*)p.in)[i], p.dtype, acc);
                continue;
            }
            const uint8_t* src = mine + ar_slot(half, r, p.world, p.max_bytes) + (i << 5);
            unsigned spins = 0;
            while (lo[r].y != e || lo[r].w != e || hi[r].y != e || hi[r].w != e) {
                if (s_missing[r] || ++spins >= kArSpinLimit) {
                    if (!s_missing[r]) {
                        s_missing[r] = 1;
                        if (p.dev_status) atomicOr(p.dev_status, FDMS_DEV_WAIT_TIMEOUT);
                    }
                    break;
                }
                lo[r] = ld_volatile16(src);
                hi[r] = ld_volatile16(src + 16);
            }
            if (lo[r].y != e || lo[r].w != e || hi[r].y != e || hi[r].w != e) continue;       // silent peer: left out
            accumulate16(make_uint4(lo[r].x, lo[r].z, hi[r].x, hi[r].z), p.dtype, acc);
        }
        uint4 o;
        if (p.dtype == FDMS_F32) {
            o = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
        } else {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (p.dtype == FDMS_BF16) {
                    const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                    w[j] = *(const uint32_t*)&b;
                } else {
                    const __half2 h = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
                    w[j] = *(const uint32_t*)&h;
                }
            }
            o = make_uint4(w[0], w[1], w[2], w[3]);
        }
        ((uint4*)p.out)[i] = o;
    }
    __syncthreads();
    if (tid == 0) p.epoch[c] = e;
}

}  // namespace fdms

using namespace fdms;

// Kernels of the CURRENT device will read and write memory that lives on `peer_device` (a region mapped
// through CUDA IPC): that needs peer access enabled in this direction, which mapping the region does
// not do by itself.  "Already enabled" is not an error.
extern "C" int32_t fdms_enable_peer_access(int32_t peer_device) {
    clear_error();
    int cur = -1;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess) return fail(FDMS_E_CUDA, "fdms_enable_peer_access: %s", cudaGetErrorString(e));
    if (cur == peer_device) return FDMS_OK;
    int can = 0;
    e = cudaDeviceCanAccessPeer(&can, cur, peer_device);
    if (e != cudaSuccess || !can) {
        cudaGetLastError();
        return fail(FDMS_E_CUDA, "fdms_enable_peer_access: device %d cannot access device %d", cur, peer_device);
    }
    e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return FDMS_OK; }
    if (e != cudaSuccess) return fail(FDMS_E_CUDA, "fdms_enable_peer_access: %s", cudaGetErrorString(e));
    return FDMS_OK;
}

// Peer regions.  A region must be a whole device allocation (an IPC handle names the allocation, not a
// pointer inside it) and a peer must open the handle with ITS OWN device current: the mapping that
// cudaIpcOpenMemHandle returns belongs to the address space of the device that is current at that
// moment.  (A mapping opened under the exporting device's index, as generic tensor-sharing helpers do,
// is not reachable from kernels of the importing rank's device, even with peer access enabled.)
extern "C" int32_t fdms_ipc_region_create(int64_t bytes, void** ptr, void* handle64) {
    clear_error();
    FDMS_REQUIRE(bytes > 0 && ptr && handle64, FDMS_E_ARG, "fdms_ipc_region_create: bad arguments");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e != cudaSuccess) return fail(FDMS_E_CUDA, "fdms_ipc_region_create: cudaMalloc: %s", cudaGetErrorString(e));
    e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        cudaGetLastError();
        return fail(FDMS_E_CUDA, "fdms_ipc_region_create: %s", cudaGetErrorString(e));
    }
    memcpy(handle64, &h, sizeof(h));
    *ptr = p;
    return FDMS_OK;
}

extern "C" int32_t fdms_ipc_region_open(const void* handle64, void** ptr) {
    clear_error();
    FDMS_REQUIRE(handle64 && ptr, FDMS_E_ARG, "fdms_ipc_region_open: bad arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(FDMS_E_CUDA, "fdms_ipc_region_open: %s", cudaGetErrorString(e));
    }
    // the mapping must be device memory that this device can read: checked through the runtime (a copy
    // that fails returns an error; a kernel that touched a bad mapping would fault)
    cudaPointerAttributes attr;
    cudaError_t e2 = cudaPointerGetAttributes(&attr, p);
    uint32_t probe = 0;
    if (e2 == cudaSuccess && attr.type != cudaMemoryTypeDevice) e2 = cudaErrorInvalidDevicePointer;
    if (e2 == cudaSuccess) e2 = cudaMemcpy(&probe, p, sizeof(probe), cudaMemcpyDeviceToHost);
    if (e2 != cudaSuccess) {
        cudaIpcCloseMemHandle(p);
        cudaGetLastError();
        return fail(FDMS_E_CUDA, "fdms_ipc_region_open: the mapped region is not readable from this device: %s",
                    cudaGetErrorString(e2));
    }
    *ptr = p;
    return FDMS_OK;
}

extern "C" int32_t fdms_ipc_region_close(void* ptr) {
    clear_error();
    if (!ptr) return FDMS_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(FDMS_E_CUDA, "fdms_ipc_region_close: %s", cudaGetErrorString(e)); }
    return FDMS_OK;
}

extern "C" int32_t fdms_ipc_region_destroy(void* ptr) {
    clear_error();
    if (!ptr) return FDMS_OK;
    const cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(FDMS_E_CUDA, "fdms_ipc_region_destroy: %s", cudaGetErrorString(e)); }
    return FDMS_OK;
}

extern "C" int64_t fdms_allreduce_region_bytes(int32_t world, int64_t max_bytes) {
    if (world < 1 || world > kArMaxWorld || max_bytes <= 0) return -1;
    const int64_t half = ((max_bytes + 255) / 256) * 256;
    return 2 * world * 2 * half + 256;             // (word, epoch) slots of both halves, then the epoch counters
}

extern "C" int32_t fdms_allreduce_oneshot(
    void* const* peer_regions, int32_t rank, int32_t world, int64_t max_bytes,
    const void* in, void* out, int64_t n, int32_t dtype, int32_t* dev_status, void* stream) {
    clear_error();
    FDMS_REQUIRE(peer_regions && in && out, FDMS_E_ARG, "fdms_allreduce_oneshot: null pointer");
    FDMS_REQUIRE(world >= 2 && world <= kArMaxWorld && rank >= 0 && rank < world, FDMS_E_ARG,
                 "fdms_allreduce_oneshot: world must be 2..%d and rank inside it", kArMaxWorld);
    FDMS_REQUIRE(dtype == FDMS_F32 || dtype == FDMS_BF16 || dtype == FDMS_F16, FDMS_E_DTYPE,
                 "fdms_allreduce_oneshot: f32, bf16 or f16 only");
    const int64_t esz = dtype == FDMS_F32 ? 4 : 2;
    FDMS_REQUIRE(n > 0 && (n * esz) % 16 == 0 && n * esz <= max_bytes, FDMS_E_CAPACITY,
                 "fdms_allreduce_oneshot: %lld bytes must be a multiple of 16 and at most %lld", (long long)(n * esz),
                 (long long)max_bytes);
    FDMS_REQUIRE(((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0, FDMS_E_ARG,
                 "fdms_allreduce_oneshot: in and out must be 16-byte aligned");
    const int64_t half = ((max_bytes + 255) / 256) * 256;
    ArParams p;
    for (int r = 0; r < kArMaxWorld; ++r) p.slots[r] = nullptr;
    for (int r = 0; r < world; ++r) {
        FDMS_REQUIRE(peer_regions[r] != nullptr, FDMS_E_ARG, "fdms_allreduce_oneshot: region of rank %d is null", r);
        p.slots[r] = (uint8_t*)peer_regions[r];
    }
    p.epoch = (uint32_t*)(p.slots[rank] + 2 * (int64_t)world * 2 * half);
    p.in = in; p.out = out; p.n = n; p.dtype = dtype; p.rank = rank; p.world = world; p.max_bytes = half;
    p.dev_status = dev_status;
    allreduce_oneshot_kernel<<<kArCtas, kArThreads, 0, (cudaStream_t)stream>>>(p);
    FDMS_CHECK_LAUNCH("allreduce_oneshot_kernel");
    return FDMS_OK;
}

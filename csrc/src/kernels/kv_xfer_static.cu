// Allocation-free variant of the paged KV-cache transfer kernel: same data movement as
// kv_xfer.cu, but the block tables and the completion counter live in a scratch area that is
// part of the library image on the GPU.  Contract and rationale: kv_xfer_static.h.
#include <cstdio>
#include <mutex>

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "device/nixl_device_layout.h"
#include "kernels/kv_xfer_static.h"

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr size_t kCounterBytes = 256;
constexpr size_t kTableBytes = size_t(NIXL_KV_STATIC_MAX_PAIRS) * sizeof(int32_t);
constexpr size_t kScratchBytes = kCounterBytes + 2 * kTableBytes;

// Layout: [0,256) completion counter (first word used) | source block table | destination block table.
// In host code this name is only a handle for cudaGetSymbolAddress; device code names it directly.
static __device__ __align__(256) unsigned char g_kvScratch[kScratchBytes];

__device__ __forceinline__ uint4 ldStream(const void *p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void stStream16(void *p, const uint4 &v) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void stStream8(void *p, const uint2 &v) {
    asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ uint32_t castPair(uint32_t packed, float scale) {
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162 *>(&packed);
    float2 f = __bfloat1622float2(b);
    f.x *= scale;
    f.y *= scale;
    return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint2 castVec(const uint4 &v, float scale) {
    uint2 o;
    o.x = castPair(v.x, scale) | (castPair(v.y, scale) << 16);
    o.y = castPair(v.z, scale) | (castPair(v.w, scale) << 16);
    return o;
}

template<bool kCast> __global__ void __launch_bounds__(kThreads) kvXferStaticKernel(const __grid_constant__ NixlKvXferParams p) {
    const nixlMemViewEntry *src_ent =
        reinterpret_cast<const nixlMemViewEntry *>(static_cast<const char *>(p.src_view) + sizeof(nixlMemViewHeader));
    const nixlMemViewEntry *dst_ent =
        reinterpret_cast<const nixlMemViewEntry *>(static_cast<const char *>(p.dst_view) + sizeof(nixlMemViewHeader));
    unsigned int *counter = reinterpret_cast<unsigned int *>(g_kvScratch);
    const int32_t *src_blocks = reinterpret_cast<const int32_t *>(g_kvScratch + kCounterBytes);
    const int32_t *dst_blocks = reinterpret_cast<const int32_t *>(g_kvScratch + kCounterBytes + kTableBytes);

    const int vec_per_row = p.head_bytes >> 4;
    const int vec_per_unit = p.tokens * p.heads * vec_per_row;
    const long long units = static_cast<long long>(p.n_tensors) * p.n_pairs;
    const int dst_vec_bytes = kCast ? 8 : 16;

    for (long long u0 = static_cast<long long>(blockIdx.x) * kUnroll; u0 < units; u0 += static_cast<long long>(gridDim.x) * kUnroll) {
        const char *sbase[kUnroll];
        char *dbase[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const long long u = u0 + k;
            if (u < units) {
                const int t = static_cast<int>(u / p.n_pairs);
                const int i = static_cast<int>(u - static_cast<long long>(t) * p.n_pairs);
                sbase[k] = reinterpret_cast<const char *>(src_ent[t].ptr) + static_cast<long long>(src_blocks[i]) * p.src_block_stride;
                dbase[k] = reinterpret_cast<char *>(dst_ent[t].ptr) + static_cast<long long>(dst_blocks[i]) * p.dst_block_stride +
                    static_cast<long long>(p.dst_head_offset) * p.dst_head_stride;
            } else {
                sbase[k] = nullptr;
                dbase[k] = nullptr;
            }
        }
        for (int idx = threadIdx.x; idx < vec_per_unit; idx += kThreads) {
            const int row = idx / vec_per_row;
            const int v = idx - row * vec_per_row;
            const int token = row / p.heads;
            const int head = row - token * p.heads;
            const long long soff = token * p.src_token_stride + head * p.src_head_stride + (static_cast<long long>(v) << 4);
            const long long doff = token * p.dst_token_stride + head * p.dst_head_stride + static_cast<long long>(v) * dst_vec_bytes;
            uint4 val[kUnroll];
#pragma unroll
            for (int k = 0; k < kUnroll; ++k)
                if (sbase[k]) val[k] = ldStream(sbase[k] + soff);
#pragma unroll
            for (int k = 0; k < kUnroll; ++k)
                if (sbase[k]) {
                    if constexpr (kCast) stStream8(dbase[k] + doff, castVec(val[k], p.scale));
                    else stStream16(dbase[k] + doff, val[k]);
                }
        }
    }

    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned prev = atomicAdd(counter, 1u);
        if (prev == gridDim.x - 1) {
            *counter = 0;
            __threadfence_system();
            if (p.done_signal) asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p.done_signal), "l"(p.done_value) : "memory");
            if (p.host_flag) asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.host_flag), "l"(p.host_seq) : "memory");
        }
    }
}

// Device address of g_kvScratch per GPU, looked up once per device with that device current.
constexpr int kMaxDevices = 64;
std::mutex g_setupMu;
unsigned char *g_scratchAddr[kMaxDevices] = {};

int scratchFor(int device, unsigned char **out) {
    if (device < 0 || device >= kMaxDevices) return NIXL_KV_STATIC_ERR_SETUP;
    std::lock_guard<std::mutex> g(g_setupMu);
    if (!g_scratchAddr[device]) {
        void *addr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&addr, g_kvScratch); // the current device is `device`
        if (e != cudaSuccess || addr == nullptr) {
            std::fprintf(stderr, "nixl_kv_xfer_launch_static: cannot obtain the scratch area's address on GPU %d: %s\n", device,
                         cudaGetErrorString(e));
            return NIXL_KV_STATIC_ERR_SETUP;
        }
        g_scratchAddr[device] = static_cast<unsigned char *>(addr);
    }
    *out = g_scratchAddr[device];
    return 0;
}

} // namespace

extern "C" int nixl_kv_xfer_static_max_pairs(void) { return NIXL_KV_STATIC_MAX_PAIRS; }

extern "C" int nixl_kv_xfer_launch_static(const NixlKvXferParams *params, const int32_t *host_src_blocks,
                                          const int32_t *host_dst_blocks, void *stream) {
    if (!params || !params->src_view || !params->dst_view || !host_src_blocks || !host_dst_blocks) return cudaErrorInvalidValue;
    const NixlKvXferParams &p = *params;
    if (p.n_pairs <= 0 || p.n_tensors <= 0 || p.tokens <= 0 || p.heads <= 0 || p.head_bytes <= 0 || (p.head_bytes & 15))
        return cudaErrorInvalidValue;
    if (p.n_pairs > NIXL_KV_STATIC_MAX_PAIRS) {
        std::fprintf(stderr,
                     "nixl_kv_xfer_launch_static: %d block pairs exceed the built-in scratch capacity of %d; split the transfer or use "
                     "nixl_kv_xfer_launch with caller-provided device memory\n",
                     p.n_pairs, NIXL_KV_STATIC_MAX_PAIRS);
        return NIXL_KV_STATIC_ERR_TOO_LARGE;
    }
    const int64_t sa = p.src_block_stride | p.src_token_stride | p.src_head_stride;
    const int64_t da = p.dst_block_stride | p.dst_token_stride | p.dst_head_stride;
    if ((sa & 15) || (da & (p.cast_fp8 ? 7 : 15))) return cudaErrorInvalidValue;

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    unsigned char *scratch = nullptr;
    if (const int rc = scratchFor(dev, &scratch); rc != 0) return rc;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Stream-ordered: clear the counter, stage both tables, then run.  The previous call's
    // contents are overwritten or ignored (only the first n_pairs entries are read).
    if ((e = cudaMemsetAsync(scratch, 0, kCounterBytes, s)) != cudaSuccess) return static_cast<int>(e);
    const size_t bytes = static_cast<size_t>(p.n_pairs) * sizeof(int32_t);
    if ((e = cudaMemcpyAsync(scratch + kCounterBytes, host_src_blocks, bytes, cudaMemcpyHostToDevice, s)) != cudaSuccess)
        return static_cast<int>(e);
    if ((e = cudaMemcpyAsync(scratch + kCounterBytes + kTableBytes, host_dst_blocks, bytes, cudaMemcpyHostToDevice, s)) != cudaSuccess)
        return static_cast<int>(e);

    int grid = p.grid;
    if (grid <= 0) {
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        grid = sms * 4;
    }
    const long long units = static_cast<long long>(p.n_tensors) * p.n_pairs;
    const long long want = (units + kUnroll - 1) / kUnroll;
    if (grid > want) grid = static_cast<int>(want);
    if (p.cast_fp8) kvXferStaticKernel<true><<<grid, kThreads, 0, s>>>(p);
    else kvXferStaticKernel<false><<<grid, kThreads, 0, s>>>(p);
    return static_cast<int>(cudaGetLastError());
}

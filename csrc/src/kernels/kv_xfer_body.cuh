// Device-side body of the paged KV-cache transfer, shared by the regular entry point
// (kv_xfer.cu: block tables and completion counter in caller-provided device memory) and the
// allocation-free one (kv_xfer_static.cu: both inside the library's own scratch area).
//
// Work unit: one (cache tensor, block pair).  A block is tokens*heads rows of head_bytes; a
// thread moves 16 source bytes at a time, so a Llama-3-8B block of a TP=4 prefill rank
// (16 tokens x 2 heads x 256 B = 8 KiB) is 512 vector loads, done by one 256-thread CTA in two
// rounds.  CTAs are persistent and walk the units with a grid stride; kKvUnroll units are
// in flight per CTA so NVLink stores of one unit overlap the HBM loads of the next.
#ifndef NIXL_B200_KV_XFER_BODY_CUH
#define NIXL_B200_KV_XFER_BODY_CUH

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "device/nixl_device_layout.h"
#include "kernels/nixl_kernels.h"

namespace nixl_kv {

constexpr int kKvThreads = 256;
constexpr int kKvUnroll = 4;

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

// Two bf16 (packed in a u32) -> two e4m3 (packed in the low 16 bits), after scaling.
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

// Moves every (tensor, block pair) unit of the request.  src_blocks / dst_blocks are the block
// tables in device memory (wherever the entry point keeps them).
template<bool kCast>
__device__ __forceinline__ void moveBlocks(const NixlKvXferParams &p, const int32_t *__restrict__ src_blocks, const int32_t *__restrict__ dst_blocks) {
    const nixlMemViewEntry *src_ent =
        reinterpret_cast<const nixlMemViewEntry *>(static_cast<const char *>(p.src_view) + sizeof(nixlMemViewHeader));
    const nixlMemViewEntry *dst_ent =
        reinterpret_cast<const nixlMemViewEntry *>(static_cast<const char *>(p.dst_view) + sizeof(nixlMemViewHeader));

    const int vec_per_row = p.head_bytes >> 4;              // 16-byte vectors per (token, head) row
    const int rows = p.tokens * p.heads;
    const int vec_per_unit = rows * vec_per_row;
    const long long units = static_cast<long long>(p.n_tensors) * p.n_pairs;
    const int dst_vec_bytes = kCast ? 8 : 16;
    // Bytes a block spans from its base on either side (strides are non-negative), for the bounds check.
    const long long src_extent = (p.tokens - 1LL) * p.src_token_stride + (p.heads - 1LL) * p.src_head_stride + p.head_bytes;
    const long long dst_extent = (p.tokens - 1LL) * p.dst_token_stride + (p.dst_head_offset + p.heads - 1LL) * p.dst_head_stride +
        (kCast ? p.head_bytes / 2 : p.head_bytes);

    for (long long u0 = static_cast<long long>(blockIdx.x) * kKvUnroll; u0 < units; u0 += static_cast<long long>(gridDim.x) * kKvUnroll) {
        const char *sbase[kKvUnroll];
        char *dbase[kKvUnroll];
#pragma unroll
        for (int k = 0; k < kKvUnroll; ++k) {
            const long long u = u0 + k;
            if (u < units) {
                // Pairs vary fastest so that consecutive units read one tensor's blocks.
                const int t = static_cast<int>(u / p.n_pairs);
                const int i = static_cast<int>(u - static_cast<long long>(t) * p.n_pairs);
                const long long sb = __ldg(src_blocks + i), db = __ldg(dst_blocks + i);
                const long long soff = sb * p.src_block_stride, doff = db * p.dst_block_stride;
                // The block tables come from device memory that nobody validated: a block must lie inside its tensor's
                // registered range on both sides, or it is skipped and reported.
                const bool inside = sb >= 0 && db >= 0 && src_ent[t].ptr != 0 && dst_ent[t].ptr != 0 &&
                    static_cast<unsigned long long>(soff + src_extent) <= src_ent[t].len && static_cast<unsigned long long>(doff + dst_extent) <= dst_ent[t].len;
                if (inside) {
                    sbase[k] = reinterpret_cast<const char *>(src_ent[t].ptr) + soff;
                    dbase[k] = reinterpret_cast<char *>(dst_ent[t].ptr) + doff + static_cast<long long>(p.dst_head_offset) * p.dst_head_stride;
                } else {
                    sbase[k] = nullptr;
                    dbase[k] = nullptr;
                    if (threadIdx.x == 0 && p.status != nullptr) *reinterpret_cast<volatile int32_t *>(p.status) = 1;
                }
            } else {
                sbase[k] = nullptr;
                dbase[k] = nullptr;
            }
        }
        for (int idx = threadIdx.x; idx < vec_per_unit; idx += kKvThreads) {
            const int row = idx / vec_per_row;
            const int v = idx - row * vec_per_row;
            const int token = row / p.heads;
            const int head = row - token * p.heads;
            const long long soff = token * p.src_token_stride + head * p.src_head_stride + (static_cast<long long>(v) << 4);
            const long long doff = token * p.dst_token_stride + head * p.dst_head_stride + static_cast<long long>(v) * dst_vec_bytes;
            uint4 val[kKvUnroll];
#pragma unroll
            for (int k = 0; k < kKvUnroll; ++k)
                if (sbase[k]) val[k] = ldStream(sbase[k] + soff);
#pragma unroll
            for (int k = 0; k < kKvUnroll; ++k)
                if (sbase[k]) {
                    if constexpr (kCast) stStream8(dbase[k] + doff, castVec(val[k], p.scale));
                    else stStream16(dbase[k] + doff, val[k]);
                }
        }
    }
}

// Completion: the last CTA to finish signals the receiver (and the host, if asked).  One
// acquire-release add at GPU scope chains the CTAs; the release operations at system scope
// that follow publish every CTA's stores before the signal becomes visible.  `counter` is zero
// before the launch and is left at zero.
__device__ __forceinline__ void signalWhenAllDone(const NixlKvXferParams &p, unsigned int *counter) {
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned prev;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(counter) : "memory");
        if (prev == gridDim.x - 1) {
            *counter = 0;
            if (p.done_signal) asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p.done_signal), "l"(p.done_value) : "memory");
            if (p.host_flag) asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.host_flag), "l"(p.host_seq) : "memory");
        }
    }
}

// Grid for a request: `wanted` (0 = four CTAs per SM of the current device), never more than there are unit groups.
inline int gridFor(const NixlKvXferParams &p, int device) {
    int grid = p.grid;
    if (grid <= 0) {
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        grid = sms * 4;
    }
    const long long units = static_cast<long long>(p.n_tensors) * p.n_pairs;
    const long long want = (units + kKvUnroll - 1) / kKvUnroll;
    return grid > want ? static_cast<int>(want) : grid;
}

// Shape and alignment checks common to both entry points; cudaSuccess when the request is well formed.
inline cudaError_t checkShape(const NixlKvXferParams &p) {
    if (p.n_pairs <= 0 || p.n_tensors <= 0 || p.tokens <= 0 || p.heads <= 0 || p.head_bytes <= 0 || (p.head_bytes & 15))
        return cudaErrorInvalidValue;
    // Vector accesses need 16-byte (8-byte when casting) aligned strides.
    const int64_t sa = p.src_block_stride | p.src_token_stride | p.src_head_stride;
    const int64_t da = p.dst_block_stride | p.dst_token_stride | p.dst_head_stride;
    if ((sa & 15) || (da & (p.cast_fp8 ? 7 : 15))) return cudaErrorInvalidValue;
    return cudaSuccess;
}

} // namespace nixl_kv

#endif

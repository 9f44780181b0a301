// GPU device API: one-sided transfers issued from inside user kernels.
//
// Same call surface as the reference's src/api/gpu/ucx/nixl_device.cuh (status handle :25,
// cooperation levels :33, defer flag :41, view element :56, nixlGpuGetXferStatus :90,
// nixlPut :121, nixlAtomicAdd :161, nixlGetPtr :192), implemented for a single NVLink
// domain: a memory view is a table of pointers into peers' memory mapped into this
// process, so a put is a cooperative copy with plain stores that travel over NVLink, and
// the "signal" is a release-ordered atomic add at system scope.  Nothing here waits on a
// network or a host thread; the only blocking helper, nixlSignalWait, is bounded in time.
//
// Ordering contract: nixlAtomicAdd on a channel becomes visible at the target after every
// nixlPut issued before it by the same calling group (thread, warp or block).  With
// nixl_gpu_flags::defer the put skips its trailing fence; issue the signal (or a put
// without defer) to flush.
//
// Additions over the reference's header (no counterpart there): nixlGet (one-sided read)
// and nixlSignalWait / nixlSignalRead for the consumer side.
#ifndef NIXL_B200_DEVICE_CUH
#define NIXL_B200_DEVICE_CUH

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

#include "device/nixl_device_layout.h"
#include "nixl_types.h"

enum class nixl_gpu_level_t : uint32_t { THREAD = 0, WARP = 1, BLOCK = 2, GRID = 3 };

namespace nixl_gpu_flags {
constexpr unsigned defer = 1u; // do not fence after this operation; a later one will
}

// Completion state of a device-side operation.  Stores over NVLink complete without a
// progress engine, so a handle is complete as soon as the issuing call returns.
struct nixlGpuXferStatusH {
    uint32_t state = 0; // 0: complete, 1: issued without flush (defer)
};

struct nixlMemViewElem {
    nixlMemViewH mvh;
    size_t index;  // entry of the view
    size_t offset; // byte offset inside that entry
};

namespace nixl_gpu_detail {

__device__ __forceinline__ const nixlMemViewEntry *entries(nixlMemViewH mvh) {
    return reinterpret_cast<const nixlMemViewEntry *>(reinterpret_cast<const char *>(mvh) + sizeof(nixlMemViewHeader));
}

__device__ __forceinline__ char *resolve(const nixlMemViewElem &e, size_t size) {
    const auto *hdr = reinterpret_cast<const nixlMemViewHeader *>(e.mvh);
    if (hdr == nullptr || e.index >= hdr->count) return nullptr;
    const nixlMemViewEntry ent = entries(e.mvh)[e.index];
    if (ent.ptr == 0 || e.offset + size > ent.len) return nullptr;
    return reinterpret_cast<char *>(ent.ptr) + e.offset;
}

template<nixl_gpu_level_t level> __device__ __forceinline__ unsigned laneOf() {
    if constexpr (level == nixl_gpu_level_t::THREAD) return 0;
    else if constexpr (level == nixl_gpu_level_t::WARP) return threadIdx.x & 31;
    else if constexpr (level == nixl_gpu_level_t::BLOCK) return threadIdx.x + threadIdx.y * blockDim.x + threadIdx.z * blockDim.x * blockDim.y;
    else return (blockIdx.x + blockIdx.y * gridDim.x) * (blockDim.x * blockDim.y * blockDim.z) + threadIdx.x + threadIdx.y * blockDim.x;
}

template<nixl_gpu_level_t level> __device__ __forceinline__ unsigned widthOf() {
    if constexpr (level == nixl_gpu_level_t::THREAD) return 1;
    else if constexpr (level == nixl_gpu_level_t::WARP) return 32;
    else if constexpr (level == nixl_gpu_level_t::BLOCK) return blockDim.x * blockDim.y * blockDim.z;
    else return gridDim.x * gridDim.y * blockDim.x * blockDim.y * blockDim.z;
}

// Barrier among the calling group (GRID callers synchronise themselves, e.g. cooperative groups).
template<nixl_gpu_level_t level> __device__ __forceinline__ void groupSync() {
    if constexpr (level == nixl_gpu_level_t::WARP) __syncwarp();
    else if constexpr (level == nixl_gpu_level_t::BLOCK) __syncthreads();
}

// Cooperative copy: 16-byte vectors when both ends allow it, bytes otherwise.
template<nixl_gpu_level_t level> __device__ __forceinline__ void copy(char *dst, const char *src, size_t n) {
    const unsigned lane = laneOf<level>(), width = widthOf<level>();
    if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
        const size_t nvec = n >> 4;
        const uint4 *s = reinterpret_cast<const uint4 *>(src);
        uint4 *d = reinterpret_cast<uint4 *>(dst);
        size_t i = lane;
        for (; i + 7 * size_t(width) < nvec; i += 8 * size_t(width)) { // eight loads in flight before the first store
            uint4 t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = s[i + k * size_t(width)];
#pragma unroll
            for (int k = 0; k < 8; ++k) d[i + k * size_t(width)] = t[k];
        }
        for (; i < nvec; i += width) d[i] = s[i];
        for (size_t k = (nvec << 4) + lane; k < n; k += width) dst[k] = src[k];
    } else {
        for (size_t k = lane; k < n; k += width) dst[k] = src[k];
    }
}

} // namespace nixl_gpu_detail

// Progress + query.  There is nothing to progress on NVLink; a deferred handle completes
// at the next fence, which this call issues.
template<nixl_gpu_level_t level = nixl_gpu_level_t::THREAD>
__device__ __forceinline__ nixl_status_t nixlGpuGetXferStatus(nixlGpuXferStatusH &status) {
    if (status.state != 0) {
        __threadfence_system();
        status.state = 0;
    }
    return NIXL_SUCCESS;
}

// One-sided write of `size` bytes from a local view element to a remote view element.
// Every thread of the calling group must make the call with the same arguments.
template<nixl_gpu_level_t level = nixl_gpu_level_t::THREAD>
__device__ __forceinline__ nixl_status_t nixlPut(const nixlMemViewElem &src, const nixlMemViewElem &dst, size_t size,
                                                unsigned channel_id = 0, unsigned flags = 0,
                                                nixlGpuXferStatusH *status = nullptr) {
    (void)channel_id; // channels are an ordering domain of NIC transports; NVLink orders per group
    const char *s = nixl_gpu_detail::resolve(src, size);
    char *d = nixl_gpu_detail::resolve(dst, size);
    if (s == nullptr || d == nullptr) return NIXL_ERR_INVALID_PARAM;
    nixl_gpu_detail::copy<level>(d, s, size);
    if (!(flags & nixl_gpu_flags::defer)) {
        nixl_gpu_detail::groupSync<level>();
        __threadfence_system();
    }
    if (status) status->state = (flags & nixl_gpu_flags::defer) ? 1u : 0u;
    return NIXL_SUCCESS;
}

// One-sided read: remote view element -> local view element.
template<nixl_gpu_level_t level = nixl_gpu_level_t::THREAD>
__device__ __forceinline__ nixl_status_t nixlGet(const nixlMemViewElem &local_dst, const nixlMemViewElem &remote_src, size_t size,
                                                unsigned channel_id = 0, unsigned flags = 0,
                                                nixlGpuXferStatusH *status = nullptr) {
    (void)channel_id;
    char *d = nixl_gpu_detail::resolve(local_dst, size);
    const char *s = nixl_gpu_detail::resolve(remote_src, size);
    if (s == nullptr || d == nullptr) return NIXL_ERR_INVALID_PARAM;
    nixl_gpu_detail::copy<level>(d, s, size);
    if (!(flags & nixl_gpu_flags::defer)) nixl_gpu_detail::groupSync<level>();
    if (status) status->state = 0;
    return NIXL_SUCCESS;
}

// Adds `value` to a 64-bit counter in a remote view, ordered after the group's earlier puts.
// One thread of the group performs the add.
template<nixl_gpu_level_t level = nixl_gpu_level_t::THREAD>
__device__ __forceinline__ nixl_status_t nixlAtomicAdd(uint64_t value, const nixlMemViewElem &counter, unsigned channel_id = 0,
                                                      unsigned flags = 0, nixlGpuXferStatusH *status = nullptr) {
    (void)channel_id;
    (void)flags;
    char *p = nixl_gpu_detail::resolve(counter, sizeof(uint64_t));
    if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 7)) return NIXL_ERR_INVALID_PARAM;
    nixl_gpu_detail::groupSync<level>(); // the group's stores happen-before the elected thread's fence
    if (nixl_gpu_detail::laneOf<level>() == 0) {
        // One release at system scope: it orders the elected thread's own stores and, through the group
        // barrier above, the other threads' (a separate fence in front of it would wait for the peer's
        // acknowledgements a second time).
        asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(value) : "memory");
    }
    if (status) status->state = 0;
    return NIXL_SUCCESS;
}

// Raw pointer to entry `index` of a view, or nullptr for a hole / bad index.  Peers of one
// NVLink domain are always load/store reachable.
__device__ __forceinline__ void *nixlGetPtr(nixlMemViewH mvh, size_t index) {
    const auto *hdr = reinterpret_cast<const nixlMemViewHeader *>(mvh);
    if (hdr == nullptr || index >= hdr->count) return nullptr;
    return reinterpret_cast<void *>(nixl_gpu_detail::entries(mvh)[index].ptr);
}

// Consumer side: current value of a local counter (acquire).
__device__ __forceinline__ uint64_t nixlSignalRead(const uint64_t *counter) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(counter) : "memory");
    return v;
}

// Spins until *counter >= expected or `timeout_ns` elapses.  NIXL_SUCCESS, or
// NIXL_ERR_REMOTE_DISCONNECT on timeout (the caller decides what to do; the GPU is never
// left spinning).  Call from one thread and broadcast, or from every thread of a group.
__device__ __forceinline__ nixl_status_t nixlSignalWait(const uint64_t *counter, uint64_t expected, uint64_t timeout_ns) {
    uint64_t t0 = 0;
    unsigned spins = 0;
    while (nixlSignalRead(counter) < expected) {
        if ((++spins & 63u) == 0) {
            uint64_t now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > timeout_ns) return NIXL_ERR_REMOTE_DISCONNECT;
        }
    }
    return NIXL_SUCCESS;
}

#endif

// Allocation-free variant of the paged KV-cache transfer kernel: the data movement of
// kv_xfer_body.cuh, with the block tables and the completion counter in a scratch area that is
// part of the library image on the GPU.  Contract and rationale: include/kernels/nixl_kv_xfer_static.h.
#include <cstdio>
#include <mutex>

#include "kernels/kv_xfer_body.cuh"
#include "kernels/nixl_kv_xfer_static.h"

namespace {

constexpr size_t kCounterBytes = 256;
constexpr size_t kTableBytes = size_t(NIXL_KV_STATIC_MAX_PAIRS) * sizeof(int32_t);
constexpr size_t kScratchBytes = kCounterBytes + 2 * kTableBytes;

// Layout: [0,256) completion counter (first word used) | source block table | destination block table.
// In host code this name is only a handle for cudaGetSymbolAddress; device code names it directly.
static __device__ __align__(256) unsigned char g_kvScratch[kScratchBytes];

template<bool kCast> __global__ void __launch_bounds__(nixl_kv::kKvThreads) kvXferStaticKernel(const __grid_constant__ NixlKvXferParams p) {
    nixl_kv::moveBlocks<kCast>(p, reinterpret_cast<const int32_t *>(g_kvScratch + kCounterBytes),
                               reinterpret_cast<const int32_t *>(g_kvScratch + kCounterBytes + kTableBytes));
    nixl_kv::signalWhenAllDone(p, reinterpret_cast<unsigned int *>(g_kvScratch));
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
    if (p.n_pairs > NIXL_KV_STATIC_MAX_PAIRS) {
        std::fprintf(stderr,
                     "nixl_kv_xfer_launch_static: %d block pairs exceed the built-in scratch capacity of %d; split the transfer or use "
                     "nixl_kv_xfer_launch with caller-provided device memory\n",
                     p.n_pairs, NIXL_KV_STATIC_MAX_PAIRS);
        return NIXL_KV_STATIC_ERR_TOO_LARGE;
    }
    if (const cudaError_t e = nixl_kv::checkShape(p); e != cudaSuccess) return e;

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

    const int grid = nixl_kv::gridFor(p, dev);
    if (p.cast_fp8) kvXferStaticKernel<true><<<grid, nixl_kv::kKvThreads, 0, s>>>(p);
    else kvXferStaticKernel<false><<<grid, nixl_kv::kKvThreads, 0, s>>>(p);
    return static_cast<int>(cudaGetLastError());
}

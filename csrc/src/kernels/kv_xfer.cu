// Fused paged-KV-cache transfer kernel (see include/kernels/nixl_kernels.h for the contract).
// The data movement itself is in kv_xfer_body.cuh, shared with the allocation-free entry point.
#include "kernels/kv_xfer_body.cuh"

namespace {

template<bool kCast> __global__ void __launch_bounds__(nixl_kv::kKvThreads) kvXferKernel(const __grid_constant__ NixlKvXferParams p) {
    nixl_kv::moveBlocks<kCast>(p, p.src_blocks, p.dst_blocks);
    nixl_kv::signalWhenAllDone(p, p.done_counter);
}

} // namespace

extern "C" int nixl_kv_xfer_launch(const NixlKvXferParams *params, void *stream) {
    if (!params || !params->src_view || !params->dst_view || !params->src_blocks || !params->dst_blocks || !params->done_counter)
        return cudaErrorInvalidValue;
    const NixlKvXferParams &p = *params;
    if (const cudaError_t e = nixl_kv::checkShape(p); e != cudaSuccess) return e;
    int dev = 0;
    cudaGetDevice(&dev);
    const int grid = nixl_kv::gridFor(p, dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (p.cast_fp8) kvXferKernel<true><<<grid, nixl_kv::kKvThreads, 0, s>>>(p);
    else kvXferKernel<false><<<grid, nixl_kv::kKvThreads, 0, s>>>(p);
    return static_cast<int>(cudaGetLastError());
}

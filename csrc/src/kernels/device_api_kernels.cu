// Kernels that exercise the GPU device API (include/device/nixl_device.cuh) from outside the
// library's own transfer paths: a correctness kernel used by the tests (put / get / atomic add
// / get-pointer at THREAD, WARP and BLOCK level) and the persistent put-with-signal kernel of
// the device-initiated benchmark.
//
// Parity: the reference's test/gtest/device_api/single_write_test.cu (putKernel :34,
// getPtrKernel :84) and benchmark/nixlbench/src/kernels/nixlbench_device_launch.cu:79
// (nixlbenchPutKernel: puts per region, then a completion counter add).
#include <cuda_runtime.h>

#include "device/nixl_device.cuh"
#include "kernels/nixl_kernels.h"

namespace {

template<nixl_gpu_level_t level>
__global__ void putTestKernel(nixlMemViewH src, nixlMemViewH dst, nixlMemViewH sig, size_t size, int iters, int use_get, int *status_out) {
    // One calling group per launch (a thread, a warp or a block); every iteration moves `size`
    // bytes from entry 0 of the local view to entry 0 of the remote view at offset iter * size
    // and then bumps the remote counter.
    nixl_status_t st = NIXL_SUCCESS;
    for (int i = 0; i < iters && st == NIXL_SUCCESS; ++i) {
        nixlMemViewElem s{src, 0, static_cast<size_t>(i) * size};
        nixlMemViewElem d{dst, 0, static_cast<size_t>(i) * size};
        nixlGpuXferStatusH h;
        if (use_get) st = nixlGet<level>(s, d, size, 0, 0, &h); // local <- remote
        else st = nixlPut<level>(s, d, size, 0, (i & 1) ? nixl_gpu_flags::defer : 0, &h);
        if (st == NIXL_SUCCESS) st = nixlGpuGetXferStatus<level>(h);
        if (st == NIXL_SUCCESS) st = nixlAtomicAdd<level>(1, nixlMemViewElem{sig, 0, 0}, 0, 0, nullptr);
    }
    // Out-of-range requests must be refused, not executed.
    nixlMemViewElem bad{dst, 99, 0};
    const nixl_status_t refused = nixlPut<level>(nixlMemViewElem{src, 0, 0}, bad, 16);
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        status_out[0] = static_cast<int>(st);
        status_out[1] = static_cast<int>(refused);
        status_out[2] = nixlGetPtr(dst, 0) != nullptr;
        status_out[3] = nixlGetPtr(dst, 99) == nullptr;
    }
}

// Persistent producer/consumer kernel of the device-initiated benchmark.
//   producer CTAs (ctas_per_peer per peer): CTA c of a peer owns iterations c+1, c+1+ctas_per_peer, ...: a stand-in
//                  compute pass over the tile, then nixlPut<BLOCK> of the whole tile into slot (it-1) % window of
//                  the peer's landing zone for this rank and an atomic add on that slot's arrival counter at the
//                  peer.  A tile's stores are acknowledged by the peer before its signal leaves (about 3 us over
//                  NVLink); with ctas_per_peer tiles in flight per peer that wait overlaps the next tiles' copies.
//   last CTA:      consumer: thread (j, s) takes the tiles of peer j in slot s in order: waits (bounded) for the slot's
//                  counter, then bumps the slot's acknowledgement counter at the peer.
// Flow control: slot s is written for the k-th time only after its (k-1)-th content was acknowledged.
// Signal words (local_signals entry 0, remote_signals entry r): arrival[peer][slot] at byte (peer * window + slot) * 8,
// acknowledgement[peer][slot] at ack_offset + the same.
__global__ void __launch_bounds__(512) putSignalKernel(NixlDevPutParams p) {
    __shared__ int failed;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    const int b = blockIdx.x;
    const int cpp = p.ctas_per_peer;
    if (b < p.peers * cpp) {
        const int pi = b / cpp, lane_it = b - pi * cpp;
        const int peer = p.peer_ids[pi];
        const size_t tile_off = static_cast<size_t>(b) * p.tile_bytes; // every producer CTA has a source tile of its own
        float4 *tile = reinterpret_cast<float4 *>(static_cast<char *>(nixlGetPtr(p.local_tiles, 0)) + tile_off);
        const size_t n4 = p.tile_bytes / sizeof(float4);
        const uint64_t *ack = reinterpret_cast<const uint64_t *>(static_cast<char *>(nixlGetPtr(p.local_signals, 0)) + p.ack_offset) +
            static_cast<size_t>(peer) * p.window;
        for (int it = lane_it + 1; it <= p.iters; it += cpp) {
            // stand-in for the compute that produces the tile
            for (int r = 0; r < p.compute_passes; ++r)
                for (size_t i = threadIdx.x; i < n4; i += blockDim.x) {
                    float4 v = tile[i];
                    v.x = fmaf(v.x, 1.0001f, 0.5f);
                    v.y = fmaf(v.y, 0.9999f, -0.5f);
                    tile[i] = v;
                }
            __syncthreads();
            const int slot = (it - 1) % p.window;
            const uint64_t uses_before = static_cast<uint64_t>((it - 1) / p.window);
            if (uses_before > 0) { // the slot's previous content must have been consumed
                if (threadIdx.x == 0 && nixlSignalWait(ack + slot, uses_before, p.timeout_ns) != NIXL_SUCCESS) failed = 1;
                __syncthreads();
                if (failed) break;
            }
            nixlMemViewElem src{p.local_tiles, 0, tile_off};
            nixlMemViewElem dst{p.remote_tiles, static_cast<size_t>(peer), (static_cast<size_t>(p.rank) * p.window + slot) * p.tile_bytes};
            // deferred: the signal that follows is the flush (one wait for the peer's acknowledgements per tile, not two)
            nixlPut<nixl_gpu_level_t::BLOCK>(src, dst, p.tile_bytes, 0, nixl_gpu_flags::defer);
            nixlAtomicAdd<nixl_gpu_level_t::BLOCK>(
                1, nixlMemViewElem{p.remote_signals, static_cast<size_t>(peer), (static_cast<size_t>(p.rank) * p.window + slot) * 8});
        }
    } else {
        // Consumer: thread (j, s) takes the tiles that peer j puts into slot s, in order.  One thread per slot: an
        // acknowledgement is a release at system scope, which waits for the previous one to be confirmed by the peer;
        // with a thread per slot those round trips overlap.
        const int pi = static_cast<int>(threadIdx.x) / p.window, slot = static_cast<int>(threadIdx.x) % p.window;
        if (pi < p.peers) {
            const int peer = p.peer_ids[pi];
            const uint64_t *arrived = reinterpret_cast<const uint64_t *>(nixlGetPtr(p.local_signals, 0)) + static_cast<size_t>(peer) * p.window + slot;
            uint64_t uses = 0;
            for (int it = slot + 1; it <= p.iters; it += p.window) {
                if (nixlSignalWait(arrived, ++uses, p.timeout_ns) != NIXL_SUCCESS) {
                    failed = 1;
                    break;
                }
                nixlAtomicAdd<nixl_gpu_level_t::THREAD>(
                    1, nixlMemViewElem{p.remote_signals, static_cast<size_t>(peer), p.ack_offset + (static_cast<size_t>(p.rank) * p.window + slot) * 8});
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && failed) atomicOr(p.status, 1);
}

} // namespace

extern "C" int nixl_devapi_put_test(int level, const void *src_view, const void *dst_view, const void *sig_view, uint64_t size, int iters,
                                    int use_get, int *status_out, void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    nixlMemViewH a = const_cast<void *>(src_view), b = const_cast<void *>(dst_view), c = const_cast<void *>(sig_view);
    switch (level) {
    case 0: putTestKernel<nixl_gpu_level_t::THREAD><<<1, 1, 0, s>>>(a, b, c, size, iters, use_get, status_out); break;
    case 1: putTestKernel<nixl_gpu_level_t::WARP><<<1, 32, 0, s>>>(a, b, c, size, iters, use_get, status_out); break;
    case 2: putTestKernel<nixl_gpu_level_t::BLOCK><<<1, 256, 0, s>>>(a, b, c, size, iters, use_get, status_out); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

extern "C" int nixl_devapi_put_signal_launch(const NixlDevPutParams *params, void *stream) {
    if (!params || params->peers <= 0 || params->peers > 64 || params->window <= 0 || params->ctas_per_peer <= 0 || (params->tile_bytes % 16ull))
        return cudaErrorInvalidValue;
    // All CTAs must be resident together (producers wait for acknowledgements raised by consumer
    // CTAs of the peers, and the local consumer CTA must run next to the producers).
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = params->peers * params->ctas_per_peer + 1;
    if (grid > sms || params->peers * params->window > 512) return cudaErrorInvalidValue;
    // Cooperative launch: the runtime refuses the launch unless every CTA can be resident at once.
    NixlDevPutParams copy = *params;
    void *args[] = {&copy};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(putSignalKernel), dim3(grid), dim3(512), args, 0, static_cast<cudaStream_t>(stream));
}

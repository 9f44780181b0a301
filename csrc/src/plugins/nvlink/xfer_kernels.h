// Host-callable launchers of the NVLink backend's copy kernels (xfer_kernels.cu).
//
// One launch moves a whole batch of descriptors.  Work is cut into power-of-two chunks;
// chunk c belongs to the descriptor i with chunkStart[i] <= c < chunkStart[i+1].  A
// persistent grid walks the chunks, so 256 x 4 KiB and 1 x 1 GiB cost one launch each.
// The CTA that finishes last publishes `seq` to a host-mapped completion word, which is
// what the backend's checkXfer polls - no event, no stream synchronisation.
#ifndef NIXL_B200_XFER_KERNELS_H
#define NIXL_B200_XFER_KERNELS_H

#include <cstdint>
#include <cuda_runtime.h>

namespace nixl_nvlink {

struct XferDesc {
    uint64_t src;
    uint64_t dst;
    uint64_t len;
};

// Small batches ride in the kernel parameters: no table upload, no device allocation.
constexpr int kInlineDescs = 32;

struct XferLaunch {
    const XferDesc *table;      // device table (nDescs entries) or nullptr when inline
    const uint32_t *chunkStart; // device array, nDescs + 1 entries, or nullptr when inline
    uint32_t nDescs;
    uint32_t totalChunks;
    uint32_t chunkShift;        // chunk size = 1 << chunkShift bytes
    uint32_t pad;
    unsigned int *doneCounter;  // device word, zero between launches
    uint64_t *hostFlag;         // device-visible address of the pinned completion word
    uint64_t seq;               // value stored to *hostFlag when the batch is complete
    XferDesc inl[kInlineDescs];
    uint32_t inlStart[kInlineDescs + 1];
};

// Ways to move a batch: SIMT vectors, bulk (TMA 1-D) staged through shared memory, or the GPU's
// copy engines (one cudaMemcpyAsync per descriptor followed by launchSignal: what a
// descriptor-at-a-time transport does, kept as the baseline the kernels are measured against).
enum class CopyPath : int { VECTOR = 0, BULK = 1, COPY_ENGINE = 2 };

// Launches on `stream` of the current device.  grid_ctas == 0 picks a default.
cudaError_t launchBatchCopy(const XferLaunch &params, int grid_ctas, CopyPath path, cudaStream_t stream);

// One thread stores `seq` to the completion word with release semantics at system scope, after
// everything queued earlier on `stream` (the copy-engine path's completion).
cudaError_t launchSignal(uint64_t *hostFlag, uint64_t seq, cudaStream_t stream);

// Largest useful grid for the current device (SM count x resident CTAs per SM).
int defaultGridCtas(int device);

} // namespace nixl_nvlink

#endif

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
    uint64_t *notifWord;        // device-visible sequence word of a notification slot in the target's host memory, or nullptr
    uint64_t notifSeq;          // value stored to *notifWord when the batch is complete (before the completion word)
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
// With notifWord, `notifSeq` goes to it first.
cudaError_t launchSignal(uint64_t *hostFlag, uint64_t seq, uint64_t *notifWord, uint64_t notifSeq, cudaStream_t stream);

// ------------------------------------------------------------------ doorbell proxy
//
// Small requests do not pay a kernel launch each: while requests keep coming, a persistent
// "proxy" kernel takes them from a ring in pinned host memory that the post path writes with
// plain stores.  CTA 0 polls the host ring and republishes each command in a ring in device
// memory (one PCIe round trip per command, not one per CTA); the worker CTAs poll that ring,
// share the command's chunks between them and the last one to finish stores the command's
// number to a completion word in host memory.  The kernel leaves by itself when nothing has
// arrived for `idleNs`, or after `lifeNs` whatever happens (so that nothing that waits for the
// device to drain waits for long); the host starts it again with the next small request.
// Every wait in it is bounded by those two budgets.
constexpr uint32_t kProxySlots = 64;   // commands in flight at most (host ring = device ring = completion words)
constexpr int kProxyMaxWorkers = 31;

// One command, 32 bytes, written by the host in the order b, c, a, seq and read by the device as two
// 16-byte pieces {seq, a} and {b, c}; c carries the low 16 bits of seq, so that a piece read before the
// host had finished writing is recognised whichever way the bus splits the read.
struct ProxyCmd {
    uint64_t seq; // command number + 1; 0 = never written
    uint64_t a;   // inline: source address      | table: device address of the XferDesc table
    uint64_t b;   // inline: destination address | table: device address of the chunk-start array (nDescs + 1 entries)
    uint64_t c;   // [63:48] low 16 bits of seq, [47:44] kind, [43:38] log2(chunk bytes), [37:0] inline: length;
                  // table: [23:0] descriptor count, [37:24] chunks per descriptor when all have the same number, else 0
};
constexpr uint64_t kProxyInline = 0, kProxyTable = 1, kProxyExit = 2, kProxySkip = 3; // exit / skip: device ring only
constexpr uint32_t kProxyMaxDescs = (1u << 24) - 1, kProxyMaxPer = (1u << 14) - 1;
#ifdef __CUDACC__
__host__ __device__
#endif
inline uint64_t proxyPackC(uint64_t seq, uint64_t kind, uint32_t shift, uint64_t n) {
    return ((seq & 0xffffull) << 48) | (kind << 44) | (uint64_t(shift & 63u) << 38) | (n & ((1ull << 38) - 1));
}

// Device-side state of one proxy (zero-initialised by the host once).
struct ProxyShared {
    ProxyCmd ring[kProxySlots];
    unsigned int counter[kProxySlots];          // "last worker" counters, zero between commands
    unsigned long long workerHead[kProxyMaxWorkers + 1]; // next command each worker will look at
};

struct ProxyLaunch {
    const ProxyCmd *hostRing; // device-visible address of the pinned ring
    ProxyShared *shared;
    uint64_t *done;           // device-visible address of kProxySlots pinned completion words: done[n % slots] = n + 1
    uint64_t *exitWord;       // pinned: written once when the kernel leaves: (1 << 63) | first command it did not take
    uint64_t start;           // first command number this launch handles
    uint64_t gen;             // launch number: tags the entries of the device ring, so that what an earlier launch left
                              // there (its closing "exit" entry carries the number of the NEXT command) is never taken for new
    uint64_t idleNs;
    uint64_t lifeNs;
};

// Launches the proxy with `workers` worker CTAs (plus the polling CTA) on `stream`.
cudaError_t launchProxy(const ProxyLaunch &p, int workers, cudaStream_t stream);

// Largest useful grid for the current device (SM count x resident CTAs per SM).
int defaultGridCtas(int device);

} // namespace nixl_nvlink

#endif

/* Allocation-free entry point of the paged KV-cache transfer.
 *
 * This entry point has no counterpart in the reference library; it exists for callers of
 * this library that are not allowed to allocate GPU memory at the moment they need a
 * transfer: code running inside a serving engine whose memory pool owns the whole device
 * and forbids cudaMalloc after start-up, code that must not take the allocator's lock on a
 * latency-critical path, or a thin C/Fortran/Go host that has no device allocator at hand.
 * nixl_kv_xfer_launch (kernels/nixl_kernels.h) asks such a caller for two things it cannot
 * provide: block tables in device memory and a zeroed device counter.  Here the caller keeps
 * its block tables in ordinary host memory and passes no scratch at all.
 *
 * How: the library carries a fixed scratch area in the GPU's global memory (a file-scope
 * __device__ array, so every GPU that loads libnixl_kernels.so holds it until the process
 * exits).  It stores the staged block tables and the kernel's completion counter:
 *     256 bytes of counters + 2 x NIXL_KV_STATIC_MAX_PAIRS x 4 bytes of tables (about 128 KiB).
 *
 * Rules for the caller:
 *   - n_pairs must not exceed NIXL_KV_STATIC_MAX_PAIRS; larger requests are rejected with
 *     NIXL_KV_STATIC_ERR_TOO_LARGE and a message on stderr.  Split them into several calls.
 *   - The first call on each GPU looks up the device address of the scratch area (a one-time
 *     set-up that talks to the driver).  Make that first call before any stream capture.
 *   - Do not call it while a stream is being captured at all: every call copies the block
 *     tables from the caller's host memory, which capture forbids for pageable memory and, for
 *     pinned memory, would freeze the table contents of that one call into the graph.
 *   - All calls on one GPU share the one scratch area, and it keeps what the previous call
 *     left there.  The entry point clears the counter and overwrites the tables itself, in
 *     stream order, so back-to-back calls on ONE stream are safe.  Calls whose work can
 *     overlap on the GPU (different streams, different threads, different processes are
 *     fine since each process has its own copy) race on the scratch area: serialise them.
 *   - params->src_blocks, params->dst_blocks and params->done_counter are ignored; every
 *     other field has the meaning documented for nixl_kv_xfer_launch.
 *   - host_src_blocks / host_dst_blocks may be pageable or pinned host memory; they can be
 *     reused as soon as the call returns when pageable, and after the stream reaches the copy
 *     when pinned.
 * The entry point calls neither cudaMalloc nor cudaFree nor any allocating library routine.
 */
#ifndef NIXL_B200_NIXL_KV_XFER_STATIC_H
#define NIXL_B200_NIXL_KV_XFER_STATIC_H

#include "kernels/nixl_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

#define NIXL_KV_STATIC_MAX_PAIRS 16384
#define NIXL_KV_STATIC_ERR_TOO_LARGE (-1001) /* n_pairs > NIXL_KV_STATIC_MAX_PAIRS */
#define NIXL_KV_STATIC_ERR_SETUP (-1002)     /* the scratch area's address could not be obtained */

/* Returns 0, a cudaError_t value (> 0), or one of the negative codes above. */
int nixl_kv_xfer_launch_static(const NixlKvXferParams *params, const int32_t *host_src_blocks, const int32_t *host_dst_blocks,
                               void *stream);

/* Capacity in block pairs (NIXL_KV_STATIC_MAX_PAIRS), for callers that size their batches at run time. */
int nixl_kv_xfer_static_max_pairs(void);

#ifdef __cplusplus
}
#endif
#endif

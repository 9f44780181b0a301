/* C ABI of libnixl_kernels.so: fused sm_100a kernels that move data between GPUs of one
 * NVLink domain together with the work next to the transfer.
 *
 * Every launcher returns 0 on success or a cudaError_t value; launches are asynchronous on
 * the given stream (a cudaStream_t passed as void*).  Pointers named *_view are device-side
 * memory views as prepared by nixlAgent::prepMemView (device/nixl_device_layout.h): a header
 * followed by {ptr,len} entries, so peer memory is named the same way as in the device API.
 */
#ifndef NIXL_B200_KERNELS_H
#define NIXL_B200_KERNELS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- paged KV-cache transfer
 *
 * Moves `n_pairs` cache blocks of `n_tensors` cache tensors (K and V of every layer) from this
 * GPU into a peer's cache in ONE launch, fused with
 *   - block-table gather (src_blocks[i]) and scatter (dst_blocks[i]),
 *   - tensor-parallel resharding: the sender's `heads` KV heads land at head slot
 *     `dst_head_offset` of the receiver's (wider or narrower) head dimension,
 *   - optional bf16 -> fp8 e4m3 cast (value * scale, saturating),
 *   - completion: a release-ordered add on a counter in the receiver's memory plus an
 *     optional host-visible flag.
 * A block is tokens x heads rows of head_bytes; both caches are described by byte strides,
 * which covers [block, token, head, dim] and [block, head, token, dim] layouts.
 * The reference moves KV caches as plain descriptor lists (benchmark/kvbench); it has no
 * counterpart of this kernel.
 */
typedef struct NixlKvXferParams {
    const void *src_view;      /* local view: entry t = base of cache tensor t */
    const void *dst_view;      /* remote view: entry t = base of the peer's cache tensor t */
    const int32_t *src_blocks; /* device, n_pairs block ids in the local cache */
    const int32_t *dst_blocks; /* device, n_pairs block ids in the peer cache */
    int32_t n_pairs;
    int32_t n_tensors;
    int32_t tokens;            /* tokens per block */
    int32_t heads;             /* KV heads held by the sender */
    int32_t head_bytes;        /* head_dim * 2 (bf16 source); multiple of 16 */
    int32_t cast_fp8;          /* 0: copy bf16, 1: write e4m3 */
    int64_t src_block_stride, src_token_stride, src_head_stride; /* bytes */
    int64_t dst_block_stride, dst_token_stride, dst_head_stride; /* bytes, in destination element size */
    int32_t dst_head_offset;   /* first head slot written at the receiver */
    float scale;               /* multiplier applied before the fp8 cast */
    uint64_t *done_signal;     /* may be NULL; peer (or local) counter that receives += done_value */
    uint64_t done_value;
    uint64_t *host_flag;       /* may be NULL; host-mapped word that receives host_seq */
    uint64_t host_seq;
    uint32_t *done_counter;    /* device scratch word, zero before the first launch; reset by the kernel */
    int32_t grid;              /* 0: default (two CTAs per SM) */
} NixlKvXferParams;

int nixl_kv_xfer_launch(const NixlKvXferParams *params, void *stream);

#ifdef __cplusplus
}
#endif
#endif

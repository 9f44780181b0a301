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
 * Every block id is checked against the length of its view entry on both sides before a byte of
 * the block moves (block tables are device data nobody validated): see `status`.
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
    int32_t *status;           /* may be NULL; device-visible word (device or pinned host memory) that receives 1 when a block id
                                  pointed outside its cache tensor's view entry: that block is skipped, nothing outside is touched */
} NixlKvXferParams;

int nixl_kv_xfer_launch(const NixlKvXferParams *params, void *stream);


/* ---------------------------------------------------------------- MoE expert-parallel all-to-all
 *
 * Every rank owns one symmetric buffer (same layout on all ranks) registered with its agent;
 * `peers` is a remote memory view whose entry r is rank r's buffer (entry `rank` is the local
 * one; a hole marks an absent rank).  All offsets below are byte offsets into that buffer and
 * already select the parity (double-buffer half) of this call.
 *
 * Dispatch ("count first, then place"):
 *   1. histogram of topk_idx -> tokens per expert;
 *   2. the E counts go to every rank (all-gather), with an epoch flag;
 *   3. once all counts are in, every sender knows where its rows belong at every receiver:
 *      rows of one expert are contiguous and ordered by source rank, so the receiver needs
 *      no second pass to pack them;
 *   4. each token is read once, quantised once (1x128 e4m3 + fp32 scale) and stored to the
 *      up-to-K receivers' packed buffers over NVLink, with its source in `info`;
 *   5. per (expert, source) flags tell the receiver - or a consumer kernel such as the grouped
 *      GEMM below - when an expert's rows from one source have landed.
 * Combine sends expert outputs back to (source rank, token, k) and the source reduces
 * sum_k w[t,k] * y[t,k] in fp32.
 * Every wait on a peer is bounded by timeout_ns; on expiry the peer is marked in `mask`, a bit
 * is set in `status` and the kernel carries on without it.  Nothing traps.
 *
 * Parity with the reference's examples/device/ep (low-latency dispatch/combine kernels
 * nixl_ep_ll.cu:72,:619 and the layout kernel layout.cu:32); the placement algorithm, the
 * single-pass receive and the throughput ("compact") layout are this library's own.
 */
typedef struct NixlEpLayout {
    int64_t off_counts;      /* int32  [R][E]   counts[r][e]: tokens rank r sends to expert e */
    int64_t off_counts_flag; /* uint64 [R]      epoch once row r of counts is complete */
    int64_t off_disp_flag;   /* uint64 [El][R]  epoch once rows of (local expert, source) landed */
    int64_t off_recv_x;      /* [cap][row_bytes] dispatched tokens (e4m3 or bf16) */
    int64_t off_recv_scales; /* float  [cap][H/128] (fp8 only) */
    int64_t off_recv_info;   /* uint32 [cap][2] {source rank, token*K + k} */
    int64_t off_comb_x;      /* bf16   [M][K][H] combine landing zone */
    int64_t off_comb_flag;   /* uint64 [R]      epoch once rank r finished its combine sends (push) / its outputs are ready (pull) */
    int64_t off_comb_in;     /* bf16   [cap][H] expert outputs exposed to peers (pull-mode combine), rows as in recv_x */
    int64_t off_grp;         /* NixlEpGroupRecord [R][M]: per source rank and token, the token's rows on this rank and their weights */
    int64_t off_grp_tokens;  /* int32  [R]      tokens source rank r dispatched (how many of its records are valid) */
} NixlEpLayout;

/* What a token's home rank tells an expert rank about the token's copies there (written by a dispatch
 * that was given the top-k weights): the rank-reduced combine adds those rows up, weighted, on the
 * expert rank and returns ONE row per (token, rank) instead of one per (token, expert). */
typedef struct NixlEpGroupRecord {
    int32_t n;        /* copies of the token on this rank, 0..8 */
    int32_t pad[3];
    int32_t rows[8];  /* their rows in the receive buffer */
    float w[8];       /* their top-k weights */
} NixlEpGroupRecord;

typedef struct NixlEpScratch { /* device memory private to the rank; zero before first use */
    int32_t *cnt;      /* [E] */
    int32_t *fill;     /* [E] */
    int32_t *sent;     /* [E] */
    uint32_t *barrier; /* [4] */
    int32_t *status;   /* [1] bit0: a peer timed out, bit1: grid barrier timed out, bit2: capacity exceeded */
    int32_t *mask;     /* [R] non-zero: rank excluded */
} NixlEpScratch;

typedef struct NixlEpDispatchParams {
    const void *x;            /* bf16 [T][H] */
    const int64_t *topk_idx;  /* [T][K], -1 = unused slot */
    int32_t T, K, H, E, R, rank;
    int32_t use_fp8;          /* 1: e4m3 + scales, 0: bf16 */
    int32_t round_scale;      /* 1: scales rounded up to a power of two */
    int32_t rows_per_expert;  /* >0: expert le starts at row le*rows_per_expert; 0: compact (prefix) layout */
    int32_t cap;              /* rows available at every receiver */
    int32_t phases;           /* bit0 send, bit1 receive (wait for arrivals), bit2 publish recv_count/offsets without waiting */
    int32_t grid;             /* CTAs (cooperative launch); 0 = one per SM */
    const void *peers;        /* remote memory view */
    NixlEpLayout lay;
    uint64_t epoch;
    uint64_t timeout_ns;
    int32_t *recv_count;      /* out [El] rows per local expert */
    int64_t *layout_range;    /* out [El][R] (first row within expert << 32) | rows */
    int32_t *expert_offsets;  /* out [El+1] first row of each local expert (both layouts) */
    NixlEpScratch scr;
    int32_t *send_row;        /* out [T][K] (optional) row each (token, k) landed on at its receiver, -1 if not sent */
    int32_t use_ue8m0;        /* 1 (with use_fp8): scales are powers of two, delivered as biased exponent bytes, four per
                                 32-bit word: recv_scales is uint8 [cap][H/128] with a row pitch of H/128 bytes */
    const float *topk_weights; /* [T][K] or NULL.  Given (K <= 8, R <= 32): group records are written for the rank-reduced combine */
    int32_t max_tokens;       /* M: row pitch of the group records and of the rank-reduced landing zone */
} NixlEpDispatchParams;

typedef struct NixlEpCombineParams {
    const void *x;              /* bf16 [cap][H] expert outputs, rows as delivered by dispatch */
    const uint32_t *recv_info;  /* [cap][2] from the dispatch being answered (local pointer) */
    const int32_t *recv_count;  /* [El] */
    const int32_t *expert_offsets; /* [El+1] */
    const int64_t *topk_idx;    /* [T][K] */
    const float *topk_weights;  /* [T][K] */
    void *out;                  /* bf16 [T][H] */
    int32_t T, K, H, E, R, rank;
    int32_t phases;
    int32_t grid;
    const void *peers;
    NixlEpLayout lay;
    uint64_t epoch;
    uint64_t timeout_ns;
    NixlEpScratch scr;
    /* Pull mode: x already lies at lay.off_comb_in of this rank's symmetric buffer; ranks announce
     * "outputs ready" and every home rank loads its tokens' rows straight from the expert ranks
     * and reduces them, so no row is written twice.  send_row comes from the dispatch. */
    int32_t pull;
    const int32_t *send_row;    /* [T][K] */
    /* Push mode only: rows cross NVLink in a logarithmic 10-bit format (9-bit magnitude code on a
     * per-128-channel grid plus sign; 0.66 of the bf16 bytes) and are decoded inside the reduction.
     * Needs H % 512 == 0. */
    int32_t use_logfmt;
    /* Rank-reduced mode (pull == 2; the dispatch wrote group records): every expert rank adds up, per token, the
     * rows it holds for it, weighted, and stores that one row at the token's home rank (landing row
     * expert_rank * max_tokens + token); the home rank adds the rows of the ranks the token went to.  A token
     * whose experts sit on fewer ranks than it has experts crosses NVLink that much less often. */
    int32_t max_tokens;
} NixlEpCombineParams;

/* Routing statistics of topk_idx [T][K]: tokens per destination rank (a token counts once per rank),
 * (token, k) pairs per expert, and in_rank [T][R] (1 if the token has an expert on that rank). */
int nixl_ep_layout_launch(const int64_t *topk_idx, int32_t T, int32_t K, int32_t E, int32_t R, int32_t *per_rank, int32_t *per_expert,
                          uint8_t *in_rank, void *stream);
int nixl_ep_dispatch_launch(const NixlEpDispatchParams *params, void *stream);
int nixl_ep_combine_launch(const NixlEpCombineParams *params, void *stream);
/* Barrier across ranks through the symmetric buffers (bounded): flag slot `slot` of
 * off_counts_flag-style array at `off_flags`. */
int nixl_ep_barrier_launch(const void *peers, int64_t off_flags, int32_t R, int32_t rank, uint64_t epoch, uint64_t timeout_ns,
                           int32_t *status, int32_t *mask, void *stream);

/* ---------------------------------------------------------------- grouped expert GEMM (tcgen05 / TMEM)
 *
 * D[rows of group g, :] = dequant(A rows) x dequant(W[g])^T, bf16 output.  A and W are e4m3;
 * scale_a has one fp32 per row per 128 channels, scale_w one per 128 x 128 block of W[g].
 * Rows of group g are row_start[g] .. row_start[g] + row_count[g] (device arrays, so the launch
 * can follow an EP dispatch without a host round trip).  With disp_flag set, the kernel waits
 * per (group, source rank) for the arrival flags of that dispatch before it reads rows written
 * by that source (see ep_kernels.cu); `counts` is the dispatch's local [ranks][experts_total]
 * count matrix and expert_base the first global expert of this rank.
 * status bits: 1 = an internal wait exceeded its budget, 2 = an arrival flag never came.
 * To overlap the GEMM with the dispatch that feeds it, launch the dispatch first on another stream
 * with a small grid and give this kernel at most (SM count - that grid) CTAs.
 */
typedef struct NixlGroupedGemmParams {
    const void *a;            /* e4m3 [a_rows][K] */
    const float *scale_a;     /* [a_rows][K/128] */
    const void *w;            /* e4m3 [groups][N][K] */
    const float *scale_w;     /* [groups][N/128][K/128] */
    void *d;                  /* bf16 [a_rows][N] */
    const int32_t *row_start; /* device [groups] */
    const int32_t *row_count; /* device [groups] */
    int32_t groups, N, K, a_rows;
    int32_t grid;             /* 0: one CTA per SM */
    int32_t ranks, experts_total, expert_base;
    int32_t *status;          /* device word, OR-ed */
    const uint64_t *disp_flag; /* [groups][ranks] or NULL */
    const int32_t *counts;     /* [ranks][experts_total] or NULL */
    uint64_t epoch;
    uint64_t timeout_ns;
    /* Overlapped mode: with counts_flag set the kernel does not read row_start / row_count (the
     * dispatch may still be running on another stream); it waits for the count all-gather
     * itself and derives them: rows_per_expert > 0 selects the expert-major layout
     * (row_start[g] = g * rows_per_expert), 0 the compact prefix layout. */
    const uint64_t *counts_flag; /* [ranks] or NULL */
    int32_t rows_per_expert;
    int32_t tile_mode;           /* 0: choose between 1 and 2; 1: 128 x 128 tiles, one CTA each; 2: 256 x 256 tiles, one CTA pair each
                                    (N % 256 == 0); 3: as 2 with power-of-two scales applied by the tensor core: scale_a and
                                    scale_w then point at biased exponent bytes (UE8M0), uint8 [a_rows][K/128] and
                                    [groups][N/128][K/128], K % 512 == 0 */
} NixlGroupedGemmParams;

int nixl_grouped_gemm_fp8_launch(const NixlGroupedGemmParams *params, void *stream);

/* ---------------------------------------------------------------- device API exercisers
 *
 * nixl_devapi_put_test: one calling group (level 0 thread, 1 warp, 2 block) performs `iters`
 * puts (or gets) of `size` bytes between entry 0 of two views, each followed by an atomic add
 * on entry 0 of `sig_view`; status_out[4] receives {last status, status of an out-of-range put,
 * get-pointer of entry 0 non-null, get-pointer of a bad index null}.
 *
 * nixl_devapi_put_signal_launch: the persistent kernel of the device-initiated benchmark.
 * ctas_per_peer producer CTAs per peer take turns at the iterations (CTA c: c+1, c+1+ctas_per_peer, ...): each computes
 * its tile, puts it whole into slot (it-1) % window of the peer's landing area and bumps that slot's arrival counter
 * at the peer; one consumer CTA waits for the slots in order and bumps the acknowledgement counters that gate the
 * producers' reuse of a slot (window >= ctas_per_peer keeps every producer busy).
 * Memory: local_tiles entry 0 = peers * ctas_per_peer source tiles; local_signals entry 0 = this rank's word array:
 * arrival[source rank][slot] (ranks * window words), then at ack_offset acknowledgement[rank][slot]; remote_signals
 * entry r = the same array of rank r; remote_tiles entry r = rank r's landing area of ranks * window * tile_bytes.
 */
typedef struct NixlDevPutParams {
    void *local_tiles;          /* local view, entry 0: peers * ctas_per_peer source tiles of tile_bytes */
    void *remote_tiles;         /* remote view, one entry per rank */
    void *local_signals;        /* local view, entry 0 */
    void *remote_signals;       /* remote view, one entry per rank */
    const int32_t *peer_ids;    /* device [peers] ranks this rank talks to */
    int32_t peers, rank, iters, window, compute_passes;
    int32_t ctas_per_peer;      /* producer CTAs per peer = tiles in flight per peer */
    uint64_t tile_bytes;
    uint64_t ack_offset;        /* bytes */
    uint64_t timeout_ns;
    int32_t *status;            /* bit0: a wait timed out */
} NixlDevPutParams;

int nixl_devapi_put_test(int level, const void *src_view, const void *dst_view, const void *sig_view, uint64_t size, int iters,
                         int use_get, int *status_out, void *stream);
int nixl_devapi_put_signal_launch(const NixlDevPutParams *params, void *stream);

#ifdef __cplusplus
}
#endif
#endif

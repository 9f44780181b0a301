// Grouped fp8 expert GEMM with power-of-two (UE8M0) block scales applied by the tensor core:
// tcgen05.mma.kind::mxf8f6f4.block_scale on CTA pairs, 256 x 256 output tiles.
//
//   D[rows of expert g, :] = (A * 2^(sa-127)) x (W[g] * 2^(sw-127))^T           (bf16 out)
//   A: e4m3 [rows][K], one biased exponent byte per row per 128 channels (what EP dispatch delivers
//      with use_ue8m0: uint8 [rows][K/128], i.e. four consecutive steps per 32-bit word)
//   W: e4m3 [G][N][K], one exponent byte per 128 x 128 block: uint8 [G][N/128][K/128]
//
// With fp32 scales the partial sums of every 128-channel step have to leave TMEM to be scaled
// (grouped_gemm_fp8_pair.cu), and that promotion, not the tensor pipe, bounds the kernel.  Here the
// scale factors ride along with the MMA: a whole K loop accumulates in TMEM and the epilogue runs
// once per tile.
//
// Scale factors reach the tensor core through TMEM.  For four steps at a time ("chunk") the
// epilogue warps, idle during the main loop, build in shared memory the 512-byte layout the
// hardware wants (byte (r % 32) * 16 + (r / 32) * 4 + step for row r: for A one 32-bit word per row
// straight from the scale tensor, for W the block's word repeated for all 128 columns), the issuing
// thread copies it to TMEM with tcgen05.cp (32x128b.warpx4) and selects the step's byte with the
// scale-factor-id fields of the instruction descriptor.  Shared-memory chunk buffers form a ring of
// four, TMEM scale columns are double-buffered by chunk parity.
//
//   warp 0      TMA producer (both CTAs; bytes counted on the even CTA's barrier)
//   warp 1      MMA issuer (even CTA): tcgen05.cp of scale chunks, eight M256 N128 K32 MMAs per step
//   warp 2      TMEM allocator (512 columns: 256 accumulator, 32 scale factors)
//   warps 4-11  scale staging during the main loop, then the epilogue (TMEM -> bf16 -> global)
//
// TMA loads read this GPU's memory only and carry no cluster multicast.  Every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels/grouped_gemm_internal.h"
#include "kernels/tcgen05_ptx.cuh"

namespace {

using namespace nixl_tc;
using nixl_gemm::GEMM_ERR_TIMEOUT;
using nixl_gemm::kMaxGroups;

constexpr int BM = 128;        // rows per CTA (256 per pair)
constexpr int BN = 256;        // tile columns
constexpr int BNS = 128;       // columns per instruction group / accumulator half
constexpr int WBOX = 64;       // W rows per TMA box (per CTA and column half)
constexpr int BK = 128;
constexpr int kStages = 6;
constexpr int kThreads = 384;
constexpr int kATileBytes = BM * BK;
constexpr int kWBoxBytes = WBOX * BK;
constexpr int kStageBytes = kATileBytes + 2 * kWBoxBytes; // 32 KiB per CTA
constexpr int kChunkSteps = 4;                 // steps whose scale bytes share one 32-bit word
constexpr int kSfRing = 4;                     // chunk buffers in shared memory
constexpr int kSfAtomBytes = 512;              // 128 rows x 4 steps
constexpr int kSfBufBytes = 3 * kSfAtomBytes;  // A, W left half, W right half
constexpr int kTmemCols = 512;
constexpr int kAccCols = 2 * BNS;              // accumulator: columns [0, 256)
constexpr int kSfTmemStride = 16;              // scale columns of a chunk parity: [256 + 16 p, ...): A +0, W left +4, W right +8
constexpr int kPromoWarps = 8;

struct Shared {
    uint64_t full[kStages];      // even CTA: both CTAs' operand bytes of a stage have landed
    uint64_t empty[kStages];     // per CTA: the MMAs that read the stage are done
    uint64_t sfFull[kSfRing];    // even CTA: both CTAs have staged the chunk's scale layouts (16 warp arrivals)
    uint64_t sfEmpty[kSfRing];   // per CTA: the chunk buffer has been copied to TMEM
    uint64_t tmemFull;           // per CTA: a tile's accumulator is complete
    uint64_t tmemEmpty;          // even CTA: all 16 epilogue warps have read the accumulator
    uint32_t tmemBase;
    int abort;
    volatile uint32_t chunksIssued; // two issuing threads take turns chunk by chunk: the next chunk whose MMAs may enter the pipe
    int tilePrefix[kMaxGroups + 1];
    int rowStart[kMaxGroups];
    int rowCount[kMaxGroups];
};

__device__ __forceinline__ uint32_t clusterCtaRank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapToCta(uint32_t smem_addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void clusterSync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Relaxed on purpose: a release at cluster scope made the arriving thread wait several hundred
// cycles, once per slot.  What the arrive has to order are this warp's TMEM reads, and those are
// complete (tcgen05.wait::ld returned, the values are in registers) before it is issued.
__device__ __forceinline__ void mbarArriveCluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tile load whose completion bytes are counted on a barrier given by its cluster address
// (the even CTA's), as the paired MMA needs both halves before it may start.
__device__ __forceinline__ void tmaLoad2dPair(void *smem_dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smemU32(smem_dst)),
                 "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void mbarArriveClusterRelease(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tcCommitPair(uint32_t bar_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar_addr),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
}
// Shared-memory descriptor of one 512-byte scale layout: 32 rows of 16 bytes, no swizzle, 8-row
// groups 128 bytes apart.
__device__ __forceinline__ uint64_t sfDesc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(128 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}
// 32 x 128 bit from shared memory into four TMEM columns, replicated to all four lane quarters, in
// both CTAs of the pair (each from its own shared memory).
__device__ __forceinline__ void tmemCpPair(uint32_t tmem_dst, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(desc) : "memory");
}
// D fp32, A and B e4m3 K-major, M = 256 (both CTAs), N = 128, scale factors E8M0, scale-factor id `sf` for A and B.
__device__ __forceinline__ uint32_t instrDescMx(uint32_t sf) {
    return (sf << 4) | (static_cast<uint32_t>(BNS >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>((2 * BM) >> 4) << 24) | (sf << 29);
}

// One 128-channel step: eight block-scaled MMAs (four per accumulator half) and the commit that frees
// the stage.  The non-blocking test of the next step's barrier sits between the two groups of
// MMAs: its latency then runs while the second group is being issued, and its result is read last.
__device__ __forceinline__ void issueKStepMx(uint32_t tmem_d0, uint32_t tmem_d1, uint64_t da, uint64_t dw0, uint64_t dw1, uint32_t idesc, uint32_t tsfa,
                                             uint32_t tsfb0, uint32_t tsfb1, uint32_t accumulate, uint32_t bar_stage_empty, uint32_t peek_bar,
                                             uint32_t peek_par, uint32_t &ready_next, uint32_t peek2_bar, uint32_t peek2_par, uint32_t &ready2) {
    uint64_t da2 = da;
    asm volatile(
        "{\n"
        " .reg .pred pf, pf2, pacc, pfirst;\n"
        " setp.ne.b32 pacc, %16, 0;\n"
        " setp.ne.b32 pfirst, %12, 0;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%2], %4, %5, %8, [%9], [%10], pfirst;\n"
        " add.u64 %4, %4, 2;\n add.u64 %5, %5, 2;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%2], %4, %5, %8, [%9], [%10], pacc;\n"
        " add.u64 %4, %4, 2;\n add.u64 %5, %5, 2;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%2], %4, %5, %8, [%9], [%10], pacc;\n"
        " add.u64 %4, %4, 2;\n add.u64 %5, %5, 2;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%2], %4, %5, %8, [%9], [%10], pacc;\n"
        " mbarrier.test_wait.parity.shared::cta.b64 pf, [%14], %15;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%3], %7, %6, %8, [%9], [%11], pfirst;\n"
        " add.u64 %7, %7, 2;\n add.u64 %6, %6, 2;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%3], %7, %6, %8, [%9], [%11], pacc;\n"
        " mbarrier.test_wait.parity.shared::cta.b64 pf2, [%18], %19;\n"
        " add.u64 %7, %7, 2;\n add.u64 %6, %6, 2;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%3], %7, %6, %8, [%9], [%11], pacc;\n"
        " add.u64 %7, %7, 2;\n add.u64 %6, %6, 2;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%3], %7, %6, %8, [%9], [%11], pacc;\n"
        " tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%13], %17;\n"
        " selp.u32 %0, 1, 0, pf;\n"
        " selp.u32 %1, 1, 0, pf2;\n"
        "}\n"
        : "=r"(ready_next), "=r"(ready2), "+r"(tmem_d0), "+r"(tmem_d1), "+l"(da), "+l"(dw0), "+l"(dw1), "+l"(da2)
        : "r"(idesc), "r"(tsfa), "r"(tsfb0), "r"(tsfb1), "r"(accumulate), "r"(bar_stage_empty), "r"(peek_bar), "r"(peek_par), "r"(1u),
          "h"(static_cast<uint16_t>(3)), "r"(peek2_bar), "r"(peek2_par)
        : "memory");
}

struct Tile {
    int g, mt, nt;
};

__device__ __forceinline__ bool tileAt(const Shared &sh, int groups, int n_tiles, int t, Tile &out) {
    if (t >= sh.tilePrefix[groups]) return false;
    int lo = 0, hi = groups;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (sh.tilePrefix[mid] <= t) lo = mid; else hi = mid;
    }
    const int local = t - sh.tilePrefix[lo];
    out.g = lo;
    out.mt = local / n_tiles;
    out.nt = local - out.mt * n_tiles;
    return true;
}

__global__ void __launch_bounds__(kThreads, 1)
groupedGemmMxPairKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapW, const NixlGroupedGemmParams p) {
    extern __shared__ __align__(1024) unsigned char dyn[];
    unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~uintptr_t(1023));
    unsigned char *sf_ring = tiles + kStages * kStageBytes; // kSfRing buffers of {A, W left, W right} layouts
    Shared &sh = *reinterpret_cast<Shared *>(sf_ring + kSfRing * kSfBufBytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.N / BN, k_steps = p.K / BK;
    const int chunks = k_steps / kChunkSteps; // K is a multiple of 512
    const uint32_t cta = clusterCtaRank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbarInit(&sh.full[s], 1);
            mbarInit(&sh.empty[s], 1);
        }
        for (int b = 0; b < kSfRing; ++b) {
            mbarInit(&sh.sfFull[b], 2 * kPromoWarps);
            mbarInit(&sh.sfEmpty[b], 1);
        }
        mbarInit(&sh.tmemFull, 2); // one commit from each issuing thread
        mbarInit(&sh.tmemEmpty, 2 * kPromoWarps);
        sh.abort = 0;
        sh.chunksIssued = 0;
        int run = 0;
        for (int g = 0; g < p.groups; ++g) {
            const int c = p.row_count[g];
            sh.tilePrefix[g] = run;
            sh.rowStart[g] = p.row_start[g];
            sh.rowCount[g] = c;
            run += ((c + 2 * BM - 1) / (2 * BM)) * n_tiles;
        }
        sh.tilePrefix[p.groups] = run;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemU32(&sh.tmemBase)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    }
    tcFenceBefore();
    __syncthreads();
    clusterSync();
    tcFenceAfter();
    const uint32_t tmem = sh.tmemBase;
    volatile int *abort_flag = &sh.abort;
    int my_tiles = 0;
    {
        const int total = sh.tilePrefix[p.groups];
        if (pair < total) my_tiles = (total - pair + pairs - 1) / pairs;
    }

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        const uint32_t full0 = mapToCta(smemU32(&sh.full[0]), 0);
        uint32_t it = 0;
        Tile t;
        for (int ti = pair; tileAt(sh, p.groups, n_tiles, ti, t); ti += pairs) {
            const int row0 = sh.rowStart[t.g] + t.mt * (2 * BM) + static_cast<int>(cta) * BM;
            const int wrow = t.g * p.N + t.nt * BN + static_cast<int>(cta) * WBOX;
            for (int ks = 0; ks < k_steps; ++ks, ++it) {
                const int s = it % kStages;
                if (!mbarWait(&sh.empty[s], ((it / kStages) & 1) ^ 1, abort_flag)) goto producer_done;
                if (cta == 0) mbarExpectTx(&sh.full[s], 2 * kStageBytes);
                const uint32_t bar = full0 + static_cast<uint32_t>(s) * 8u;
                unsigned char *st = tiles + s * kStageBytes;
                tmaLoad2dPair(st, &mapA, ks * BK, row0, bar);
                tmaLoad2dPair(st + kATileBytes, &mapW, ks * BK, wrow, bar);
                tmaLoad2dPair(st + kATileBytes + kWBoxBytes, &mapW, ks * BK, wrow + BNS, bar);
            }
        }
    producer_done:;
    } else if ((warp == 1 || warp == 3) && lane == 0 && cta == 0) {
        // ---------------------------------------------------------------- two MMA issuers (even CTA)
        // The tensor pipe idles whenever its issuing thread does anything but issue (an MMA's issue
        // returns about when its predecessor starts).  Two threads therefore alternate chunk by chunk
        // (four steps, 32 MMAs): while one is parked in the issue of its chunk, the other waits for its
        // next chunk's barriers and sits ready.  A turn counter keeps the chunks entering the pipe in
        // order (the first step of a tile overwrites the accumulator, and a chunk's scale copy must
        // precede its MMAs); even chunks use TMEM scale columns of parity 0, odd chunks parity 1.
        const uint32_t me = warp == 1 ? 0u : 1u;
        const uint32_t full_bar0 = smemU32(&sh.full[0]), empty_bar0 = smemU32(&sh.empty[0]), sfempty_bar0 = smemU32(&sh.sfEmpty[0]);
        const uint64_t desc0 = smemDesc(smemU32(tiles));
        const uint32_t sf_smem0 = smemU32(sf_ring);
        const uint32_t total_chunks = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(chunks);
        for (uint32_t cc = me; cc < total_chunks; cc += 2) {
            const uint32_t tile = cc / static_cast<uint32_t>(chunks), c = cc - tile * static_cast<uint32_t>(chunks);
            const uint32_t it0 = cc * kChunkSteps;
            uint32_t s = it0 % kStages, full_par = (it0 / kStages) & 1u;
            const uint32_t b = cc % kSfRing;
            // Everything this chunk depends on, before asking for the turn.
            if (c == 0 && !mbarWait(&sh.tmemEmpty, (tile & 1u) ^ 1u, abort_flag)) goto issuer_done; // accumulator drained by the previous epilogue
            if (!mbarWait(&sh.sfFull[b], (cc / kSfRing) & 1u, abort_flag)) goto issuer_done;
            if (!mbarWait(&sh.full[s], full_par, abort_flag)) goto issuer_done;
            {
                const long long t0 = clock64();
                while (sh.chunksIssued != cc) {
                    if (*abort_flag) goto issuer_done;
                    if (clock64() - t0 > (1ll << 33)) {
                        *abort_flag = 1;
                        goto issuer_done;
                    }
                }
            }
            tcFenceAfter();
            const uint32_t src = sf_smem0 + b * kSfBufBytes;
            const uint32_t sfc = tmem + kAccCols + (cc & 1u) * kSfTmemStride;
            tmemCpPair(sfc, sfDesc(src));
            tmemCpPair(sfc + 4, sfDesc(src + kSfAtomBytes));
            tmemCpPair(sfc + 8, sfDesc(src + 2 * kSfAtomBytes));
            tcCommitPair(sfempty_bar0 + b * 8u); // the buffer may be refilled once the copies have read it
            uint32_t ready = 1; // the first step's barrier was waited for above
#pragma unroll
            for (uint32_t sub = 0; sub < kChunkSteps; ++sub) {
                if (!ready && !mbarWait(&sh.full[s], full_par, abort_flag)) goto issuer_done;
                tcFenceAfter();
                uint32_t ns = s + 1, nfull_par = full_par;
                if (ns == kStages) {
                    ns = 0;
                    nfull_par ^= 1u;
                }
                const uint64_t da = desc0 + static_cast<uint64_t>((s * kStageBytes) >> 4);
                const uint64_t dw0 = da + static_cast<uint64_t>(kATileBytes >> 4);
                const uint64_t dw1 = da + static_cast<uint64_t>((kATileBytes + kWBoxBytes) >> 4);
                uint32_t unused = 0;
                issueKStepMx(tmem, tmem + BNS, da, dw0, dw1, instrDescMx(sub), sfc, sfc + 4, sfc + 8, (c | sub) ? 1u : 0u, empty_bar0 + s * 8u,
                             full_bar0 + ns * 8u, nfull_par, ready, full_bar0 + ns * 8u, nfull_par, unused);
                s = ns;
                full_par = nfull_par;
            }
            // All of this chunk's MMAs are in the pipe: the other thread's chunk may follow.
            asm volatile("" ::: "memory");
            sh.chunksIssued = cc + 1;
            if (c + 1 == static_cast<uint32_t>(chunks) || c + 2 == static_cast<uint32_t>(chunks)) {
                // This thread's last chunk of the tile: its share of "accumulator complete" (both shares when
                // the tile has a single chunk and the other thread never touches it).
                tcCommitPair(smemU32(&sh.tmemFull));
                if (chunks == 1) tcCommitPair(smemU32(&sh.tmemFull));
            }
        }
    issuer_done:;
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- scale staging, then the epilogue
        const int q = warp & 3;
        const int part = (warp - 4) >> 2; // 0: stages A's layout, 1: stages W's two layouts; epilogue: 64-column part of each half
        const int row_in_tile = q * 32 + lane;
        const uint32_t sffull0 = mapToCta(smemU32(&sh.sfFull[0]), 0);
        const uint32_t tempty = mapToCta(smemU32(&sh.tmemEmpty), 0);
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(q * 32) << 16) + part * 64;
        const uint32_t *sa32 = reinterpret_cast<const uint32_t *>(p.scale_a);
        const uint32_t *sw32 = reinterpret_cast<const uint32_t *>(p.scale_w);
        const int n_blocks = p.N / 128;
        // Rows and scale words of a tile, as this thread sees them.
        struct TileView {
            Tile t;
            bool valid;
            long long grow;
        };
        auto view = [&](int ti, TileView &v) -> bool {
            if (!tileAt(sh, p.groups, n_tiles, ti, v.t)) return false;
            const int local_row = v.t.mt * (2 * BM) + static_cast<int>(cta) * BM + row_in_tile;
            v.valid = local_row < sh.rowCount[v.t.g];
            v.grow = static_cast<long long>(sh.rowStart[v.t.g]) + local_row;
            return true;
        };
        // Builds chunk c of a tile in ring buffer gcc % kSfRing once the issuer has copied that buffer's previous content out.
        auto stage = [&](const TileView &v, int c, uint32_t gcc) -> bool {
            const uint32_t b = gcc % kSfRing;
            if (!mbarWait(&sh.sfEmpty[b], ((gcc / kSfRing) & 1u) ^ 1u, abort_flag)) return false;
            uint32_t *buf = reinterpret_cast<uint32_t *>(sf_ring + b * kSfBufBytes);
            if (part == 0) {
                // Row r of this CTA's half: word (r % 32) * 4 + r / 32 (rows beyond the expert get exponent 127 = 1.0).
                buf[lane * 4 + q] = v.valid ? __ldg(sa32 + v.grow * chunks + c) : 0x7f7f7f7fu;
            } else {
                const long long blk = (static_cast<long long>(v.t.g) * n_blocks + v.t.nt * 2) * chunks + c;
                buf[128 + row_in_tile] = __ldg(sw32 + blk);
                buf[256 + row_in_tile] = __ldg(sw32 + blk + chunks);
            }
            asm volatile("fence.proxy.async;" ::: "memory"); // these generic-proxy writes are read by tcgen05.cp
            __syncwarp();
            if (lane == 0) mbarArriveClusterRelease(sffull0 + b * 8u);
            return true;
        };
        // Staging runs ahead of the issuer by up to the ring's depth, across tile boundaries: the first
        // chunks of the next tile are built before this tile's epilogue, so the issuer finds them
        // waiting when the accumulator is free again.
        const int ahead = chunks < kSfRing ? chunks : kSfRing;
        TileView cur, nxt;
        int ti = pair;
        bool have = view(ti, cur);
        uint32_t cc_base = 0;
        bool ok = true;
        if (have)
            for (int c = 0; c < ahead && ok; ++c) ok = stage(cur, c, cc_base + c);
        for (int tile = 0; have && ok; ++tile) {
            for (int c = ahead; c < chunks && ok; ++c) ok = stage(cur, c, cc_base + c);
            const bool have_next = view(ti + pairs, nxt);
            if (have_next)
                for (int c = 0; c < ahead && ok; ++c) ok = stage(nxt, c, cc_base + chunks + c);
            if (!ok) break;
            const Tile &t = cur.t;
            // Epilogue: the tile's accumulator, two halves of 128 columns, this warp's 64 columns of each.
            // All four TMEM loads first, then the accumulator goes back to the issuer at once; conversion
            // and stores follow while the next tile's main loop is already running.
            if (!mbarWait(&sh.tmemFull, static_cast<uint32_t>(tile) & 1u, abort_flag)) break;
            tcFenceAfter();
            float v0[32], v1[32], v2[32], v3[32];
            tmemLoad32(lane_base, v0);
            tmemLoad32(lane_base + 32, v1);
            tmemLoad32(lane_base + BNS, v2);
            tmemLoad32(lane_base + BNS + 32, v3);
            tmemLoadWait(v0);
            tmemLoadWait(v1);
            tmemLoadWait(v2);
            tmemLoadWait(v3);
            tcFenceBefore();
            __syncwarp();
            if (lane == 0) mbarArriveCluster(tempty);
            // A thread holds 64 consecutive columns of its own row: eight 16-byte pieces per half.  Eight
            // lanes exchange pieces (8 x 8 transpose by three butterfly steps) so that every store
            // instruction writes whole 128-byte runs: lane 8g + c then holds piece c of rows 8g .. 8g + 7.
            const int first_row = t.mt * (2 * BM) + static_cast<int>(cta) * BM + q * 32 + (lane & ~7); // tile-local row of this lane group
            const long long first_grow = static_cast<long long>(sh.rowStart[t.g]) + first_row;
            const int rows_left = sh.rowCount[t.g] - first_row; // rows of the group that belong to the expert
            __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.d) + first_grow * p.N + t.nt * BN + part * 64 + (lane & 7) * 8;
            storeRows64(v0, v1, out, p.N, rows_left, lane);
            storeRows64(v2, v3, out + BNS, p.N, rows_left, lane);
            cur = nxt;
            have = have_next;
            ti += pairs;
            cc_base += static_cast<uint32_t>(chunks);
        }
    }

    tcFenceBefore();
    __syncthreads();
    clusterSync();
    if (threadIdx.x == 0 && sh.abort) atomicOr(p.status, GEMM_ERR_TIMEOUT);
    if (warp == 2) {
        tcFenceAfter();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
    }
}

} // namespace

cudaError_t nixl_gemm::launchMxPairKernel(const CUtensorMap &mapA, const CUtensorMap &mapW, const NixlGroupedGemmParams &p, cudaStream_t stream) {
    const size_t smem = size_t(kStages) * kStageBytes + size_t(kSfRing) * kSfBufBytes + sizeof(Shared) + 1024;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    static bool attr_done[64] = {};
    static int max_pairs[64] = {};
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(groupedGemmMxPairKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1));
        int clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&clusters, groupedGemmMxPairKernel, &cfg);
        if (e != cudaSuccess || clusters <= 0) {
            cudaGetLastError();
            clusters = sms / 2;
        }
        max_pairs[dev] = clusters;
        attr_done[dev] = true;
    }
    int pairs = (dev >= 0 && dev < 64) ? max_pairs[dev] : sms / 2;
    if (p.grid > 0 && p.grid / 2 < pairs) pairs = p.grid / 2 > 0 ? p.grid / 2 : 1;
    const long long max_tiles = (static_cast<long long>(p.a_rows + 2 * BM - 1) / (2 * BM) + p.groups) * (p.N / BN);
    if (pairs > max_tiles) pairs = static_cast<int>(max_tiles);
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    return cudaLaunchKernelEx(&cfg, groupedGemmMxPairKernel, mapA, mapW, p);
}

// Grouped fp8 expert GEMM, 256 x 256 output tiles computed by CTA pairs (tcgen05 cta_group::2).
//
// Same math and operand formats as grouped_gemm_fp8.cu.  Two CTAs of a cluster share one tile:
// each loads its own 128 rows of A and 128 of the tile's 256 W rows per 128-channel step (32 KiB
// per CTA and step: half the L2 -> shared-memory traffic per MAC of 128 x 128 tiles), the even CTA
// issues M256 N128 K32 MMAs that read both CTAs' shared memory and write both CTAs' TMEM, and each
// CTA promotes and stores its own 128 rows.
//
// A 128-channel step is eight MMAs: four into one 128-column TMEM slot for the left half of the
// tile's columns and four into a second slot for the right half; two steps (four slots, all of
// TMEM) are in flight.  To make the two N = 128 instruction groups cover contiguous columns, CTA c
// keeps W rows [64c, 64c+64) of the left half and of the right half (two 64-row TMA boxes).
//
// What bounds this kernel is not the tensor pipe (eight MMAs take 512 cycles) but the hand-offs
// around it, so they are kept to a minimum:
//  * the issuing thread polls one barrier per step.  full[s] collects the producer's arrival (with
//    both CTAs' byte count) and one arrival from each of the pair's sixteen promotion warps, sent
//    when the warp has read the two slots the step will overwrite;
//  * that poll is a non-blocking test issued behind the previous step's MMAs: barrier instructions
//    in front of the MMAs delayed them by a few hundred cycles each;
//  * promotion warps poll once per step too (one commit covers both slots), arrive with relaxed
//    semantics (a cluster-scope release cost several hundred cycles per arrive) and fetch their
//    scales behind the arrive;
//  * ring positions are counters, not divisions, on the single-thread roles.
//
//   warp 0      TMA producer (both CTAs; completion bytes are counted on the even CTA's barrier)
//   warp 1      MMA issuer (even CTA only); commits are multicast to both CTAs' barriers
//   warp 2      TMEM allocator (512 columns, cta_group::2)
//   warps 4-11  promotion + epilogue: lane quarter q = warp % 4, 64-column part (warp - 4) / 4 of
//               every slot; 128 fp32 accumulators per thread, so these warps raise their register
//               budget (setmaxnreg 232) with what the role warps give back (setmaxnreg 40; the two
//               budgets must leave the register file some slack, an exact fit never got its
//               increase granted)
//
// TMA loads read this GPU's memory only and carry no cluster multicast.  Every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels/grouped_gemm_internal.h"
#include "kernels/tcgen05_ptx.cuh"

namespace {

using namespace nixl_tc;
using nixl_gemm::GEMM_ERR_ARRIVAL;
using nixl_gemm::GEMM_ERR_TIMEOUT;
using nixl_gemm::kMaxGroups;

constexpr int BM = 128;        // rows per CTA (256 per pair)
constexpr int BN = 256;        // tile columns
constexpr int BNS = 128;       // columns per half-step / TMEM slot
constexpr int WBOX = 64;       // W rows per TMA box (per CTA and column half)
constexpr int BK = 128;
constexpr int kStages = 6;
constexpr int kThreads = 384;
constexpr int kATileBytes = BM * BK;           // 16 KiB
constexpr int kWBoxBytes = WBOX * BK;          // 8 KiB
constexpr int kStageBytes = kATileBytes + 2 * kWBoxBytes; // 32 KiB per CTA
constexpr int kSlots = 4;
constexpr int kTmemCols = kSlots * BNS;        // 512
constexpr int kPromoWarps = 8;
// A step's full[] barrier collects the producer's arrival (which carries both CTAs' byte count) and
// one arrival from every promotion warp of the pair, sent when the warp has read the two TMEM
// slots the step is going to overwrite (the slots of the step two before it).
constexpr int kFullArrivals = 1 + 2 * kPromoWarps;

struct Shared {
    uint64_t full[kStages];       // used on the even CTA: a step may be issued (see kFullArrivals)
    uint64_t empty[kStages];      // per CTA: the MMAs that read the stage are done
    uint64_t tmemFull[2];         // per CTA: the two slots of an even / odd step are ready for promotion
    uint32_t tmemBase;
    int abort;
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
// A whole 128-channel step of the issuer as one instruction sequence: eight MMAs (four per TMEM
// slot), the two commits, and then a non-blocking test of the next step's barrier.  Barrier
// instructions placed in front of the MMAs delayed them by a few hundred cycles each, so the only
// poll of a step sits behind its MMAs, where the tensor pipe still has work queued.
__device__ __forceinline__ void issueKStep(uint32_t tmem_d0, uint32_t tmem_d1, uint64_t da, uint64_t dw0, uint64_t dw1, uint32_t idesc,
                                           uint32_t bar_tmem_full, uint32_t bar_stage_empty, uint32_t peek_bar, uint32_t peek_par,
                                           uint32_t &ready_next) {
    uint64_t da2 = da;
    asm volatile(
        "{\n"
        " .reg .pred pf, pacc, pnew;\n"
        " setp.ne.b32 pacc, %12, 0;\n"
        " setp.eq.b32 pnew, %12, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%1], %3, %4, %7, {%13, %13, %13, %13, %13, %13, %13, %13}, pnew;\n"
        " add.u64 %3, %3, 2;\n add.u64 %4, %4, 2;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%1], %3, %4, %7, {%13, %13, %13, %13, %13, %13, %13, %13}, pacc;\n"
        " add.u64 %3, %3, 2;\n add.u64 %4, %4, 2;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%1], %3, %4, %7, {%13, %13, %13, %13, %13, %13, %13, %13}, pacc;\n"
        " add.u64 %3, %3, 2;\n add.u64 %4, %4, 2;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%1], %3, %4, %7, {%13, %13, %13, %13, %13, %13, %13, %13}, pacc;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%2], %6, %5, %7, {%13, %13, %13, %13, %13, %13, %13, %13}, pnew;\n"
        " add.u64 %6, %6, 2;\n add.u64 %5, %5, 2;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%2], %6, %5, %7, {%13, %13, %13, %13, %13, %13, %13, %13}, pacc;\n"
        " add.u64 %6, %6, 2;\n add.u64 %5, %5, 2;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%2], %6, %5, %7, {%13, %13, %13, %13, %13, %13, %13, %13}, pacc;\n"
        " add.u64 %6, %6, 2;\n add.u64 %5, %5, 2;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%2], %6, %5, %7, {%13, %13, %13, %13, %13, %13, %13, %13}, pacc;\n"
        " tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%8], %14;\n"
        " tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%9], %14;\n"
        " mbarrier.test_wait.parity.shared::cta.b64 pf, [%10], %11;\n"
        " selp.u32 %0, 1, 0, pf;\n"
        "}\n"
        : "=r"(ready_next), "+r"(tmem_d0), "+r"(tmem_d1), "+l"(da), "+l"(dw0), "+l"(dw1), "+l"(da2)
        : "r"(idesc), "r"(bar_tmem_full), "r"(bar_stage_empty), "r"(peek_bar), "r"(peek_par), "r"(1u), "r"(0u), "h"(static_cast<uint16_t>(3))
        : "memory");
}

// D fp32, A and B e4m3, both K-major, M = 256 (both CTAs), N = 128.
__device__ __forceinline__ constexpr uint32_t instrDescPair() {
    return (1u << 4) | (static_cast<uint32_t>(BNS >> 3) << 17) | (static_cast<uint32_t>((2 * BM) >> 4) << 24);
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
groupedGemmPairKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapW, const NixlGroupedGemmParams p) {
    extern __shared__ __align__(1024) unsigned char dyn[];
    unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~uintptr_t(1023));
    Shared &sh = *reinterpret_cast<Shared *>(tiles + kStages * kStageBytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.N / BN, k_steps = p.K / BK;
    const uint32_t cta = clusterCtaRank(); // 0: issues the MMAs, 1: its partner
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbarInit(&sh.full[s], kFullArrivals);
            mbarInit(&sh.empty[s], 1);
        }
        mbarInit(&sh.tmemFull[0], 1);
        mbarInit(&sh.tmemFull[1], 1);
        // The first two steps find their slots free: stand in for the promotion warps' arrivals.
        for (int s = 0; s < 2; ++s)
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smemU32(&sh.full[s])), "r"(2 * kPromoWarps) : "memory");
        sh.abort = 0;
        int run = 0;
        if (p.counts_flag) {
            for (int r = 0; r < p.ranks; ++r) {
                uint64_t t0 = 0;
                unsigned spins = 0;
                while (ldAcquireSys(p.counts_flag + r) < p.epoch) {
                    if ((++spins & 63u) == 0) {
                        const uint64_t now = nowNs();
                        if (t0 == 0) t0 = now;
                        else if (now - t0 > p.timeout_ns) {
                            atomicOr(p.status, GEMM_ERR_ARRIVAL);
                            break;
                        }
                    }
                }
            }
            int next = 0;
            for (int g = 0; g < p.groups; ++g) {
                int c = 0;
                for (int r = 0; r < p.ranks; ++r) c += p.counts[static_cast<long long>(r) * p.experts_total + p.expert_base + g];
                sh.tilePrefix[g] = run;
                sh.rowStart[g] = p.rows_per_expert > 0 ? g * p.rows_per_expert : next;
                sh.rowCount[g] = c;
                next += c;
                run += ((c + 2 * BM - 1) / (2 * BM)) * n_tiles;
            }
        } else {
            for (int g = 0; g < p.groups; ++g) {
                const int c = p.row_count[g];
                sh.tilePrefix[g] = run;
                sh.rowStart[g] = p.row_start[g];
                sh.rowCount[g] = c;
                run += ((c + 2 * BM - 1) / (2 * BM)) * n_tiles;
            }
        }
        sh.tilePrefix[p.groups] = run;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        // Both CTAs of the pair issue the paired allocation from the same warp and shared offset.
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemU32(&sh.tmemBase)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    }
    tcFenceBefore();
    __syncthreads();
    clusterSync(); // the partner's barriers exist before anything arrives on them
    tcFenceAfter();
    const uint32_t tmem = sh.tmemBase;
    volatile int *abort_flag = &sh.abort;
    // k-steps this pair executes in total (every tile has k_steps of them)
    int my_tiles = 0;
    {
        const int total = sh.tilePrefix[p.groups];
        if (pair < total) my_tiles = (total - pair + pairs - 1) / pairs;
    }

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------------------ TMA producer (both CTAs)
            const uint32_t full0 = mapToCta(smemU32(&sh.full[0]), 0);
            uint32_t it = 0;
            Tile t;
            for (int ti = pair; tileAt(sh, p.groups, n_tiles, ti, t); ti += pairs) {
                const int row0 = sh.rowStart[t.g] + t.mt * (2 * BM) + static_cast<int>(cta) * BM;
                if (p.disp_flag) {
                    const int lo = t.mt * (2 * BM) + static_cast<int>(cta) * BM, hi = min(lo + BM, sh.rowCount[t.g]);
                    int first = 0;
                    for (int r = 0; r < p.ranks; ++r) {
                        const int c = p.counts[static_cast<long long>(r) * p.experts_total + p.expert_base + t.g];
                        if (c > 0 && first < hi && first + c > lo) {
                            const uint64_t *flag = p.disp_flag + static_cast<long long>(t.g) * p.ranks + r;
                            uint64_t t0 = 0;
                            unsigned spins = 0;
                            while (ldAcquireSys(flag) < p.epoch) {
                                if ((++spins & 63u) == 0) {
                                    const uint64_t now = nowNs();
                                    if (t0 == 0) t0 = now;
                                    else if (now - t0 > p.timeout_ns) {
                                        atomicOr(p.status, GEMM_ERR_ARRIVAL);
                                        break;
                                    }
                                }
                            }
                        }
                        first += c;
                    }
                    asm volatile("fence.proxy.async;" ::: "memory");
                }
                const int wrow = t.g * p.N + t.nt * BN + static_cast<int>(cta) * WBOX;
                for (int ks = 0; ks < k_steps; ++ks, ++it) {
                    const int s = it % kStages;
                    if (!mbarWait(&sh.empty[s], ((it / kStages) & 1) ^ 1, abort_flag)) goto role_done;
                    if (cta == 0) mbarExpectTx(&sh.full[s], 2 * kStageBytes); // both CTAs' shares
                    const uint32_t bar = full0 + static_cast<uint32_t>(s) * 8u;
                    unsigned char *st = tiles + s * kStageBytes;
                    tmaLoad2dPair(st, &mapA, ks * BK, row0, bar);
                    tmaLoad2dPair(st + kATileBytes, &mapW, ks * BK, wrow, bar);               // columns [64c, 64c+64) of the left half
                    tmaLoad2dPair(st + kATileBytes + kWBoxBytes, &mapW, ks * BK, wrow + BNS, bar); // and of the right half
                }
            }
        } else if (warp == 1 && lane == 0 && cta == 0) {
            // ------------------------------------------------------------ MMA issuer (even CTA)
            // One poll per eight MMAs: full[s] completes when both CTAs' bytes have landed and all
            // promotion warps of the pair have read the step's two TMEM slots.
            const uint32_t ksteps_total = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(k_steps);
            uint32_t s = 0, full_par = 0, sl = 0; // ring positions as counters: no divisions on this thread
            uint32_t ready = 0;
            const uint32_t full_bar0 = smemU32(&sh.full[0]), empty_bar0 = smemU32(&sh.empty[0]), tfull_bar0 = smemU32(&sh.tmemFull[0]);
            const uint64_t desc0 = smemDesc(smemU32(tiles));
            for (uint32_t it = 0; it < ksteps_total; ++it) {
                if (!ready && !mbarWait(&sh.full[s], full_par, abort_flag)) goto role_done;
                tcFenceAfter();
                uint32_t ns = s + 1, nfull_par = full_par;
                if (ns == kStages) {
                    ns = 0;
                    nfull_par ^= 1u;
                }
                const uint64_t da = desc0 + static_cast<uint64_t>((s * kStageBytes) >> 4);
                const uint64_t dw0 = da + static_cast<uint64_t>(kATileBytes >> 4);
                const uint64_t dw1 = da + static_cast<uint64_t>((kATileBytes + kWBoxBytes) >> 4);
                issueKStep(tmem + sl * BNS, tmem + (sl + 1) * BNS, da, dw0, dw1, instrDescPair(), tfull_bar0 + (sl >> 1) * 8u, empty_bar0 + s * 8u,
                           full_bar0 + ns * 8u, nfull_par, ready);
                sl ^= 2u;
                s = ns;
                full_par = nfull_par;
            }
        }
    role_done:;
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        // ---------------------------------------------------------------- promotion + epilogue
        const int q = warp & 3;
        const int part = (warp - 4) >> 2; // which 64 of a slot's 128 columns
        const int row_in_tile = q * 32 + lane;
        const uint32_t full0 = mapToCta(smemU32(&sh.full[0]), 0);
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(q * 32) << 16) + part * 64;
        uint32_t it = 0;      // step counter, same numbering as the issuer's
        uint32_t s2 = 2;      // stage of step it + 2, the step that reuses this step's slots
        Tile t;
        const int n_blocks = p.N / 128;
        bool rdy = false;
        bool ok = true;
        for (int ti = pair; ok && tileAt(sh, p.groups, n_tiles, ti, t); ti += pairs) {
            const int local_row = t.mt * (2 * BM) + static_cast<int>(cta) * BM + row_in_tile;
            const bool valid = local_row < sh.rowCount[t.g];
            const long long grow = static_cast<long long>(sh.rowStart[t.g]) + local_row;
            const float *sa_row = p.scale_a + grow * k_steps;
            const float *sw0 = p.scale_w + (static_cast<long long>(t.g) * n_blocks + t.nt * 2) * k_steps;
            const float *sw1 = sw0 + k_steps;
            float acc[2 * 64];
#pragma unroll
            for (int i = 0; i < 2 * 64; ++i) acc[i] = 0.f;
            // Scales are fetched kPrefetch steps ahead and kept as loaded: multiplying them right away
            // would make the warp wait for the loads it has just issued.
            constexpr int kPrefetch = 4;
            float ring_a[kPrefetch], ring_w0[kPrefetch], ring_w1[kPrefetch];
#pragma unroll
            for (int i = 0; i < kPrefetch; ++i) {
                ring_a[i] = (i < k_steps && valid) ? __ldg(sa_row + i) : 0.f;
                ring_w0[i] = i < k_steps ? __ldg(sw0 + i) : 0.f;
                ring_w1[i] = i < k_steps ? __ldg(sw1 + i) : 0.f;
            }
            for (int ks0 = 0; ks0 < k_steps && ok; ks0 += kPrefetch) {
#pragma unroll
                for (int i = 0; i < kPrefetch; ++i, ++it) {
                    const int ks = ks0 + i;
                    if (ks >= k_steps) break;
                    const float s0 = ring_a[i] * ring_w0[i], s1 = ring_a[i] * ring_w1[i];
                    const int nxt = ks + kPrefetch;
                    const uint32_t kp = it & 1u, sl = kp * 2u;
                    if (!rdy && !mbarWait(&sh.tmemFull[kp], (it >> 1) & 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tcFenceAfter();
                    float v0[32], v1[32];
                    tmemLoad32(lane_base + sl * BNS, v0);
                    tmemLoad32(lane_base + sl * BNS + 32, v1);
                    tmemLoadWait(v0);
                    tmemLoadWait(v1);
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[e] = fmaf(v0[e], s0, acc[e]);
                    tmemLoad32(lane_base + (sl + 1) * BNS, v0); // second slot's loads run behind the first slot's FMAs
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[32 + e] = fmaf(v1[e], s0, acc[32 + e]);
                    tmemLoad32(lane_base + (sl + 1) * BNS + 32, v1);
                    // While those are in flight, look at the next step's barrier.
                    rdy = mbarTest(&sh.tmemFull[kp ^ 1u], ((it + 1) >> 1) & 1);
                    tmemLoadWait(v0);
                    tmemLoadWait(v1);
                    // Both slots of this step are in registers: tell the step that reuses them.
                    tcFenceBefore();
                    __syncwarp();
                    if (lane == 0) mbarArriveCluster(full0 + s2 * 8u);
                    if (++s2 == kStages) s2 = 0;
                    // The scale prefetch goes behind the arrive (loads issued before it would hold it up).
                    if (nxt < k_steps) {
                        ring_a[i] = valid ? __ldg(sa_row + nxt) : 0.f;
                        ring_w0[i] = __ldg(sw0 + nxt);
                        ring_w1[i] = __ldg(sw1 + nxt);
                    }
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[64 + e] = fmaf(v0[e], s1, acc[64 + e]);
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[96 + e] = fmaf(v1[e], s1, acc[96 + e]);
                }
            }
            if (!ok) break;
            {
                // Coalesced stores: see storeRows64.  acc[h * 64 ..] are this row's 64 columns of half h.
                const int first_row = t.mt * (2 * BM) + static_cast<int>(cta) * BM + q * 32 + (lane & ~7);
                const long long first_grow = static_cast<long long>(sh.rowStart[t.g]) + first_row;
                const int rows_left = sh.rowCount[t.g] - first_row;
                __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.d) + first_grow * p.N + t.nt * BN + part * 64 + (lane & 7) * 8;
                storeRows64(reinterpret_cast<const float(&)[32]>(acc[0]), reinterpret_cast<const float(&)[32]>(acc[32]), out, p.N, rows_left, lane);
                storeRows64(reinterpret_cast<const float(&)[32]>(acc[64]), reinterpret_cast<const float(&)[32]>(acc[96]), out + BNS, p.N, rows_left, lane);
            }
        }
    }

    // Neither CTA may leave (or free TMEM) while its partner can still read its shared memory,
    // write its TMEM or arrive on its barriers.
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

cudaError_t nixl_gemm::launchPairKernel(const CUtensorMap &mapA, const CUtensorMap &mapW, const NixlGroupedGemmParams &p, cudaStream_t stream) {
    const size_t smem = size_t(kStages) * kStageBytes + sizeof(Shared) + 1024;
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
        cudaError_t e = cudaFuncSetAttribute(groupedGemmPairKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        // How many pairs can be resident at once: a persistent grid must not exceed it.
        cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1));
        int clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&clusters, groupedGemmPairKernel, &cfg);
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
    return cudaLaunchKernelEx(&cfg, groupedGemmPairKernel, mapA, mapW, p);
}

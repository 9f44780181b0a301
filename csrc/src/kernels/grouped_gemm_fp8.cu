// Grouped expert GEMM on 5th-generation tensor cores, optionally fed by EP dispatch arrivals.
//
//   D[rows of expert g, :] = dequant(A[rows, K]) x dequant(W[g, N, K])^T        (bf16 out)
//   A: e4m3, one fp32 scale per row per 128 channels (what EP dispatch delivers)
//   W: e4m3, one fp32 scale per 128 x 128 block
//
// sm_100a only.  One persistent CTA per SM, 384 threads, warp-specialised:
//   warp 0  TMA producer   cp.async.bulk.tensor (2-D, 128-byte swizzle) of a 128x128 A tile and a
//                          128x128 W tile per 128-channel step into a 5-stage shared-memory ring
//   warp 1  MMA issuer     4 x tcgen05.mma.kind::f8f6f4 (M128 N128 K32) per step into one of four
//                          TMEM accumulators (128 lanes x 128 fp32 columns each: all 512 columns).
//                          It polls one barrier per step, with a non-blocking test issued behind
//                          the previous step's MMAs (barrier instructions in front of the MMAs
//                          delay them by hundreds of cycles)
//   warp 2  TMEM allocator
//   warp 3  slot watcher   forwards "accumulator free again" into the step's full[] barrier, so
//                          that barrier alone tells the issuer that a step may go
//   warps 4-11 promotion + epilogue (two warps per TMEM lane quarter, 64 columns each):
//                          tcgen05.ld the step's partial sums, multiply by
//                          scaleA[row, step] * scaleW[g, n-block, step], accumulate in registers
//                          (the per-128-channel scales cannot be folded into the MMA), finally
//                          store bf16.  Four accumulators keep the MMA pipe fed across the
//                          commit -> wait -> load -> release round trip of each step.
// TMA loads read this GPU's own memory only and use no cluster multicast.  When `disp_flag` is
// given, the producer waits (bounded) for the per-(expert, source rank) arrival flags raised by
// ep_kernels.cu before it loads rows that those sources wrote: dispatch and GEMM overlap tile by
// tile instead of being separated by a receive phase.
//
// The reference has no GEMM (it moves tokens only); this kernel is the "dispatch fused into a
// tcgen05/TMEM grouped expert GEMM" variant of the EP path.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "kernels/nixl_kernels.h"
#include "kernels/grouped_gemm_internal.h"
#include "kernels/tcgen05_ptx.cuh"

namespace {

using namespace nixl_tc;

constexpr int BM = 128, BN = 128, BK = 128; // tile; BK is also the scale granularity
constexpr int kStages = 5;
constexpr int kThreads = 384;              // 4 role warps + 8 promotion warps
constexpr int kTileBytes = BM * BK;         // 16 KiB (fp8)
constexpr int kStageBytes = 2 * kTileBytes; // A + W
constexpr int kAccBufs = 4;                 // TMEM accumulators in flight (4 x 128 columns = all of TMEM)
constexpr int kTmemCols = kAccBufs * BN;

using nixl_gemm::GEMM_ERR_ARRIVAL;
using nixl_gemm::GEMM_ERR_TIMEOUT;
using nixl_gemm::kMaxGroups;

struct Shared {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmemFull[kAccBufs];
    uint64_t tmemEmpty[kAccBufs];
    uint32_t tmemBase;
    int abort;
    int tilePrefix[kMaxGroups + 1]; // tiles before group g
    int rowStart[kMaxGroups];
    int rowCount[kMaxGroups];
};

// Instruction descriptor: D fp32, A and B e4m3, both K-major, M = 128, N = 128.
__device__ __forceinline__ constexpr uint32_t instrDesc() {
    return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
        (static_cast<uint32_t>(BM >> 4) << 24);
}

// One 128-channel step of the issuer as a single instruction sequence: four MMAs, the two
// commits, then a non-blocking test of the next step's barrier.  Barrier instructions in front of
// the MMAs delay them by a few hundred cycles each, so the step's only poll sits behind them.
__device__ __forceinline__ void issueStep(uint32_t tmem_d, uint64_t da, uint64_t dw, uint32_t idesc, uint32_t bar_tmem_full, uint32_t bar_stage_empty,
                                          uint32_t peek_bar, uint32_t peek_par, uint32_t &ready_next) {
    asm volatile(
        "{\n"
        " .reg .pred pf, pacc, pnew;\n"
        " setp.ne.b32 pacc, %9, 0;\n"
        " setp.eq.b32 pnew, %9, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], %2, %3, %4, {%10, %10, %10, %10}, pnew;\n"
        " add.u64 %2, %2, 2;\n add.u64 %3, %3, 2;\n"
        " tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], %2, %3, %4, {%10, %10, %10, %10}, pacc;\n"
        " add.u64 %2, %2, 2;\n add.u64 %3, %3, 2;\n"
        " tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], %2, %3, %4, {%10, %10, %10, %10}, pacc;\n"
        " add.u64 %2, %2, 2;\n add.u64 %3, %3, 2;\n"
        " tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], %2, %3, %4, {%10, %10, %10, %10}, pacc;\n"
        " tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n"
        " tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n"
        " mbarrier.test_wait.parity.shared::cta.b64 pf, [%7], %8;\n"
        " selp.u32 %0, 1, 0, pf;\n"
        "}\n"
        : "=r"(ready_next), "+r"(tmem_d), "+l"(da), "+l"(dw)
        : "r"(idesc), "r"(bar_tmem_full), "r"(bar_stage_empty), "r"(peek_bar), "r"(peek_par), "r"(1u), "r"(0u)
        : "memory");
}

struct Tile {
    int g, mt, nt;
};

__device__ __forceinline__ bool tileAt(const Shared &sh, int groups, int n_tiles, int t, Tile &out) {
    if (t >= sh.tilePrefix[groups]) return false;
    int lo = 0, hi = groups; // tilePrefix[lo] <= t < tilePrefix[hi]
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
groupedGemmKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapW, const NixlGroupedGemmParams p) {
    extern __shared__ __align__(1024) unsigned char dyn[];
    unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~uintptr_t(1023));
    Shared &sh = *reinterpret_cast<Shared *>(tiles + kStages * kStageBytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.N / BN, k_steps = p.K / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbarInit(&sh.full[s], 2); // producer (with the byte count) + slot watcher
            mbarInit(&sh.empty[s], 1);
        }
        for (int b = 0; b < kAccBufs; ++b) {
            mbarInit(&sh.tmemFull[b], 1);
            mbarInit(&sh.tmemEmpty[b], 8); // one arrival per promotion warp
        }
        sh.abort = 0;
        // Tile table: group g owns ceil(count/BM) x n_tiles tiles.
        int run = 0;
        if (p.counts_flag) {
            // Overlapped with the dispatch: wait for everybody's counts, then derive the rows.
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
                run += ((c + BM - 1) / BM) * n_tiles;
            }
        } else {
            for (int g = 0; g < p.groups; ++g) {
                const int c = p.row_count[g];
                sh.tilePrefix[g] = run;
                sh.rowStart[g] = p.row_start[g];
                sh.rowCount[g] = c;
                run += ((c + BM - 1) / BM) * n_tiles;
            }
        }
        sh.tilePrefix[p.groups] = run;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemU32(&sh.tmemBase)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tcFenceBefore();
    __syncthreads();
    tcFenceAfter();
    const uint32_t tmem = sh.tmemBase;
    volatile int *abort_flag = &sh.abort;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        uint32_t it = 0; // k-steps issued so far (ring position)
        Tile t;
        for (int ti = blockIdx.x; tileAt(sh, p.groups, n_tiles, ti, t); ti += gridDim.x) {
            const int row0 = sh.rowStart[t.g] + t.mt * BM;
            if (p.disp_flag) {
                // Rows of an expert are ordered by source rank: wait for the sources whose rows
                // intersect this tile.
                const int lo = t.mt * BM, hi = min(lo + BM, sh.rowCount[t.g]);
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
                                    atomicOr(p.status, GEMM_ERR_ARRIVAL); // compute on what is there; the host sees the bit
                                    break;
                                }
                            }
                        }
                    }
                    first += c;
                }
                asm volatile("fence.proxy.async;" ::: "memory"); // peers' generic-proxy stores before our async-proxy reads
            }
            for (int ks = 0; ks < k_steps; ++ks, ++it) {
                const int s = it % kStages;
                if (!mbarWait(&sh.empty[s], ((it / kStages) & 1) ^ 1, abort_flag)) goto producer_done;
                mbarExpectTx(&sh.full[s], kStageBytes);
                tmaLoad2d(tiles + s * kStageBytes, &mapA, ks * BK, row0, &sh.full[s]);
                tmaLoad2d(tiles + s * kStageBytes + kTileBytes, &mapW, ks * BK, t.g * p.N + t.nt * BN, &sh.full[s]);
            }
        }
    producer_done:;
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------------- MMA issuer
        // One barrier per step: full[s] completes when the stage's bytes have landed (producer) and
        // the step's TMEM accumulator is free again (slot watcher), so this thread polls once per
        // four MMAs, and that poll is started behind the previous step's MMAs.
        int my_tiles = 0;
        {
            const int total = sh.tilePrefix[p.groups];
            if (static_cast<int>(blockIdx.x) < total) my_tiles = (total - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
        }
        const uint32_t steps_total = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(k_steps);
        uint32_t s = 0, full_par = 0, buf = 0, ready = 0;
        const uint32_t full_bar0 = smemU32(&sh.full[0]), empty_bar0 = smemU32(&sh.empty[0]), tfull_bar0 = smemU32(&sh.tmemFull[0]);
        const uint64_t desc0 = smemDesc(smemU32(tiles));
        for (uint32_t it = 0; it < steps_total; ++it) {
            if (!ready && !mbarWait(&sh.full[s], full_par, abort_flag)) goto mma_done;
            tcFenceAfter();
            uint32_t ns = s + 1, nfull_par = full_par;
            if (ns == kStages) {
                ns = 0;
                nfull_par ^= 1u;
            }
            // Advancing 32 bytes along K inside the swizzle atom = +2 in the 16-byte address field (done in issueStep).
            const uint64_t da = desc0 + static_cast<uint64_t>((s * kStageBytes) >> 4);
            const uint64_t dw = da + static_cast<uint64_t>(kTileBytes >> 4);
            issueStep(tmem + buf * BN, da, dw, instrDesc(), tfull_bar0 + buf * 8u, empty_bar0 + s * 8u, full_bar0 + ns * 8u, nfull_par, ready);
            buf = (buf + 1) & (kAccBufs - 1);
            s = ns;
            full_par = nfull_par;
        }
    mma_done:;
    } else if (warp == 3 && lane == 0) {
        // ---------------------------------------------------------------- slot watcher
        // Adds its arrival to a step's full[] barrier once the promotion warps have handed back the
        // TMEM accumulator that step will write.
        int my_tiles = 0;
        {
            const int total = sh.tilePrefix[p.groups];
            if (static_cast<int>(blockIdx.x) < total) my_tiles = (total - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
        }
        const uint32_t steps_total = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(k_steps);
        uint32_t s = 0, buf = 0, e_par = 1;
        for (uint32_t it = 0; it < steps_total; ++it) {
            if (!mbarWait(&sh.tmemEmpty[buf], e_par, abort_flag)) break;
            mbarArrive(&sh.full[s]);
            buf = (buf + 1) & (kAccBufs - 1);
            if (buf == 0) e_par ^= 1u;
            if (++s == kStages) s = 0;
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- promotion + epilogue
        const int q = warp & 3;            // TMEM lane quarter this warp may touch (fixed by warp id % 4)
        const int half = (warp - 4) >> 2;  // which 64 of the tile's 128 columns this warp promotes
        constexpr int HN = BN / 2;
        const int row_in_tile = q * 32 + lane;
        uint32_t it = 0;
        Tile t;
        const float *scale_a = p.scale_a;
        for (int ti = blockIdx.x; tileAt(sh, p.groups, n_tiles, ti, t); ti += gridDim.x) {
            const int local_row = t.mt * BM + row_in_tile;
            const bool valid = local_row < sh.rowCount[t.g];
            const long long grow = static_cast<long long>(sh.rowStart[t.g]) + local_row;
            const float *sa_row = scale_a + grow * k_steps;
            const float *sw = p.scale_w + (static_cast<long long>(t.g) * n_tiles + t.nt) * k_steps;
            float acc[HN];
#pragma unroll
            for (int i = 0; i < HN; ++i) acc[i] = 0.f;
            bool ok = true;
            // The scales of a step are needed by every FMA of that step, so their loads must not sit on
            // the critical path: a register ring keeps them kPrefetch steps ahead.  They are kept as
            // loaded; multiplying them right away would make the warp wait for the loads it just issued.
            constexpr int kPrefetch = 4;
            float ring_a[kPrefetch], ring_w[kPrefetch];
#pragma unroll
            for (int j = 0; j < kPrefetch; ++j) {
                ring_a[j] = (j < k_steps && valid) ? __ldg(sa_row + j) : 0.f;
                ring_w[j] = j < k_steps ? __ldg(sw + j) : 0.f;
            }
            for (int ks0 = 0; ks0 < k_steps && ok; ks0 += kPrefetch) {
#pragma unroll
                for (int j = 0; j < kPrefetch; ++j) {
                    const int ks = ks0 + j;
                    if (ks >= k_steps) break;
                    const int buf = it % kAccBufs;
                    const float s = ring_a[j] * ring_w[j];
                    const int nxt = ks + kPrefetch;
                    if (nxt < k_steps) {
                        ring_a[j] = valid ? __ldg(sa_row + nxt) : 0.f;
                        ring_w[j] = __ldg(sw + nxt);
                    }
                    if (!mbarWait(&sh.tmemFull[buf], (it / kAccBufs) & 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tcFenceAfter();
                    const uint32_t base = tmem + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + half * HN;
                    // Two register buffers: the second load is in flight while the first is scaled and added.
                    float v0[32], v1[32];
                    tmemLoad32(base, v0);
                    tmemLoad32(base + 32, v1);
                    tmemLoadWait(v0);
                    tmemLoadWait(v1);
                    // This warp's part of the accumulator has been read: hand it back before the FMAs.
                    tcFenceBefore();
                    __syncwarp();
                    if (lane == 0) mbarArrive(&sh.tmemEmpty[buf]);
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] = fmaf(v0[i], s, acc[i]);
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(v1[i], s, acc[32 + i]);
                    ++it;
                }
            }
            if (!ok) break;
            {
                // Coalesced stores (see storeRows64): this thread's 64 columns of its row.
                const int first_row = t.mt * BM + q * 32 + (lane & ~7);
                const long long first_grow = static_cast<long long>(sh.rowStart[t.g]) + first_row;
                const int rows_left = sh.rowCount[t.g] - first_row;
                __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.d) + first_grow * p.N + t.nt * BN + half * HN + (lane & 7) * 8;
                storeRows64(reinterpret_cast<const float(&)[32]>(acc[0]), reinterpret_cast<const float(&)[32]>(acc[32]), out, p.N, rows_left, lane);
            }
        }
    }

    tcFenceBefore();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort) atomicOr(p.status, GEMM_ERR_TIMEOUT);
    if (warp == 2) {
        tcFenceAfter();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
    }
}

// ------------------------------------------------------------------ host side

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encoder() {
    static EncodeFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

} // namespace

bool nixl_gemm::makeTileMap(CUtensorMap *map, const void *base, uint64_t rows, uint64_t k, uint32_t box_rows) {
    EncodeFn fn = encoder();
    if (!fn) return false;
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {k};
    const cuuint32_t box[2] = {BK, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

extern "C" int nixl_grouped_gemm_fp8_launch(const NixlGroupedGemmParams *params, void *stream) {
    if (!params || !params->a || !params->w || !params->d || !params->scale_a || !params->scale_w || !params->status)
        return cudaErrorInvalidValue;
    if (!params->counts_flag && (!params->row_start || !params->row_count)) return cudaErrorInvalidValue;
    const NixlGroupedGemmParams &p = *params;
    if (p.groups <= 0 || p.groups > kMaxGroups || p.N <= 0 || p.N % BN || p.K <= 0 || p.K % BK || p.a_rows <= 0)
        return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(p.a) | reinterpret_cast<uintptr_t>(p.w) | reinterpret_cast<uintptr_t>(p.d)) & 15) return cudaErrorInvalidValue;
    if ((p.disp_flag || p.counts_flag) && (!p.counts || p.ranks <= 0)) return cudaErrorInvalidValue;
    CUtensorMap mapA, mapW;
    if (!nixl_gemm::makeTileMap(&mapA, p.a, static_cast<uint64_t>(p.a_rows), static_cast<uint64_t>(p.K)) ||
        !nixl_gemm::makeTileMap(&mapW, p.w, static_cast<uint64_t>(p.groups) * p.N, static_cast<uint64_t>(p.K))) {
        std::fprintf(stderr, "nixl_grouped_gemm_fp8_launch: cuTensorMapEncodeTiled failed\n");
        return cudaErrorInvalidValue;
    }
    // Tile shape: CTA pairs with 256 x 256 tiles when rows per expert are plentiful (compact layout
    // of a throughput dispatch), single CTAs with 128 x 128 tiles for the expert-major low-latency
    // layout, where most tiles hold a handful of rows.
    int mode = p.tile_mode & 0xff;
    if (mode == 0) mode = (p.rows_per_expert == 0 && !p.counts_flag && p.N % 256 == 0 && p.a_rows >= 256LL * p.groups) ? 2 : 1;
    if (mode == 3) {
        if (p.N % 256 || p.K % 512 || p.counts_flag || p.disp_flag) return cudaErrorInvalidValue;
        if ((reinterpret_cast<uintptr_t>(p.scale_a) | reinterpret_cast<uintptr_t>(p.scale_w)) & 3) return cudaErrorInvalidValue;
        CUtensorMap mapW64;
        if (!nixl_gemm::makeTileMap(&mapW64, p.w, static_cast<uint64_t>(p.groups) * p.N, static_cast<uint64_t>(p.K), 64)) return cudaErrorInvalidValue;
        return nixl_gemm::launchMxPairKernel(mapA, mapW64, p, static_cast<cudaStream_t>(stream));
    }
    if (mode == 2) {
        if (p.N % 256) return cudaErrorInvalidValue;
        CUtensorMap mapW64; // the pair kernel loads W in 64-row boxes
        if (!nixl_gemm::makeTileMap(&mapW64, p.w, static_cast<uint64_t>(p.groups) * p.N, static_cast<uint64_t>(p.K), 64)) return cudaErrorInvalidValue;
        return nixl_gemm::launchPairKernel(mapA, mapW64, p, static_cast<cudaStream_t>(stream));
    }
    const size_t smem = size_t(kStages) * kStageBytes + sizeof(Shared) + 1024;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    {
        // The shared-memory limit is a per-device function attribute.
        static bool attr_done[64] = {};
        if (dev >= 0 && dev < 64 && !attr_done[dev]) {
            cudaError_t e = cudaFuncSetAttribute(groupedGemmKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (e != cudaSuccess) return e;
            attr_done[dev] = true;
        }
    }
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int grid = p.grid > 0 ? p.grid : sms;
    // Upper bound of tiles (row counts live on the device): never launch more CTAs than that.
    const long long max_tiles = (static_cast<long long>(p.a_rows + BM - 1) / BM + p.groups) * (p.N / BN);
    if (grid > max_tiles) grid = static_cast<int>(max_tiles);
    groupedGemmKernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(mapA, mapW, p);
    return cudaGetLastError();
}

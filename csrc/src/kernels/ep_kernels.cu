// MoE expert-parallel dispatch / combine for one NVLink domain (contract and algorithm:
// include/kernels/nixl_kernels.h).
//
// Both kernels are persistent, cooperatively launched grids (every CTA resident, so the
// in-kernel grid barrier cannot deadlock) of 256 threads.  Peer memory is reached through the
// remote memory view prepared by the agent: plain stores over NVLink, release-ordered flags,
// and bounded waits that mask a silent peer instead of hanging the GPU.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "device/nixl_device_layout.h"
#include "kernels/nixl_kernels.h"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxRanks = 64;
constexpr int kMaxTopk = 16;
constexpr int kGroup = 128; // channels per quantisation group

enum : int { ST_PEER_TIMEOUT = 1, ST_BARRIER_TIMEOUT = 2, ST_CAPACITY = 4 };

// ------------------------------------------------------------------ small device helpers

__device__ __forceinline__ uint64_t nowNs() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint64_t ldAcquireSys(const uint64_t *p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void stReleaseSys(uint64_t *p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned ldAcquireGpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ldVolatile(const int *p) { return *reinterpret_cast<const volatile int *>(p); }
__device__ __forceinline__ uint4 ldNc(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void stPeer16(void *p, const uint4 &v) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ char *peerBase(const void *view, int r) {
    const nixlMemViewEntry *e = reinterpret_cast<const nixlMemViewEntry *>(static_cast<const char *>(view) + sizeof(nixlMemViewHeader));
    return reinterpret_cast<char *>(e[r].ptr);
}

// Waits until *flag >= epoch.  False on timeout.
__device__ __forceinline__ bool waitFlag(const uint64_t *flag, uint64_t epoch, uint64_t timeout_ns) {
    uint64_t t0 = 0;
    unsigned spins = 0;
    while (ldAcquireSys(flag) < epoch) {
        if ((++spins & 31u) == 0) {
            const uint64_t now = nowNs();
            if (t0 == 0) t0 = now;
            else if (now - t0 > timeout_ns) return false;
        }
    }
    return true;
}

// Grid-wide barrier on two words {arrivals, generation}.  Bounded: on timeout sets the status
// bit and returns (the caller's results are then unreliable, which the host sees in `status`).
__device__ __forceinline__ void gridBarrier(unsigned *bar, int *status, uint64_t timeout_ns) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned gen = ldAcquireGpu(bar + 1);
        __threadfence();
        if (atomicAdd(bar, 1u) == gridDim.x - 1) {
            bar[0] = 0;
            __threadfence();
            atomicAdd(bar + 1, 1u);
        } else {
            uint64_t t0 = 0;
            unsigned spins = 0;
            while (ldAcquireGpu(bar + 1) == gen) {
                if ((++spins & 63u) == 0) {
                    const uint64_t now = nowNs();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > timeout_ns) {
                        atomicOr(status, ST_BARRIER_TIMEOUT);
                        break;
                    }
                }
            }
        }
    }
    __syncthreads();
}

// Barrier among the `nthreads` threads of one token group (named barrier `id`, 1..15).
__device__ __forceinline__ void groupBarrier(int id, int nthreads) {
    if (nthreads == 32) __syncwarp();
    else asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Threads cooperating on one token / row: as many as keeps the whole grid busy, a power of two
// between one warp and one CTA.
__device__ __forceinline__ int threadsPerItem(long long items) {
    const long long avail = static_cast<long long>(gridDim.x) * kThreads;
    int t = kThreads;
    while (t > 32 && static_cast<long long>(t) * items > avail) t >>= 1;
    return t;
}

// ------------------------------------------------------------------ dispatch

// Quantises one 128-channel group held by 16 lanes (8 bf16 each): returns 8 e4m3 bytes and,
// in lane%16 == 0, the group's scale.
__device__ __forceinline__ uint2 quantGroup(const uint4 &raw, bool round_scale, float &scale_out) {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    amax = fmaxf(amax, 1e-4f); // margin of the reference's cast (csrc/kernels/utils.cuh:430-456): never divide by ~0
    float scale = amax / 448.f, inv;
    if (round_scale) {
        const int ex = static_cast<int>(ceilf(log2f(scale)));
        scale = exp2f(static_cast<float>(ex));
        inv = exp2f(static_cast<float>(-ex));
    } else {
        inv = 448.f / amax;
    }
    scale_out = scale;
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        w[i] = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(f[2 * i] * inv, f[2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3));
    return make_uint2(w[0] | (w[1] << 16), w[2] | (w[3] << 16));
}

// Counts the rows of up to kPending tokens as sent.  Lane k < K of a token group holds, per token,
// the expert its k-th copy went to (-1: none).  The caller has passed a group barrier since the last
// of those stores was issued; the fence makes them visible system-wide before any count moves.
// Whoever completes an expert's rows raises that expert's arrival flag at its rank.
constexpr int kPending = 4;
__device__ __forceinline__ void countSent(const NixlEpDispatchParams &p, int El, const int (&pend)[kPending], int npend, int gtid) {
    if (gtid >= p.K) return;
    __threadfence_system();
#pragma unroll
    for (int i = 0; i < kPending; ++i) {
        if (i >= npend || pend[i] < 0) continue;
        const int e = pend[i];
        const int done = atomicAdd(p.scr.sent + e, 1) + 1;
        if (done == ldVolatile(p.scr.cnt + e)) {
            __threadfence_system(); // acquire side of the count: other groups' rows of this expert are out
            char *peer = peerBase(p.peers, e / El);
            stReleaseSys(reinterpret_cast<uint64_t *>(peer + p.lay.off_disp_flag) + static_cast<long long>(e % El) * p.R + p.rank, p.epoch);
        }
    }
}

__global__ void __launch_bounds__(kThreads, 2) epDispatchKernel(const __grid_constant__ NixlEpDispatchParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int El = p.E / p.R;
    const int groups = p.H / kGroup;
    const int row_bytes = p.use_fp8 ? p.H : p.H * 2;
    // shared: before[E] | ebase[E] | per token group: rows[kMaxTopk] | dests[kMaxTopk] | row bytes | scales
    int *before = reinterpret_cast<int *>(smem);
    int *ebase = before + p.E;
    unsigned char *group_area = reinterpret_cast<unsigned char *>(ebase + p.E);
    const int group_bytes = (2 * kMaxTopk * 4 + row_bytes + groups * 4 + 15) & ~15;

    char *self = peerBase(p.peers, p.rank);
    const int tid = threadIdx.x;
    __shared__ char *peer_sh[kMaxRanks]; // the data phase looks a peer up per row: keep the table on chip
    if (tid < p.R) peer_sh[tid] = peerBase(p.peers, tid);

    if (p.phases & 1) {
        // 1. histogram of destinations
        const long long n = static_cast<long long>(p.T) * p.K;
        for (long long i = static_cast<long long>(blockIdx.x) * kThreads + tid; i < n; i += static_cast<long long>(gridDim.x) * kThreads) {
            const long long e = p.topk_idx[i];
            if (e >= 0 && e < p.E && ldVolatile(p.scr.mask + static_cast<int>(e) / El) == 0) atomicAdd(p.scr.cnt + e, 1);
        }
        gridBarrier(p.scr.barrier, p.scr.status, p.timeout_ns);

        // 2. all-gather of counts: CTA b serves destination ranks b, b+grid, ...
        for (int d = blockIdx.x; d < p.R; d += gridDim.x) {
            if (ldVolatile(p.scr.mask + d) != 0) continue;
            char *peer = peerBase(p.peers, d);
            if (peer == nullptr) continue;
            int *dst = reinterpret_cast<int *>(peer + p.lay.off_counts) + static_cast<long long>(p.rank) * p.E;
            for (int e = tid; e < p.E; e += kThreads) dst[e] = ldVolatile(p.scr.cnt + e);
            if (tid == 0) reinterpret_cast<int *>(peer + p.lay.off_grp_tokens)[p.rank] = p.topk_weights != nullptr ? p.T : 0;
            // Experts of that rank that get nothing from us are complete right away.
            uint64_t *dflag = reinterpret_cast<uint64_t *>(peer + p.lay.off_disp_flag);
            __syncthreads();
            if (tid == 0) {
                __threadfence_system();
                stReleaseSys(reinterpret_cast<uint64_t *>(peer + p.lay.off_counts_flag) + p.rank, p.epoch);
            }
            for (int le = tid; le < El; le += kThreads)
                if (ldVolatile(p.scr.cnt + d * El + le) == 0) stReleaseSys(dflag + static_cast<long long>(le) * p.R + p.rank, p.epoch);
        }
    }

    // 3. wait for everybody's counts (every CTA looks for itself: 8 flags, no grid barrier needed)
    const uint64_t *cflag = reinterpret_cast<const uint64_t *>(self + p.lay.off_counts_flag);
    if (tid < p.R) {
        if (ldVolatile(p.scr.mask + tid) == 0 && peerBase(p.peers, tid) != nullptr) {
            if (!waitFlag(cflag + tid, p.epoch, p.timeout_ns)) {
                atomicExch(p.scr.mask + tid, 1);
                atomicOr(p.scr.status, ST_PEER_TIMEOUT);
            }
        } else if (peerBase(p.peers, tid) == nullptr) {
            atomicExch(p.scr.mask + tid, 1);
        }
    }
    __syncthreads();

    // 4. placement tables.  counts[r][e] is the local copy of the all-gather.
    const int *counts = reinterpret_cast<const int *>(self + p.lay.off_counts);
    for (int e = tid; e < p.E; e += kThreads) {
        int b = 0, total = 0;
        for (int r = 0; r < p.R; ++r) {
            if (ldVolatile(p.scr.mask + r) != 0) continue;
            const int c = ldVolatile(counts + static_cast<long long>(r) * p.E + e);
            if (r < p.rank) b += c;
            total += c;
        }
        before[e] = b;
        ebase[e] = total; // totals first, turned into per-rank prefixes below
    }
    __syncthreads();
    if (p.rows_per_expert > 0) {
        for (int e = tid; e < p.E; e += kThreads) {
            const int total = ebase[e];
            if (total > p.rows_per_expert) atomicOr(p.scr.status, ST_CAPACITY);
        }
        __syncthreads();
        for (int e = tid; e < p.E; e += kThreads) ebase[e] = (e % El) * p.rows_per_expert;
    } else if (tid < p.R) {
        // exclusive prefix over the local experts of destination rank `tid`
        int run = 0;
        for (int le = 0; le < El; ++le) {
            const int total = ebase[tid * El + le];
            ebase[tid * El + le] = run;
            run += total;
        }
        if (run > p.cap) atomicOr(p.scr.status, ST_CAPACITY);
    }
    __syncthreads();

    // Receiver-side bookkeeping is known as soon as the counts are: CTA 0 publishes it.
    if (blockIdx.x == 0 && (p.phases & 6)) {
        for (int le = tid; le < El; le += kThreads) {
            const int e = p.rank * El + le;
            int total = 0;
            for (int r = 0; r < p.R; ++r) {
                int c = 0;
                if (ldVolatile(p.scr.mask + r) == 0) c = ldVolatile(counts + static_cast<long long>(r) * p.E + e);
                p.layout_range[static_cast<long long>(le) * p.R + r] = (static_cast<long long>(total) << 32) | static_cast<unsigned>(c);
                total += c;
            }
            p.recv_count[le] = total;
            p.expert_offsets[le] = ebase[e];
            if (le == El - 1) p.expert_offsets[El] = ebase[e] + (p.rows_per_expert > 0 ? p.rows_per_expert : total);
        }
    }

    if (p.phases & 1) {
        // 5. data: a group of `nt` threads (one warp ... the whole CTA) owns a token: read once,
        //    quantise once into the group's shared buffer, store to up to K receivers.
        const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(p.x);
        const int vecs = p.H / 8; // 16-byte bf16 vectors per row
        const int nt = threadsPerItem(p.T);
        const int groups_per_cta = kThreads / nt;
        const int grp = tid / nt, gtid = tid - grp * nt;
        // Per copy of the token: the row it lands on at its receiver (-1: none) and the receiver.
        int *rows = reinterpret_cast<int *>(group_area + static_cast<size_t>(grp) * group_bytes);
        int *dests = rows + kMaxTopk;
        unsigned char *rowbuf = reinterpret_cast<unsigned char *>(dests + kMaxTopk);
        float *scalebuf = reinterpret_cast<float *>(rowbuf + row_bytes);
        const int bar_id = 1 + grp;
        int pend[kPending];
        int npend = 0; // uniform over the group
#pragma unroll
        for (int i = 0; i < kPending; ++i) pend[i] = -1;
        for (int t = blockIdx.x * groups_per_cta + grp; t < p.T; t += gridDim.x * groups_per_cta) {
            const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<long long>(t) * p.H);
            // Seven loads in flight per thread (a 7168-channel row is four such rounds for a warp).
            // `vecs` is a multiple of 32, so the guards are warp-uniform.
            constexpr int kLoads = 7;
            for (int v0 = gtid; v0 < vecs; v0 += kLoads * nt) {
                uint4 raw[kLoads];
#pragma unroll
                for (int j = 0; j < kLoads; ++j)
                    if (v0 + j * nt < vecs) raw[j] = ldNc(src + v0 + j * nt);
#pragma unroll
                for (int j = 0; j < kLoads; ++j) {
                    const int v = v0 + j * nt;
                    if (v >= vecs) continue;
                    if (p.use_fp8) {
                        float scale;
                        const uint2 q = quantGroup(raw[j], (p.round_scale | p.use_ue8m0) != 0, scale); // 16 lanes own one 128-channel group
                        reinterpret_cast<uint2 *>(rowbuf)[v] = q;
                        if ((v & 15) == 0) scalebuf[v >> 4] = scale;
                    } else {
                        reinterpret_cast<uint4 *>(rowbuf)[v] = raw[j];
                    }
                }
            }
            // Lane k reserves the slot of the token's k-th copy and leaves its row and receiver in
            // shared memory, so that the store loop below starts without a global load.
            int e_now = -1; // expert whose sent-count this lane owes (set even when the row exceeds the capacity)
            if (gtid < p.K) {
                const long long e = p.topk_idx[static_cast<long long>(t) * p.K + gtid];
                long long row = -1;
                if (e >= 0 && e < p.E && ldVolatile(p.scr.mask + static_cast<int>(e) / El) == 0) {
                    e_now = static_cast<int>(e);
                    row = static_cast<long long>(ebase[e]) + before[e] + atomicAdd(p.scr.fill + e, 1);
                    if (row >= p.cap) row = -1; // flagged as ST_CAPACITY above
                }
                rows[gtid] = static_cast<int>(row);
                dests[gtid] = e_now >= 0 ? e_now / El : 0;
                if (p.send_row != nullptr) p.send_row[static_cast<long long>(t) * p.K + gtid] = static_cast<int>(row);
            }
            groupBarrier(bar_id, nt);
            for (int k = 0; k < p.K; ++k) {
                const long long row = rows[k];
                if (row < 0) continue;
                const int d = dests[k];
                char *peer = peer_sh[d];
                uint4 *dx = reinterpret_cast<uint4 *>(peer + p.lay.off_recv_x + row * row_bytes);
                for (int v = gtid; v < row_bytes / 16; v += nt) stPeer16(dx + v, reinterpret_cast<const uint4 *>(rowbuf)[v]);
                if (p.use_fp8 && p.use_ue8m0) {
                    // A power-of-two scale is its exponent: one biased byte per group, four groups per word.
                    uint32_t *ds = reinterpret_cast<uint32_t *>(peer + p.lay.off_recv_scales + row * groups);
                    for (int g = gtid; g < groups / 4; g += nt) {
                        const float4 f = reinterpret_cast<const float4 *>(scalebuf)[g];
                        ds[g] = ((__float_as_uint(f.x) >> 23) & 0xffu) | (((__float_as_uint(f.y) >> 23) & 0xffu) << 8) |
                            (((__float_as_uint(f.z) >> 23) & 0xffu) << 16) | (((__float_as_uint(f.w) >> 23) & 0xffu) << 24);
                    }
                } else if (p.use_fp8) {
                    float4 *ds = reinterpret_cast<float4 *>(reinterpret_cast<float *>(peer + p.lay.off_recv_scales) + row * groups);
                    for (int g = gtid; g < groups / 4; g += nt) ds[g] = reinterpret_cast<const float4 *>(scalebuf)[g];
                }
                if (gtid == 0) {
                    uint2 info = make_uint2(static_cast<unsigned>(p.rank), static_cast<unsigned>(t * p.K + k));
                    *reinterpret_cast<uint2 *>(peer + p.lay.off_recv_info + row * 8) = info;
                }
            }
            // Group record of this token for every rank that got copies of it (lane d serves rank d): the rows
            // and their weights, tagged with the step number so that what an earlier step left in the slot
            // is never taken for new.  Ranks without a copy get nothing; their slot keeps an old tag.
            if (p.topk_weights != nullptr && gtid < p.R) {
                const int d = gtid;
                alignas(16) NixlEpGroupRecord rec;
                rec.n = 0;
                for (int k = 0; k < p.K && k < 8; ++k)
                    if (rows[k] >= 0 && dests[k] == d) {
                        rec.rows[rec.n] = rows[k];
                        rec.w[rec.n] = p.topk_weights[static_cast<long long>(t) * p.K + k];
                        ++rec.n;
                    }
                if (rec.n > 0) {
                    for (int i = rec.n; i < 8; ++i) {
                        rec.rows[i] = 0;
                        rec.w[i] = 0.f;
                    }
                    rec.pad[0] = static_cast<int>(p.epoch & 0x7fffffffull);
                    rec.pad[1] = rec.pad[2] = 0;
                    uint4 *dst = reinterpret_cast<uint4 *>(peer_sh[d] + p.lay.off_grp) + (static_cast<long long>(p.rank) * p.max_tokens + t) * 5;
                    const uint4 *src = reinterpret_cast<const uint4 *>(&rec);
#pragma unroll
                    for (int i = 0; i < 5; ++i) stPeer16(dst + i, src[i]);
                }
            }
            groupBarrier(bar_id, nt); // all stores of this token issued (and the buffer is free for the next one)
            // The rows still have to be counted as sent, behind a system-wide fence.  That fence waits
            // for every store in flight to be acknowledged by the peer, so it is paid once per
            // kPending tokens, not per token: lane k keeps the experts of its tokens until then.
#pragma unroll
            for (int i = 0; i < kPending; ++i)
                if (i == npend) pend[i] = e_now;
            if (++npend == kPending) {
                countSent(p, El, pend, npend, gtid);
                npend = 0;
            }
            groupBarrier(bar_id, nt);
        }
        if (npend > 0) countSent(p, El, pend, npend, gtid);
    }

    if (p.phases & 2) {
        // 6. arrivals: El x R flags, spread over the grid's threads
        const uint64_t *dflag = reinterpret_cast<const uint64_t *>(self + p.lay.off_disp_flag);
        const int nflags = El * p.R;
        for (int i = blockIdx.x * kThreads + tid; i < nflags; i += gridDim.x * kThreads) {
            const int r = i % p.R;
            if (ldVolatile(p.scr.mask + r) != 0) continue;
            if (!waitFlag(dflag + i, p.epoch, p.timeout_ns)) {
                atomicExch(p.scr.mask + r, 1);
                atomicOr(p.scr.status, ST_PEER_TIMEOUT);
            }
        }
    }

    // 7. leave the scratch counters at zero for the next call
    if (p.phases & 1) {
        gridBarrier(p.scr.barrier, p.scr.status, p.timeout_ns);
        if (blockIdx.x == 0)
            for (int e = tid; e < p.E; e += kThreads) {
                p.scr.cnt[e] = 0;
                p.scr.fill[e] = 0;
                p.scr.sent[e] = 0;
            }
    }
}

// ------------------------------------------------------------------ combine

// Logarithmic 10-bit row format for combine (role of the reference's LogFMT-10 codec,
// examples/device/ep/csrc/kernels/nixl_ep_ll.cu:459-616).  The 15-bit magnitude pattern of a bf16
// (exponent and mantissa read as one integer) is a piecewise-linear logarithm of the value, so
// the codec works on patterns with integer and fp32 arithmetic only: per 128-channel group the
// patterns between the smallest non-zero one (at most 32 octaves = 4096 patterns below the
// largest) and the largest are mapped onto 510 steps; code 0 is exact zero and one further bit
// holds the sign.  A group that spans at most 510 patterns (four octaves) is coded exactly;
// otherwise the value is rounded to the nearest grid pattern, a relative error of at most
// (range / 510 + 1) * 2^-8.  Non-finite inputs are clamped to the largest finite bf16.
//
// Layout of a row of H channels (H % 512 == 0) in its H * 2-byte landing slot: H / 512 blocks of
// 160 words; in a block, lane l (16 channels l*16 .. l*16+15 of the block) owns words j*32 + l,
// j < 5, so that a warp's five stores are each one contiguous 128 bytes; words 0..3 and the low
// half of word 4 hold the sixteen 9-bit codes as one little-endian bit stream, the high half of
// word 4 the sixteen sign bits.  After the blocks, at byte H * 10 / 8, one (smallest pattern as
// int32, patterns per step as float) pair per group.
constexpr unsigned kLogFmtSteps = 510;
constexpr int kLogFmtMaxPatterns = 32 * 128;

__device__ __forceinline__ void stPeer4(void *p, uint32_t v) {
    asm volatile("st.global.L1::no_allocate.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void stPeer8(void *p, const uint2 &v) {
    asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// Encodes the 16 bf16 values a lane holds; the eight lanes of a 128-channel group cooperate on
// the range.  `meta` is the group's (smallest pattern, patterns per step), identical in the eight lanes.
__device__ __forceinline__ void logfmtEncode16(const uint4 &lo, const uint4 &hi, uint32_t (&w)[5], uint2 &meta) {
    const uint32_t raw[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    uint32_t pat[16];
    uint32_t signs = 0, pmax = 0, pmin_m1 = 0xffffffffu; // zero patterns wrap to the top and drop out of the minimum
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        signs |= ((raw[i] >> 15) & 1u) << (2 * i);
        signs |= (raw[i] >> 31) << (2 * i + 1);
        pat[2 * i] = min(raw[i] & 0x7fffu, 0x7f7fu);
        pat[2 * i + 1] = min((raw[i] >> 16) & 0x7fffu, 0x7f7fu);
        pmax = max(pmax, max(pat[2 * i], pat[2 * i + 1]));
        pmin_m1 = min(pmin_m1, min(pat[2 * i] - 1u, pat[2 * i + 1] - 1u));
    }
#pragma unroll
    for (int off = 4; off >= 1; off >>= 1) {
        pmax = max(pmax, __shfl_xor_sync(0xffffffffu, pmax, off));
        pmin_m1 = min(pmin_m1, __shfl_xor_sync(0xffffffffu, pmin_m1, off));
    }
    int pmin = pmax ? static_cast<int>(pmin_m1 + 1u) : 0;
    pmin = max(pmin, static_cast<int>(pmax) - kLogFmtMaxPatterns);
    const unsigned range = pmax - static_cast<unsigned>(pmin);
    const bool wide = range > kLogFmtSteps;
    const float scale = wide ? static_cast<float>(kLogFmtSteps) / static_cast<float>(range) : 1.f;
    meta = make_uint2(static_cast<uint32_t>(pmin), __float_as_uint(wide ? static_cast<float>(range) / static_cast<float>(kLogFmtSteps) : 1.f));
    uint64_t acc = 0;
    int bits = 0, wi = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int above = max(static_cast<int>(pat[i]) - pmin, 0);
        const uint32_t code = pat[i] ? 1u + min(__float2uint_rn(static_cast<float>(above) * scale), kLogFmtSteps) : 0u;
        acc |= static_cast<uint64_t>(code) << bits;
        bits += 9;
        if (bits >= 32) {
            w[wi++] = static_cast<uint32_t>(acc);
            acc >>= 32;
            bits -= 32;
        }
    }
    w[4] = static_cast<uint32_t>(acc) | (signs << 16);
}

// acc[i] += weight * value_i for the 16 values of one lane's words.
__device__ __forceinline__ void logfmtDecodeAdd16(const uint32_t (&w)[5], const uint2 &meta, float weight, float (&acc)[16]) {
    const float per_step = __uint_as_float(meta.y);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int bit = 9 * i, idx = bit >> 5, sh = bit & 31;
        const uint32_t next = idx < 4 ? w[idx + 1] : 0u;
        const uint32_t code = __funnelshift_r(w[idx], next, sh) & 0x1ffu;
        const uint32_t pat = meta.x + __float2uint_rn(static_cast<float>(code - 1u) * per_step);
        const uint32_t sign = (w[4] >> (16 + i)) << 31;
        const float v = __uint_as_float(code ? ((pat << 16) | sign) : 0u);
        acc[i] = fmaf(weight, v, acc[i]);
    }
}

// The reduction of pull-mode combine for the tokens of this thread group.  KMAX bounds top-k at
// compile time so that the K rows' 16-byte vectors live in registers.  With kDouble the loads of
// the next vector position are issued before the current one is reduced: a load from a peer takes
// microseconds, and without the overlap every position would pay that latency in full.
template <int KMAX, bool kDouble>
__device__ __forceinline__ void pullReduce(const NixlEpCombineParams &p, int El, int vecs, int nt, int groups_per_cta, int grp, int gtid) {
    __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.out);
    for (int t = blockIdx.x * groups_per_cta + grp; t < p.T; t += gridDim.x * groups_per_cta) {
        float w[KMAX];
        const uint4 *src[KMAX];
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
            w[k] = __int_as_float(0x7fc00000); // NaN marks "skip" (a real weight may be 0)
            src[k] = nullptr;
            if (k < p.K) {
                const long long e = p.topk_idx[static_cast<long long>(t) * p.K + k];
                const int row = p.send_row[static_cast<long long>(t) * p.K + k];
                if (e >= 0 && e < p.E && row >= 0) {
                    const int r = static_cast<int>(e) / El;
                    char *peer = peerBase(p.peers, r);
                    if (peer != nullptr && ldVolatile(p.scr.mask + r) == 0) {
                        w[k] = p.topk_weights[static_cast<long long>(t) * p.K + k];
                        src[k] = reinterpret_cast<const uint4 *>(peer + p.lay.off_comb_in + static_cast<long long>(row) * p.H * 2);
                    }
                }
            }
        }
        auto load = [&](uint4(&buf)[KMAX], int v) {
#pragma unroll
            for (int k = 0; k < KMAX; ++k)
                if (k < p.K && w[k] == w[k]) buf[k] = ldNc(src[k] + v);
        };
        auto reduceStore = [&](const uint4(&buf)[KMAX], int v) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < KMAX; ++k) {
                if (k >= p.K || w[k] != w[k]) continue;
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&buf[k]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(h[i]);
                    acc[2 * i] = fmaf(w[k], f.x, acc[2 * i]);
                    acc[2 * i + 1] = fmaf(w[k], f.y, acc[2 * i + 1]);
                }
            }
            uint4 o;
            __nv_bfloat162 *oh = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            *reinterpret_cast<uint4 *>(out + static_cast<long long>(t) * p.H + v * 8) = o;
        };
        if constexpr (kDouble) {
            uint4 a[KMAX], b[KMAX];
            int v = gtid;
            if (v < vecs) load(a, v);
            while (v < vecs) {
                const int v1 = v + nt;
                if (v1 < vecs) load(b, v1);
                reduceStore(a, v);
                if (v1 >= vecs) break;
                const int v2 = v1 + nt;
                if (v2 < vecs) load(a, v2);
                reduceStore(b, v1);
                v = v2;
            }
        } else {
            for (int v = gtid; v < vecs; v += nt) {
                uint4 raw[KMAX];
                load(raw, v);
                reduceStore(raw, v);
            }
        }
    }
}

// Pull-mode combine: announce that this rank's expert outputs are complete, wait for the same
// word from every peer, then each token's home rank loads the K rows from where dispatch put
// them and reduces in fp32.  Every row crosses NVLink once and is never staged.
__device__ __forceinline__ void epCombinePull(const NixlEpCombineParams &p) {
    const int El = p.E / p.R;
    const int tid = threadIdx.x;
    char *self = peerBase(p.peers, p.rank);
    const int vecs = p.H / 8;
    if ((p.phases & 1) && blockIdx.x == 0 && tid < p.R) {
        char *peer = peerBase(p.peers, tid);
        if (peer != nullptr && ldVolatile(p.scr.mask + tid) == 0) {
            __threadfence_system();
            stReleaseSys(reinterpret_cast<uint64_t *>(peer + p.lay.off_comb_flag) + p.rank, p.epoch);
        }
    }
    if (!(p.phases & 2)) return;
    const uint64_t *flag = reinterpret_cast<const uint64_t *>(self + p.lay.off_comb_flag);
    if (tid < p.R && ldVolatile(p.scr.mask + tid) == 0 && peerBase(p.peers, tid) != nullptr) {
        if (!waitFlag(flag + tid, p.epoch, p.timeout_ns)) {
            atomicExch(p.scr.mask + tid, 1);
            atomicOr(p.scr.status, ST_PEER_TIMEOUT);
        }
    }
    __syncthreads();
    const int nt = threadsPerItem(p.T);
    const int groups_per_cta = kThreads / nt;
    const int grp = tid / nt, gtid = tid - grp * nt;
    if (p.K <= 8) pullReduce<8, true>(p, El, vecs, nt, groups_per_cta, grp, gtid);
    else pullReduce<kMaxTopk, false>(p, El, vecs, nt, groups_per_cta, grp, gtid);
}

// Staging area of one warp of the rank-reduced combine: kRrSlots 16-byte slots per lane, filled by asynchronous
// copies.  Loads that wait in shared memory instead of registers let a warp keep 12 KB in flight, and two CTAs fit
// on an SM.
constexpr int kRrSlots = 24;
constexpr int kRrWarpBytes = kRrSlots * 32 * 16;
constexpr int kRrCtaBytes = (kThreads / 32) * kRrWarpBytes;

__device__ __forceinline__ void cpAsync16(uint32_t smem_addr, const void *g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(g) : "memory"); // through L2: sees what peers wrote
}
__device__ __forceinline__ void cpAsyncWaitAll() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// One warp: dst[v] = sum over the n rows (1..8) of w[k] * src[k][v] for the row's `vecs` 16-byte vectors, fp32
// accumulation, bf16 out.  kRrSlots / n vector positions of every row are in flight per lane.  Each lane reads back
// only the slots it filled itself, so its own wait is all the synchronisation the area needs.  dst may be a peer's memory.
__device__ __forceinline__ void warpWeightedRows(int n, const uint4 *const (&src)[8], const float (&w)[8], uint4 *dst, int vecs, int lane,
                                                 uint4 *stage) {
    const int per_pass = kRrSlots / n;
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(stage)) + lane * 16;
    for (int v0 = lane; v0 < vecs; v0 += 32 * per_pass) {
#pragma unroll 1
        for (int u = 0; u < per_pass; ++u) {
            const int v = v0 + u * 32;
            if (v >= vecs) break;
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < n) cpAsync16(sbase + static_cast<uint32_t>((u * n + k) * 32 * 16), src[k] + v);
        }
        cpAsyncWaitAll();
#pragma unroll 1
        for (int u = 0; u < per_pass; ++u) {
            const int v = v0 + u * 32;
            if (v >= vecs) break;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (k >= n) continue;
                const uint4 raw = stage[(u * n + k) * 32 + lane];
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h[j]);
                    acc[2 * j] = fmaf(w[k], f.x, acc[2 * j]);
                    acc[2 * j + 1] = fmaf(w[k], f.y, acc[2 * j + 1]);
                }
            }
            uint4 o;
            __nv_bfloat162 *oh = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
            stPeer16(dst + v, o);
        }
    }
}

// Rank-reduced combine (NixlEpCombineParams::max_tokens).  Phase 1, expert rank: one warp per (token, home
// rank) group record adds the token's rows up in fp32, weighted, and stores ONE bf16 row at the home rank.
// Phase 2, home rank: add the rows of the ranks the token went to.
template <int kPhases>
__device__ __forceinline__ void epCombineRankReduce(const NixlEpCombineParams &p) {
    const int El = p.E / p.R;
    const int tid = threadIdx.x, lane = tid & 31;
    char *self = peerBase(p.peers, p.rank);
    const int vecs = p.H / 8;
    const long long M = p.max_tokens;
    const int tag = static_cast<int>(p.epoch & 0x7fffffffull);
    extern __shared__ __align__(16) unsigned char rr_stage[];
    uint4 *stage = reinterpret_cast<uint4 *>(rr_stage + (tid >> 5) * kRrWarpBytes);

    if constexpr ((kPhases & 1) != 0) {
        const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(p.x);
        const int *tokens_of = reinterpret_cast<const int *>(self + p.lay.off_grp_tokens);
        const uint4 *records = reinterpret_cast<const uint4 *>(self + p.lay.off_grp);
        int max_t = 0;
        for (int r = 0; r < p.R; ++r) {
            const int n = ldVolatile(tokens_of + r);
            max_t = n > max_t ? (n < M ? n : static_cast<int>(M)) : max_t;
        }
        const long long items = static_cast<long long>(max_t) * p.R;
        const long long warps = static_cast<long long>(gridDim.x) * (kThreads / 32);
        // item = token * R + home rank: neighbouring warps store to different peers
        for (long long i = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (tid >> 5); i < items; i += warps) {
            const int r = static_cast<int>(i % p.R);
            const long long t = i / p.R;
            if (t >= ldVolatile(tokens_of + r) || ldVolatile(p.scr.mask + r) != 0) continue;
            char *peer = peerBase(p.peers, r);
            if (peer == nullptr) continue;
            const uint4 *rec = records + (static_cast<long long>(r) * M + t) * 5;
            const uint4 head = rec[0];
            const int n = static_cast<int>(head.x);
            if (static_cast<int>(head.y) != tag || n <= 0 || n > 8) continue;
            const uint4 r0 = rec[1], r1 = rec[2], w0 = rec[3], w1 = rec[4];
            const int rows[8] = {int(r0.x), int(r0.y), int(r0.z), int(r0.w), int(r1.x), int(r1.y), int(r1.z), int(r1.w)};
            const float w[8] = {__uint_as_float(w0.x), __uint_as_float(w0.y), __uint_as_float(w0.z), __uint_as_float(w0.w),
                                __uint_as_float(w1.x), __uint_as_float(w1.y), __uint_as_float(w1.z), __uint_as_float(w1.w)};
            const uint4 *src[8];
            float wk[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                src[k] = reinterpret_cast<const uint4 *>(x + static_cast<long long>(k < n ? rows[k] : rows[0]) * p.H);
                wk[k] = k < n ? w[k] : 0.f; // padding rows repeat the first one with weight zero
            }
            uint4 *dst = reinterpret_cast<uint4 *>(peer + p.lay.off_comb_x + (static_cast<long long>(p.rank) * M + t) * p.H * 2);
            warpWeightedRows(n, src, wk, dst, vecs, lane, stage);
        }
        __syncthreads();
        if (tid == 0) __threadfence_system();
        gridBarrier(p.scr.barrier, p.scr.status, p.timeout_ns);
        // Everybody's rows are out: tell each home rank.
        for (int d = blockIdx.x; d < p.R; d += gridDim.x) {
            if (ldVolatile(p.scr.mask + d) != 0) continue;
            char *peer = peerBase(p.peers, d);
            if (peer != nullptr && tid == 0) {
                __threadfence_system();
                stReleaseSys(reinterpret_cast<uint64_t *>(peer + p.lay.off_comb_flag) + p.rank, p.epoch);
            }
        }
    }

    if constexpr ((kPhases & 2) != 0) {
        const uint64_t *flag = reinterpret_cast<const uint64_t *>(self + p.lay.off_comb_flag);
        if (tid < p.R && ldVolatile(p.scr.mask + tid) == 0 && peerBase(p.peers, tid) != nullptr) {
            if (!waitFlag(flag + tid, p.epoch, p.timeout_ns)) {
                atomicExch(p.scr.mask + tid, 1);
                atomicOr(p.scr.status, ST_PEER_TIMEOUT);
            }
        }
        __syncthreads();
        const __nv_bfloat16 *landing = reinterpret_cast<const __nv_bfloat16 *>(self + p.lay.off_comb_x);
        __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.out);
        const int warps = gridDim.x * (kThreads / 32);
        for (int t = blockIdx.x * (kThreads / 32) + (tid >> 5); t < p.T; t += warps) { // one warp per token
            // ranks that hold copies of this token (and answered)
            unsigned ranks = 0;
            for (int k = 0; k < p.K; ++k) {
                const long long e = p.topk_idx[static_cast<long long>(t) * p.K + k];
                if (e >= 0 && e < p.E && ldVolatile(p.scr.mask + static_cast<int>(e) / El) == 0) ranks |= 1u << (static_cast<int>(e) / El);
            }
            uint4 *dst = reinterpret_cast<uint4 *>(out + static_cast<long long>(t) * p.H);
            if (ranks == 0) {
                for (int v = lane; v < vecs; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
                continue;
            }
            if (__popc(ranks) <= 8) {
                const uint4 *src[8];
                float one[8];
                unsigned left = ranks;
                const int first = __ffs(ranks) - 1;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int d = left ? __ffs(left) - 1 : first;
                    one[j] = left ? 1.f : 0.f;
                    left &= left - 1; // (0 stays 0)
                    src[j] = reinterpret_cast<const uint4 *>(landing + (static_cast<long long>(d) * M + t) * p.H);
                }
                warpWeightedRows(__popc(ranks), src, one, dst, vecs, lane, stage);
                continue;
            }
            for (int v = lane; v < vecs; v += 32) { // more than eight ranks hold copies: plain loads, eight rows at a time
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                unsigned left = ranks;
                while (left) {
                    const int d = __ffs(left) - 1;
                    left &= left - 1;
                    const uint4 raw = *reinterpret_cast<const uint4 *>(landing + (static_cast<long long>(d) * M + t) * p.H + v * 8);
                    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(h[i]);
                        acc[2 * i] += f.x;
                        acc[2 * i + 1] += f.y;
                    }
                }
                uint4 o;
                __nv_bfloat162 *oh = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                dst[v] = o;
            }
        }
    }
}

// The rank-reduced mode as two kernels of its own: each phase alone needs few enough registers for two CTAs per SM,
// which is what keeps enough loads in flight; the second launch starts when every CTA of the first has left.
__global__ void __launch_bounds__(kThreads, 2) epCombineRankReduceSend(const __grid_constant__ NixlEpCombineParams p) { epCombineRankReduce<1>(p); }
__global__ void __launch_bounds__(kThreads, 2) epCombineRankReduceRecv(const __grid_constant__ NixlEpCombineParams p) { epCombineRankReduce<2>(p); }

__global__ void __launch_bounds__(kThreads) epCombineKernel(const __grid_constant__ NixlEpCombineParams p) {
    __shared__ int offs[kMaxRanks * 8 + 1]; // expert_offsets copy (El + 1 <= 513)
    __shared__ int cnts[kMaxRanks * 8];
    const int El = p.E / p.R;
    const int tid = threadIdx.x;
    char *self = peerBase(p.peers, p.rank);
    const int vecs = p.H / 8;

    if (p.pull) {
        epCombinePull(p);
        return;
    }

    if (p.phases & 1) {
        for (int i = tid; i <= El; i += kThreads) offs[i] = p.expert_offsets[i];
        for (int i = tid; i < El; i += kThreads) cnts[i] = p.recv_count[i];
        __syncthreads();
        // Rows are enumerated expert by expert; every warp of the grid takes every n-th valid row.
        const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(p.x);
        const int lane = tid & 31;
        const long long warps = static_cast<long long>(gridDim.x) * (kThreads / 32);
        int le = 0, seen = 0; // rows of experts < le
        for (long long j = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (tid >> 5);; j += warps) {
            while (le < El && j >= seen + cnts[le]) seen += cnts[le++];
            if (le >= El) break;
            const long long row = static_cast<long long>(offs[le]) + (j - seen);
            const uint2 info = *reinterpret_cast<const uint2 *>(p.recv_info + row * 2);
            const int r = static_cast<int>(info.x);
            if (r < 0 || r >= p.R || ldVolatile(p.scr.mask + r) != 0) continue;
            char *peer = peerBase(p.peers, r);
            if (peer == nullptr) continue;
            const uint4 *src = reinterpret_cast<const uint4 *>(x + row * p.H);
            uint4 *dst = reinterpret_cast<uint4 *>(peer + p.lay.off_comb_x + static_cast<long long>(info.y) * p.H * 2);
            if (p.use_logfmt) {
                uint32_t *words = reinterpret_cast<uint32_t *>(dst);
                uint2 *meta = reinterpret_cast<uint2 *>(reinterpret_cast<char *>(dst) + static_cast<long long>(p.H) * 10 / 8);
                const int blocks = p.H / 512;
                uint4 lo = ldNc(src + lane * 2), hi = ldNc(src + lane * 2 + 1);
                for (int b = 0; b < blocks; ++b) {
                    uint4 nlo = lo, nhi = hi;
                    if (b + 1 < blocks) { // next block's loads fly while this one is encoded
                        nlo = ldNc(src + (b + 1) * 64 + lane * 2);
                        nhi = ldNc(src + (b + 1) * 64 + lane * 2 + 1);
                    }
                    uint32_t w[5];
                    uint2 m;
                    logfmtEncode16(lo, hi, w, m);
#pragma unroll
                    for (int j = 0; j < 5; ++j) stPeer4(words + b * 160 + j * 32 + lane, w[j]);
                    if ((lane & 7) == 0) stPeer8(meta + b * 4 + (lane >> 3), m);
                    lo = nlo;
                    hi = nhi;
                }
                continue;
            }
            for (int v0 = lane; v0 < vecs; v0 += 8 * 32) { // eight loads in flight per lane
                uint4 val[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (v0 + i * 32 < vecs) val[i] = ldNc(src + v0 + i * 32);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (v0 + i * 32 < vecs) stPeer16(dst + v0 + i * 32, val[i]);
            }
        }
        __syncthreads();
        if (tid == 0) __threadfence_system();
        gridBarrier(p.scr.barrier, p.scr.status, p.timeout_ns);
        // Everybody's rows are out: tell each source rank.
        for (int d = blockIdx.x; d < p.R; d += gridDim.x) {
            if (ldVolatile(p.scr.mask + d) != 0) continue;
            char *peer = peerBase(p.peers, d);
            if (peer != nullptr && tid == 0) {
                __threadfence_system();
                stReleaseSys(reinterpret_cast<uint64_t *>(peer + p.lay.off_comb_flag) + p.rank, p.epoch);
            }
        }
    }

    if (p.phases & 2) {
        const uint64_t *flag = reinterpret_cast<const uint64_t *>(self + p.lay.off_comb_flag);
        if (tid < p.R && ldVolatile(p.scr.mask + tid) == 0 && peerBase(p.peers, tid) != nullptr) {
            if (!waitFlag(flag + tid, p.epoch, p.timeout_ns)) {
                atomicExch(p.scr.mask + tid, 1);
                atomicOr(p.scr.status, ST_PEER_TIMEOUT);
            }
        }
        __syncthreads();
        // out[t] = sum_k w[t,k] * y[t,k] in fp32
        const __nv_bfloat16 *landing = reinterpret_cast<const __nv_bfloat16 *>(self + p.lay.off_comb_x);
        __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.out);
        const int nt = threadsPerItem(p.T);
        const int groups_per_cta = kThreads / nt;
        const int grp = tid / nt, gtid = tid - grp * nt;
        for (int t = blockIdx.x * groups_per_cta + grp; t < p.T; t += gridDim.x * groups_per_cta) {
            float w[kMaxTopk];
#pragma unroll
            for (int k = 0; k < kMaxTopk; ++k) {
                w[k] = 0.f;
                if (k < p.K) {
                    const long long e = p.topk_idx[static_cast<long long>(t) * p.K + k];
                    if (e >= 0 && e < p.E && ldVolatile(p.scr.mask + static_cast<int>(e) / El) == 0)
                        w[k] = p.topk_weights[static_cast<long long>(t) * p.K + k];
                    else w[k] = __int_as_float(0x7fc00000); // NaN marks "skip" (a real weight may be 0)
                }
            }
            if (p.use_logfmt) {
                const long long meta_off = static_cast<long long>(p.H) * 10 / 8;
                for (int u = gtid; u < p.H / 16; u += nt) {
                    const int b = u >> 5, l = u & 31;
                    float acc[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll
                    for (int k0 = 0; k0 < kMaxTopk; k0 += 4) { // four rows' words in flight
                        if (k0 >= p.K) break;
                        uint32_t cw[4][5];
                        uint2 m[4];
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const int k = k0 + kk;
                            if (k < p.K && w[k] == w[k]) {
                                const char *slot = reinterpret_cast<const char *>(landing + (static_cast<long long>(t) * p.K + k) * p.H);
                                const uint32_t *words = reinterpret_cast<const uint32_t *>(slot) + b * 160 + l;
#pragma unroll
                                for (int j = 0; j < 5; ++j) cw[kk][j] = words[j * 32];
                                m[kk] = *reinterpret_cast<const uint2 *>(slot + meta_off + (b * 4 + (l >> 3)) * 8);
                            }
                        }
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const int k = k0 + kk;
                            if (k < p.K && w[k] == w[k]) logfmtDecodeAdd16(cw[kk], m[kk], w[k], acc);
                        }
                    }
                    uint4 o[2];
                    __nv_bfloat162 *oh = reinterpret_cast<__nv_bfloat162 *>(o);
#pragma unroll
                    for (int i = 0; i < 8; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                    uint4 *dst = reinterpret_cast<uint4 *>(out + static_cast<long long>(t) * p.H + b * 512 + l * 16);
                    dst[0] = o[0];
                    dst[1] = o[1];
                }
                continue;
            }
            for (int v = gtid; v < vecs; v += nt) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                uint4 raw[kMaxTopk];
#pragma unroll
                for (int k = 0; k < kMaxTopk; ++k)
                    if (k < p.K && w[k] == w[k])
                        raw[k] = *reinterpret_cast<const uint4 *>(landing + (static_cast<long long>(t) * p.K + k) * p.H + v * 8);
#pragma unroll
                for (int k = 0; k < kMaxTopk; ++k) {
                    if (k >= p.K || w[k] != w[k]) continue;
                    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[k]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(h[i]);
                        acc[2 * i] = fmaf(w[k], f.x, acc[2 * i]);
                        acc[2 * i + 1] = fmaf(w[k], f.y, acc[2 * i + 1]);
                    }
                }
                uint4 o;
                __nv_bfloat162 *oh = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                *reinterpret_cast<uint4 *>(out + static_cast<long long>(t) * p.H + v * 8) = o;
            }
        }
    }
}

// ------------------------------------------------------------------ dispatch layout (counts only)

// Per-rank and per-expert token counts and the token x rank membership matrix of a routing table
// (what the reference computes in examples/device/ep/csrc/kernels/layout.cu before a
// high-throughput dispatch).  Dispatch here does its own counting; this kernel serves callers that
// want the numbers up front (capacity planning, load-balance statistics).
__global__ void __launch_bounds__(256) epLayoutKernel(const int64_t *topk_idx, int T, int K, int E, int R, int *per_rank, int *per_expert,
                                                      unsigned char *in_rank) {
    extern __shared__ int hist[]; // [E] experts, then [R] ranks
    int *h_expert = hist, *h_rank = hist + E;
    for (int i = threadIdx.x; i < E + R; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const int El = E / R;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) {
        unsigned long long mask = 0;
        for (int k = 0; k < K; ++k) {
            const long long e = topk_idx[static_cast<long long>(t) * K + k];
            if (e < 0 || e >= E) continue;
            atomicAdd(h_expert + e, 1);
            mask |= 1ull << (static_cast<int>(e) / El);
        }
        for (int r = 0; r < R; ++r) {
            const bool in = (mask >> r) & 1ull;
            in_rank[static_cast<long long>(t) * R + r] = in ? 1 : 0;
            if (in) atomicAdd(h_rank + r, 1);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < E; i += blockDim.x)
        if (h_expert[i]) atomicAdd(per_expert + i, h_expert[i]);
    for (int i = threadIdx.x; i < R; i += blockDim.x)
        if (h_rank[i]) atomicAdd(per_rank + i, h_rank[i]);
}

// ------------------------------------------------------------------ barrier across ranks

__global__ void epBarrierKernel(const void *peers, int64_t off_flags, int R, int rank, uint64_t epoch, uint64_t timeout_ns, int *status,
                                int *mask) {
    const int r = threadIdx.x;
    if (r >= R) return;
    char *peer = peerBase(peers, r);
    if (peer == nullptr || ldVolatile(mask + r) != 0) return;
    __threadfence_system();
    stReleaseSys(reinterpret_cast<uint64_t *>(peer + off_flags) + rank, epoch);
    const uint64_t *mine = reinterpret_cast<const uint64_t *>(peerBase(peers, rank) + off_flags);
    if (!waitFlag(mine + r, epoch, timeout_ns)) {
        atomicExch(mask + r, 1);
        atomicOr(status, ST_PEER_TIMEOUT);
    }
}

int coopGrid(const void *kernel, int requested, size_t smem) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem);
    const int limit = sms * (per_sm > 0 ? per_sm : 1);
    int grid = requested > 0 ? requested : sms;
    return grid > limit ? limit : grid;
}

} // namespace

extern "C" int nixl_ep_dispatch_launch(const NixlEpDispatchParams *params, void *stream) {
    if (!params || !params->peers || !params->topk_idx || (!params->x && (params->phases & 1))) return cudaErrorInvalidValue;
    const NixlEpDispatchParams &p = *params;
    if (p.R <= 0 || p.R > kMaxRanks || p.E <= 0 || p.E % p.R || p.K <= 0 || p.K > kMaxTopk || p.H <= 0 || p.H % kGroup ||
        p.E / p.R > kMaxRanks * 8 || p.rank < 0 || p.rank >= p.R || p.T < 0)
        return cudaErrorInvalidValue;
    if (p.H % 512) return cudaErrorInvalidValue; // whole warps per pass; scales move as float4
    if (p.topk_weights && (p.K > 8 || p.R > 32 || p.max_tokens < p.T)) return cudaErrorInvalidValue; // a group record holds eight copies
    if (p.rows_per_expert > 0 && static_cast<long long>(p.rows_per_expert) < static_cast<long long>(p.R) * p.T) return cudaErrorInvalidValue;
    const size_t group_bytes = (2 * kMaxTopk * sizeof(int) + size_t(p.use_fp8 ? p.H : p.H * 2) + (p.H / kGroup) * sizeof(float) + 15) & ~size_t(15);
    const size_t smem = size_t(2) * p.E * sizeof(int) + (kThreads / 32) * group_bytes + 16;
    {
        // The shared-memory limit is a per-device function attribute.
        static bool attr_done[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !attr_done[dev]) {
            cudaError_t e = cudaFuncSetAttribute(epDispatchKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return e;
            attr_done[dev] = true;
        }
    }
    // With many tokens per CTA the data phase is a chain of dependent steps per token (load,
    // quantise, reserve slots, store); a second CTA per SM hides that latency.
    int requested = p.grid;
    if (requested <= 0) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (p.T >= 4 * sms) requested = 2 * sms;
    }
    const int grid = coopGrid(reinterpret_cast<const void *>(epDispatchKernel), requested, smem);
    void *args[] = {const_cast<NixlEpDispatchParams *>(params)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(epDispatchKernel), dim3(grid), dim3(kThreads), args, smem,
                                       static_cast<cudaStream_t>(stream));
}

extern "C" int nixl_ep_combine_launch(const NixlEpCombineParams *params, void *stream) {
    if (!params || !params->peers || !params->topk_idx) return cudaErrorInvalidValue;
    const NixlEpCombineParams &p = *params;
    if (p.pull == 1 && !p.send_row) return cudaErrorInvalidValue;
    if (p.pull == 2 && (p.max_tokens <= 0 || p.R > 32 || p.T > p.max_tokens || !p.x)) return cudaErrorInvalidValue;
    if (p.use_logfmt && (p.pull || p.H % 512)) return cudaErrorInvalidValue;
    if (p.R <= 0 || p.R > kMaxRanks || p.E <= 0 || p.E % p.R || p.K <= 0 || p.K > kMaxTopk || p.H <= 0 || p.H % 8 ||
        p.E / p.R > kMaxRanks * 8 || p.rank < 0 || p.rank >= p.R)
        return cudaErrorInvalidValue;
    void *args[] = {const_cast<NixlEpCombineParams *>(params)};
    if (p.pull == 2) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        static bool attr_done[64] = {};
        if (dev >= 0 && dev < 64 && !attr_done[dev]) {
            cudaError_t e = cudaFuncSetAttribute(epCombineRankReduceSend, cudaFuncAttributeMaxDynamicSharedMemorySize, kRrCtaBytes);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(epCombineRankReduceRecv, cudaFuncAttributeMaxDynamicSharedMemorySize, kRrCtaBytes);
            if (e != cudaSuccess) return e;
            attr_done[dev] = true;
        }
        const int want = 2 * (p.grid > 0 ? p.grid : sms); // p.grid counts SMs
        if (p.phases & 1) { // cooperative: its CTAs meet at a grid barrier before the flags go out
            const int grid = coopGrid(reinterpret_cast<const void *>(epCombineRankReduceSend), want, kRrCtaBytes);
            const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(epCombineRankReduceSend), dim3(grid), dim3(kThreads), args,
                                                              kRrCtaBytes, static_cast<cudaStream_t>(stream));
            if (e != cudaSuccess) return e;
        }
        if (p.phases & 2) {
            epCombineRankReduceRecv<<<want, kThreads, kRrCtaBytes, static_cast<cudaStream_t>(stream)>>>(p);
            return cudaGetLastError();
        }
        return cudaSuccess;
    }
    const int grid = coopGrid(reinterpret_cast<const void *>(epCombineKernel), p.grid, 0);
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(epCombineKernel), dim3(grid), dim3(kThreads), args, 0,
                                       static_cast<cudaStream_t>(stream));
}

extern "C" int nixl_ep_barrier_launch(const void *peers, int64_t off_flags, int32_t R, int32_t rank, uint64_t epoch, uint64_t timeout_ns,
                                      int32_t *status, int32_t *mask, void *stream) {
    if (!peers || R <= 0 || R > kMaxRanks || !status || !mask) return cudaErrorInvalidValue;
    epBarrierKernel<<<1, kMaxRanks, 0, static_cast<cudaStream_t>(stream)>>>(peers, off_flags, R, rank, epoch, timeout_ns, status, mask);
    return cudaGetLastError();
}

extern "C" int nixl_ep_layout_launch(const int64_t *topk_idx, int32_t T, int32_t K, int32_t E, int32_t R, int32_t *per_rank, int32_t *per_expert,
                                     uint8_t *in_rank, void *stream) {
    if (!topk_idx || !per_rank || !per_expert || !in_rank || T < 0 || K <= 0 || E <= 0 || R <= 0 || R > kMaxRanks || E % R) return cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(per_rank, 0, sizeof(int32_t) * R, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(per_expert, 0, sizeof(int32_t) * E, st);
    if (e != cudaSuccess) return e;
    if (T == 0) return cudaSuccess;
    const int blocks = (T + 255) / 256 < 148 ? (T + 255) / 256 : 148;
    epLayoutKernel<<<blocks, 256, sizeof(int) * (E + R), st>>>(topk_idx, T, K, E, R, per_rank, per_expert, in_rank);
    return cudaGetLastError();
}

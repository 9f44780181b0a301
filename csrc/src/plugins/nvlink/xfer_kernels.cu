// Batched descriptor copy kernels for sm_100a.
//
// Replaces the per-descriptor put/get loop of the reference's UCX backend
// (src/plugins/ucx/ucx_backend.cpp:1184-1265): a WRITE pushes with local loads and
// stores into the peer's mapped memory, a READ pulls with loads over NVLink; both are
// the same kernel because source and destination are just device-visible addresses
// (local HBM, a peer GPU's HBM through NVLink, or pinned host memory through PCIe).
// Completion and the hand-off to the host are fused into the kernel's tail.
#include "plugins/nvlink/xfer_kernels.h"

#include <cuda.h>

namespace nixl_nvlink {
namespace {

constexpr int kThreads = 512;
constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 ld_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void st_stream(uint4 *p, const uint4 &v) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ void st_release_sys(uint64_t *p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

struct Vec32 {
    float v[8];
};
__device__ __forceinline__ Vec32 ld_stream32(const void *p) {
    Vec32 r;
    asm volatile("ld.global.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void st_stream32(void *p, const Vec32 &r) {
    asm volatile("st.global.L1::no_allocate.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]),
                 "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]), "f"(r.v[7])
                 : "memory");
}

// Copies n bytes with a group of kGroup threads (tid = index within the group).  Fastest path: source and destination share their offset
// within 32 bytes, so after a short head both take 256-bit accesses (sm_100: one warp
// instruction moves 1 KiB).  Otherwise 16-byte, 4-byte or byte accesses by relative alignment.
template<int kGroup> __device__ __forceinline__ void copyRangeBy(const char *__restrict__ s, char *__restrict__ d, size_t n, const unsigned tid) {
    constexpr int kThreads = kGroup; // the threads that share this range: a whole CTA, or one warp
    if ((((uintptr_t)s ^ (uintptr_t)d) & 31) == 0) {
        size_t head = (32 - ((uintptr_t)s & 31)) & 31;
        if (head > n) head = n;
        if (tid < head) d[tid] = s[tid];
        s += head;
        d += head;
        n -= head;
        const size_t nvec = n >> 5;
        size_t i = tid;
        for (; i + (kUnroll - 1) * kThreads < nvec; i += kUnroll * kThreads) {
            Vec32 v[kUnroll];
#pragma unroll
            for (int k = 0; k < kUnroll; ++k) v[k] = ld_stream32(s + ((i + k * kThreads) << 5));
#pragma unroll
            for (int k = 0; k < kUnroll; ++k) st_stream32(d + ((i + k * kThreads) << 5), v[k]);
        }
        for (; i < nvec; i += kThreads) st_stream32(d + (i << 5), ld_stream32(s + (i << 5)));
        const size_t done = nvec << 5;
        const size_t tail = n - done;
        if (tid < tail) d[done + tid] = s[done + tid];
    } else if ((((uintptr_t)s ^ (uintptr_t)d) & 15) == 0) {
        size_t head = (16 - ((uintptr_t)s & 15)) & 15;
        if (head > n) head = n;
        if (tid < head) d[tid] = s[tid];
        s += head;
        d += head;
        n -= head;
        const size_t nvec = n >> 4;
        const uint4 *sv = reinterpret_cast<const uint4 *>(s);
        uint4 *dv = reinterpret_cast<uint4 *>(d);
        size_t i = tid;
        // kUnroll independent loads in flight per thread before the first store.
        for (; i + (kUnroll - 1) * kThreads < nvec; i += kUnroll * kThreads) {
            uint4 v[kUnroll];
#pragma unroll
            for (int k = 0; k < kUnroll; ++k) v[k] = ld_stream(sv + i + k * kThreads);
#pragma unroll
            for (int k = 0; k < kUnroll; ++k) st_stream(dv + i + k * kThreads, v[k]);
        }
        for (; i < nvec; i += kThreads) st_stream(dv + i, ld_stream(sv + i));
        const size_t done = nvec << 4;
        const size_t tail = n - done;
        if (tid < tail) d[done + tid] = s[done + tid];
    } else if ((((uintptr_t)s ^ (uintptr_t)d) & 3) == 0) {
        size_t head = (4 - ((uintptr_t)s & 3)) & 3;
        if (head > n) head = n;
        if (tid < head) d[tid] = s[tid];
        s += head;
        d += head;
        n -= head;
        const size_t nw = n >> 2;
        const uint32_t *sw = reinterpret_cast<const uint32_t *>(s);
        uint32_t *dw = reinterpret_cast<uint32_t *>(d);
        for (size_t i = tid; i < nw; i += kThreads) dw[i] = sw[i];
        const size_t done = nw << 2;
        if (tid < n - done) d[done + tid] = s[done + tid];
    } else {
        for (size_t i = tid; i < n; i += kThreads) d[i] = s[i];
    }
}

__device__ __forceinline__ void copyRange(const char *__restrict__ s, char *__restrict__ d, size_t n) {
    copyRangeBy<kThreads>(s, d, n, threadIdx.x);
}

// Which descriptor owns chunk c?  Upper-bound search in the prefix array.
template<class StartFn> __device__ __forceinline__ uint32_t ownerOf(uint32_t c, uint32_t n, StartFn start) {
    uint32_t lo = 0, hi = n; // invariant: start(lo) <= c < start(hi)
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (start(mid) <= c) lo = mid; else hi = mid;
    }
    return lo;
}

// Tail shared by all variants: publish completion once every CTA has finished.
// One acquire-release add at GPU scope chains the CTAs (each CTA's stores are ordered before
// its add by the barrier; the add that sees all others therefore follows every store), and one
// release store at system scope makes all of it visible before the completion word changes.
// System-scope fences are expensive when stores to a peer GPU and to host memory are in
// flight, so the tail uses exactly one.
__device__ __forceinline__ void finishBatch(const XferLaunch &p) {
    __syncthreads();
    if (threadIdx.x == 0) {
        bool last = true;
        if (gridDim.x > 1) {
            unsigned prev;
            asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(p.doneCounter) : "memory");
            last = prev == gridDim.x - 1;
            if (last) *p.doneCounter = 0; // ready for the next post of this request (stream order protects it)
        }
        if (last) {
            if (p.notifWord) st_release_sys(p.notifWord, p.notifSeq); // the target learns of the data without this side's host
            st_release_sys(p.hostFlag, p.seq);
        }
    }
}

__global__ void __launch_bounds__(kThreads) batchCopyVector(const __grid_constant__ XferLaunch p) {
    const bool inl = p.table == nullptr;
    const size_t chunk = size_t(1) << p.chunkShift;
    for (uint32_t c = blockIdx.x; c < p.totalChunks; c += gridDim.x) {
        uint32_t i, first;
        XferDesc d;
        if (inl) {
            i = ownerOf(c, p.nDescs, [&](uint32_t k) { return p.inlStart[k]; });
            first = p.inlStart[i];
            d = p.inl[i];
        } else {
            i = ownerOf(c, p.nDescs, [&](uint32_t k) { return __ldg(p.chunkStart + k); });
            first = __ldg(p.chunkStart + i);
            d.src = __ldg(&p.table[i].src);
            d.dst = __ldg(&p.table[i].dst);
            d.len = __ldg(&p.table[i].len);
        }
        const size_t off = size_t(c - first) << p.chunkShift;
        const size_t n = d.len - off < chunk ? d.len - off : chunk;
        copyRange(reinterpret_cast<const char *>(d.src) + off, reinterpret_cast<char *>(d.dst) + off, n);
    }
    finishBatch(p);
}

// ------------------------------------------------------------------ bulk (TMA 1-D) variant
//
// One elected thread per CTA drives a ring of shared-memory stages:
//   cp.async.bulk global -> shared (completion on an mbarrier), then
//   cp.async.bulk shared -> global (completion tracked by bulk groups).
// No multicast anywhere: the source may be another GPU's memory.  Every wait is bounded;
// on expiry the kernel records the failure in the completion word's top bit and leaves.

constexpr int kStages = 4;
constexpr uint32_t kStageBytes = 32 * 1024;
constexpr uint64_t kWaitBudgetNs = 2000000000ull; // a bulk load that has not landed after 2 s is treated as lost
constexpr uint64_t kDrainBudgetNs = 100000000ull; // after a loss: 0.1 s for each younger load before the CTA leaves
static_assert(kStages == 4, "the wait_group.read switch in batchCopyBulk enumerates kStages cases");

__device__ __forceinline__ uint64_t globalTimerNs() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smemAddr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbarInit(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarExpectTx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smemAddr(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulkLoad(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smemAddr(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smemAddr(bar))
                 : "memory");
}
__device__ __forceinline__ void bulkStore(void *gdst, const void *smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smemAddr(smem_src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template<int N> __device__ __forceinline__ void bulkWaitRead() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template<int N> __device__ __forceinline__ void bulkWait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

// Waits for a phase of an mbarrier for at most budget_ns (looking at the clock only now and then).
__device__ __forceinline__ bool mbarWaitBounded(uint64_t *bar, uint32_t parity, uint64_t budget_ns) {
    uint32_t spins = 0;
    uint64_t t0 = 0;
    while (!mbarTryWait(bar, parity)) {
        if ((++spins & 255u) == 0) {
            const uint64_t now = globalTimerNs();
            if (t0 == 0) t0 = now;
            else if (now - t0 > budget_ns) return false;
        }
    }
    return true;
}

__global__ void __launch_bounds__(128) batchCopyBulk(const __grid_constant__ XferLaunch p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t full[kStages];
    __shared__ int failed;
    const bool inl = p.table == nullptr;
    const size_t chunk = size_t(1) << p.chunkShift;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbarInit(&full[s], 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    uint32_t issued = 0; // pieces handed to the ring by thread 0
    for (uint32_t c = blockIdx.x; c < p.totalChunks; c += gridDim.x) {
        uint32_t i, first;
        XferDesc d;
        if (inl) {
            i = ownerOf(c, p.nDescs, [&](uint32_t k) { return p.inlStart[k]; });
            first = p.inlStart[i];
            d = p.inl[i];
        } else {
            i = ownerOf(c, p.nDescs, [&](uint32_t k) { return __ldg(p.chunkStart + k); });
            first = __ldg(p.chunkStart + i);
            d.src = __ldg(&p.table[i].src);
            d.dst = __ldg(&p.table[i].dst);
            d.len = __ldg(&p.table[i].len);
        }
        const size_t off = size_t(c - first) << p.chunkShift;
        const size_t n = d.len - off < chunk ? d.len - off : chunk;
        const char *s = reinterpret_cast<const char *>(d.src) + off;
        char *dst = reinterpret_cast<char *>(d.dst) + off;
        // Bulk copies need 16-byte aligned addresses and sizes; anything else goes the SIMT way.
        const bool bulk_ok = ((((uintptr_t)s | (uintptr_t)dst) & 15) == 0) && n >= 16;
        if (!bulk_ok) {
            for (size_t k = threadIdx.x; k < n; k += blockDim.x) dst[k] = s[k];
            continue;
        }
        const size_t body = n & ~size_t(15);
        if (threadIdx.x == 0 && !failed) {
            // Software pipeline: up to kStages loads in flight.  Piece g uses slot g % kStages, and
            // its store is bulk group number g.  Before slot g % kStages is loaded again, group
            // g - kStages must have finished READING shared memory; `stored_total - 1 - (g - kStages)`
            // groups were committed after it, which is the number wait_group.read may leave pending.
            // In steady state that number is 0: the store just issued is waited for (its read of
            // shared memory, not its arrival), while kStages - 1 younger loads stay in flight.
            const uint32_t pieces = static_cast<uint32_t>((body + kStageBytes - 1) / kStageBytes);
            uint32_t loaded = 0, stored = 0;
            while (stored < pieces) {
                while (loaded < pieces && loaded - stored < kStages) {
                    const uint32_t g = issued + loaded;
                    const uint32_t slot = g % kStages;
                    if (g >= kStages) {
                        const uint32_t may_pend = (issued + stored) - 1 - (g - kStages); // 0 .. kStages - 1
                        switch (may_pend) {
                        case 0: bulkWaitRead<0>(); break;
                        case 1: bulkWaitRead<1>(); break;
                        case 2: bulkWaitRead<2>(); break;
                        default: bulkWaitRead<3>(); break;
                        }
                    }
                    const size_t o = size_t(loaded) * kStageBytes;
                    const uint32_t bytes = static_cast<uint32_t>(body - o < kStageBytes ? body - o : kStageBytes);
                    mbarExpectTx(&full[slot], bytes);
                    bulkLoad(smem + size_t(slot) * kStageBytes, s + o, bytes, &full[slot]);
                    ++loaded;
                }
                const uint32_t g = issued + stored;
                const uint32_t slot = g % kStages;
                const uint32_t parity = (g / kStages) & 1;
                if (!mbarWaitBounded(&full[slot], parity, kWaitBudgetNs)) {
                    failed = 1;
                    // Loads already issued still target this CTA's shared memory: give each a short
                    // second chance to land before the CTA may exit and its shared memory be reused.
                    for (uint32_t k = stored + 1; k < loaded; ++k) {
                        const uint32_t gk = issued + k;
                        mbarWaitBounded(&full[gk % kStages], (gk / kStages) & 1, kDrainBudgetNs);
                    }
                    break;
                }
                const size_t o = size_t(stored) * kStageBytes;
                const uint32_t bytes = static_cast<uint32_t>(body - o < kStageBytes ? body - o : kStageBytes);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                bulkStore(dst + o, smem + size_t(slot) * kStageBytes, bytes);
                bulkCommit();
                ++stored;
            }
            issued += pieces;
        }
        // Sub-16-byte tail of the chunk.
        if (threadIdx.x >= 32 && threadIdx.x - 32 < n - body) dst[body + threadIdx.x - 32] = s[body + threadIdx.x - 32];
    }
    if (threadIdx.x == 0) bulkWait<0>(); // this CTA's bulk stores are complete
    __syncthreads();
    if (threadIdx.x == 0) {
        asm volatile("fence.proxy.async;" ::: "memory"); // async-proxy stores before the generic-proxy flag
        if (failed) atomicOr(reinterpret_cast<unsigned long long *>(p.hostFlag), 1ull << 63);
        bool last = true;
        if (gridDim.x > 1) {
            unsigned prev;
            asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(p.doneCounter) : "memory");
            last = prev == gridDim.x - 1;
            if (last) *p.doneCounter = 0;
        }
        if (last) {
            // Bit 63 set by any CTA marks the batch as failed; keep it.
            const unsigned long long cur = failed ? (1ull << 63) : (atomicAdd(reinterpret_cast<unsigned long long *>(p.hostFlag), 0ull) & (1ull << 63));
            if (p.notifWord && !cur) st_release_sys(p.notifWord, p.notifSeq); // a failed batch notifies nobody: the host voids the slot
            st_release_sys(p.hostFlag, p.seq | cur);
        }
    }
}

// ------------------------------------------------------------------ doorbell proxy (contract: xfer_kernels.h)

constexpr uint64_t kProxyGraceNs = 1000000000ull; // a worker that has not heard from the polling CTA for lifeNs + 1 s leaves

__device__ __forceinline__ void ldVolatile16(const void *p, uint64_t &x, uint64_t &y) {
    asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(x), "=l"(y) : "l"(p) : "memory");
}
__device__ __forceinline__ void stReleaseGpu(uint64_t *p, uint64_t v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ldVolatile8(const void *p) {
    uint64_t v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Sequence word of a device-ring entry: launch number in the top 16 bits, command number + 1 below.
__device__ __forceinline__ uint64_t ringTag(uint64_t gen, uint64_t n) { return ((gen & 0xffffull) << 48) | ((n + 1) & 0xffffffffffffull); }

struct ProxyWork {
    uint64_t a, b, kind, count;
    uint32_t shift, per, total;
};

__device__ __forceinline__ ProxyWork proxyDecode(uint64_t a, uint64_t b, uint64_t c) {
    ProxyWork w;
    w.a = a;
    w.b = b;
    w.kind = (c >> 44) & 15u;
    w.shift = static_cast<uint32_t>((c >> 38) & 63u);
    const uint64_t low = c & ((1ull << 38) - 1);
    if (w.kind == kProxyInline) {
        w.count = low;
        w.per = 0;
        w.total = static_cast<uint32_t>((low + (uint64_t(1) << w.shift) - 1) >> w.shift);
    } else {
        w.count = low & 0xffffffull;
        w.per = static_cast<uint32_t>(low >> 24);
        // The tables of a request may have been written while this kernel was already running: read
        // them past L1 (ld.global.cg), never through the non-coherent path.
        w.total = w.kind == kProxyTable ? (w.per ? w.per * static_cast<uint32_t>(w.count) : __ldcg(reinterpret_cast<const uint32_t *>(b) + w.count)) : 0;
    }
    return w;
}

// One warp copies chunk `ch` of the command.
__device__ __forceinline__ void proxyCopyChunk(const ProxyWork &w, uint32_t ch, unsigned lane) {
    const size_t chunk = size_t(1) << w.shift;
    if (w.kind == kProxyInline) {
        const size_t off = size_t(ch) << w.shift;
        const size_t len = w.count - off < chunk ? w.count - off : chunk;
        copyRangeBy<32>(reinterpret_cast<const char *>(w.a) + off, reinterpret_cast<char *>(w.b) + off, len, lane);
        return;
    }
    const XferDesc *table = reinterpret_cast<const XferDesc *>(w.a);
    const uint32_t *starts = reinterpret_cast<const uint32_t *>(w.b);
    uint32_t i, first;
    if (w.per) { // every descriptor has the same number of chunks: no search
        i = ch / w.per;
        first = i * w.per;
    } else {
        i = ownerOf(ch, static_cast<uint32_t>(w.count), [&](uint32_t k) { return __ldcg(starts + k); });
        first = __ldcg(starts + i);
    }
    const uint64_t src = __ldcg(&table[i].src), dst = __ldcg(&table[i].dst), dlen = __ldcg(&table[i].len);
    const size_t off = size_t(ch - first) << w.shift;
    const size_t len = dlen - off < chunk ? dlen - off : chunk;
    copyRangeBy<32>(reinterpret_cast<const char *>(src) + off, reinterpret_cast<char *>(dst) + off, len, lane);
}

constexpr unsigned kProxyWarps = kThreads / 32;
constexpr unsigned kProxyChunksPerWarp = 2; // chunks one warp takes of a command before another CTA is drawn in

__global__ void __launch_bounds__(kThreads) proxyKernel(const __grid_constant__ ProxyLaunch p) {
    __shared__ ProxyCmd cmd;
    __shared__ unsigned long long cmdNumber;
    const unsigned workers = gridDim.x - 1;
    const unsigned lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;

    if (blockIdx.x == 0) {
        // ---------------- polling CTA: host ring -> device ring; commands of at most one chunk per warp it runs itself.
        uint64_t n = p.start, floor_head = 0;
        const uint64_t t_start = globalTimerNs();
        uint64_t t_last = t_start;
        bool skip_owed = false; // a command this CTA ran itself has not been entered in the device ring yet
        uint32_t empty_polls = 0; // polls that found nothing since the last command
        for (;;) {
            if (threadIdx.x == 0) {
                // Room in the device ring: no worker may be a whole ring behind command `upto`.  Workers wait for
                // nothing but this CTA and their own copies, so the wait ends; it is bounded all the same.
                auto wait_room = [&](uint64_t upto) {
                    while (upto - floor_head >= kProxySlots) {
                        uint64_t m = ~0ull;
                        for (unsigned w = 0; w < workers; ++w) {
                            const uint64_t h = ldVolatile8(&p.shared->workerHead[w]);
                            m = h < m ? h : m;
                        }
                        floor_head = m;
                        if (globalTimerNs() - t_start > p.lifeNs + kProxyGraceNs) break;
                    }
                };
                auto publish = [&](uint64_t a, uint64_t b, uint64_t c) {
                    wait_room(n);
                    ProxyCmd *d = &p.shared->ring[n % kProxySlots];
                    d->a = a;
                    d->b = b;
                    d->c = c;
                    stReleaseGpu(&d->seq, ringTag(p.gen, n));
                };
                if (skip_owed) { // the workers just step over a command that was run here
                    n -= 1;
                    publish(0, 0, proxyPackC(n + 1, kProxySkip, 0, 0));
                    n += 1;
                    skip_owed = false;
                }
                for (;;) {
                    // Two slots per poll, all four loads in flight together: when requests stream in, one PCIe
                    // round trip hands over two commands.
                    const ProxyCmd *slot = p.hostRing + (n % kProxySlots), *next = p.hostRing + ((n + 1) % kProxySlots);
                    uint64_t seq, a, b, c, seq2, a2, b2, c2;
                    ldVolatile16(&slot->seq, seq, a);
                    ldVolatile16(&slot->b, b, c);
                    ldVolatile16(&next->seq, seq2, a2);
                    ldVolatile16(&next->b, b2, c2);
                    const uint64_t now = globalTimerNs();
                    bool leave = now - t_start > p.lifeNs;
                    if (seq == n + 1 && (c >> 48) == ((n + 1) & 0xffffull)) {
                        t_last = now;
                        const bool second = seq2 == n + 2 && (c2 >> 48) == ((n + 2) & 0xffffull);
                        const uint64_t kind = (c >> 44) & 15u, low = c & ((1ull << 38) - 1);
                        const uint32_t shift = static_cast<uint32_t>((c >> 38) & 63u);
                        // Small enough for this CTA alone?  (inline: by length; table: only when the chunk count is in the command)
                        const uint64_t chunks = kind == kProxyInline ? (low + (uint64_t(1) << shift) - 1) >> shift : (low >> 24) * (low & 0xffffffull);
                        // ... and nothing queued around it?  A command found by the first poll after the previous one, or
                        // with a successor already waiting, is part of a stream, and the workers overlap those; one that
                        // arrives alone after an idle poll is run here, which saves the hop through the device ring.
                        const bool alone = empty_polls > 0 && !second;
                        empty_polls = 0;
                        if (alone && chunks >= 1 && chunks <= kProxyWarps) {
                            skip_owed = true; // entered in the device ring after the copy: off the critical path
                            cmd.a = a;
                            cmd.b = b;
                            cmd.c = c;
                            cmdNumber = n;
                            ++n;
                            break; // run it (all threads, below)
                        }
                        publish(a, b, c);
                        ++n;
                        if (second) {
                            publish(a2, b2, c2);
                            ++n;
                        }
                    } else {
                        ++empty_polls;
                        if (now - t_last > p.idleNs) leave = true;
                    }
                    if (leave) {
                        publish(0, 0, proxyPackC(n + 1, kProxyExit, 0, 0));
                        st_release_sys(p.exitWord, (1ull << 63) | n);
                        cmd.c = proxyPackC(0, kProxyExit, 0, 0);
                        break;
                    }
                }
            }
            __syncthreads();
            const uint64_t a = cmd.a, b = cmd.b, c = cmd.c;
            const uint64_t number = cmdNumber;
            __syncthreads();
            if (((c >> 44) & 15u) == kProxyExit) return;
            const ProxyWork w = proxyDecode(a, b, c);
            if (warp < w.total) proxyCopyChunk(w, warp, lane);
            __syncthreads();
            if (threadIdx.x == 0) st_release_sys(&p.done[number % kProxySlots], number + 1);
        }
    }

    // ---------------- worker CTAs
    const unsigned w = blockIdx.x - 1;
    const uint64_t t_start = globalTimerNs();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned long long *>(&p.shared->workerHead[w]) = p.start;
    for (uint64_t n = p.start;; ++n) {
        if (threadIdx.x == 0) {
            ProxyCmd *slot = &p.shared->ring[n % kProxySlots];
            const uint64_t expect = ringTag(p.gen, n);
            uint32_t spins = 0;
            uint64_t seq, a, b, c;
            for (;;) {
                // both halves in flight at once; c repeats the low bits of the command number, so a half read
                // before the polling CTA had written it is recognised
                ldVolatile16(&slot->seq, seq, a);
                ldVolatile16(&slot->b, b, c);
                if (seq == expect && (c >> 48) == ((n + 1) & 0xffffull)) break;
                if ((++spins & 1023u) == 0 && globalTimerNs() - t_start > p.lifeNs + kProxyGraceNs) {
                    c = proxyPackC(0, kProxyExit, 0, 0);
                    break;
                }
            }
            asm volatile("fence.acq_rel.gpu;" ::: "memory"); // the command's tables are read after the command
            cmd.a = a;
            cmd.b = b;
            cmd.c = c;
        }
        __syncthreads();
        const uint64_t a = cmd.a, b = cmd.b, c = cmd.c;
        __syncthreads(); // everyone has its copy before thread 0 fetches the next command
        const uint64_t kind = (c >> 44) & 15u;
        if (kind == kProxyExit) return;
        if (kind != kProxySkip) {
            const ProxyWork work = proxyDecode(a, b, c);
            // Every warp takes whole chunks, so that a batch of 4 KiB descriptors keeps sixteen of them in flight
            // per CTA; a command draws in only as many CTAs as it has chunks for, and the first one rotates with the
            // command number, so that consecutive commands run side by side on different CTAs.
            const unsigned per_cta = kProxyWarps * kProxyChunksPerWarp;
            const unsigned want = (work.total + per_cta - 1) / per_cta;
            const unsigned parts = want < workers ? want : workers;
            const unsigned r = (w + workers - static_cast<unsigned>(n % workers)) % workers;
            if (r < parts) {
                for (uint32_t ch = r * kProxyWarps + warp; ch < work.total; ch += parts * kProxyWarps) proxyCopyChunk(work, ch, lane);
                __syncthreads();
                if (threadIdx.x == 0) {
                    bool last = true;
                    if (parts > 1) {
                        unsigned prev;
                        unsigned int *ctr = &p.shared->counter[n % kProxySlots];
                        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(ctr) : "memory");
                        last = prev == parts - 1;
                        if (last) *ctr = 0;
                    }
                    if (last) st_release_sys(&p.done[n % kProxySlots], n + 1);
                }
            }
        }
        if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned long long *>(&p.shared->workerHead[w]) = n + 1;
    }
}

__global__ void signalOnly(uint64_t *flag, uint64_t seq, uint64_t *notifWord, uint64_t notifSeq) {
    if (notifWord) st_release_sys(notifWord, notifSeq);
    st_release_sys(flag, seq);
}

} // namespace

cudaError_t launchProxy(const ProxyLaunch &p, int workers, cudaStream_t stream) {
    if (workers < 1 || workers > kProxyMaxWorkers || !p.hostRing || !p.shared || !p.done || !p.exitWord) return cudaErrorInvalidValue;
    proxyKernel<<<workers + 1, kThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launchSignal(uint64_t *hostFlag, uint64_t seq, uint64_t *notifWord, uint64_t notifSeq, cudaStream_t stream) {
    signalOnly<<<1, 1, 0, stream>>>(hostFlag, seq, notifWord, notifSeq);
    return cudaGetLastError();
}

int defaultGridCtas(int device) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
    // Eight times what is resident at once (two CTAs of 512 threads per SM): with many more CTAs
    // than slots the tail of a large copy balances itself, which measured 3.22 TB/s against 2.95
    // with a grid of resident CTAs only.  Small batches never get here: the grid is capped by the
    // number of chunks.
    return sms * 16;
}

cudaError_t launchBatchCopy(const XferLaunch &params, int grid_ctas, CopyPath path, cudaStream_t stream) {
    if (params.totalChunks == 0) return cudaErrorInvalidValue;
    int grid = grid_ctas > 0 ? grid_ctas : 2368;
    // Up to three rounds of resident CTAs' worth of chunks run as a persistent grid (every CTA
    // loops over its share: no second, half-empty wave); beyond that one short-lived CTA per chunk,
    // up to the configured maximum, balances better.
    static int sm_count[64] = {}; // per device, looked up once (this is the post path)
    int dev = 0;
    cudaGetDevice(&dev);
    int sms = (dev >= 0 && dev < 64) ? sm_count[dev] : 0;
    if (sms <= 0) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        if (dev >= 0 && dev < 64) sm_count[dev] = sms;
    }
    const int resident = 2 * sms;
    if (grid > resident && params.totalChunks < 3u * static_cast<uint32_t>(resident)) grid = resident;
    if (static_cast<uint32_t>(grid) > params.totalChunks) grid = static_cast<int>(params.totalChunks);
    if (path == CopyPath::BULK) {
        static bool attr_set[64] = {};
        const size_t smem = size_t(kStages) * kStageBytes;
        if (dev >= 0 && dev < 64 && !attr_set[dev]) {
            cudaError_t e = cudaFuncSetAttribute(batchCopyBulk, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (e != cudaSuccess) return e;
            attr_set[dev] = true;
        }
        batchCopyBulk<<<grid, 128, smem, stream>>>(params);
    } else {
        batchCopyVector<<<grid, kThreads, 0, stream>>>(params);
    }
    return cudaGetLastError();
}

} // namespace nixl_nvlink

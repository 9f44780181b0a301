// PTX wrappers shared by the tcgen05 GEMM kernels (sm_100a): mbarrier, TMA tile loads, tcgen05
// MMA / commit / TMEM loads, shared-memory matrix descriptors.  Every wait is bounded.
#ifndef NIXL_B200_TCGEN05_PTX_CUH
#define NIXL_B200_TCGEN05_PTX_CUH

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace nixl_tc {


__device__ __forceinline__ uint32_t smemU32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint64_t nowNs() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbarInit(uint64_t *b, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemU32(b)), "r"(count));
}
__device__ __forceinline__ void mbarExpectTx(uint64_t *b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemU32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint64_t *b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemU32(b)) : "memory");
}
// One blocking attempt.  The suspend-time hint (nanoseconds) bounds how long the hardware may
// park the thread before it returns "not yet": without it the limit is system-dependent, and
// the caller's own time budget would only be looked at after many such sleeps.
__device__ __forceinline__ bool mbarTry(uint64_t *b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smemU32(b)), "r"(parity), "r"(20000u)
                 : "memory");
    return ok != 0;
}
// Non-blocking look at a phase (never suspends the thread): used to start a poll before work that
// does not depend on it, so the barrier's latency is hidden behind that work.
__device__ __forceinline__ bool mbarTest(uint64_t *b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smemU32(b)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Bounded wait; false when the budget ran out or another role aborted.
__device__ __forceinline__ bool mbarWait(uint64_t *b, uint32_t parity, volatile int *abort_flag) {
    if (mbarTry(b, parity)) return true;
    // The budget is counted on the SM's cycle counter (cheap to read after every failed attempt;
    // the global nanosecond timer is not): 2^33 cycles are 4.4 s at 1.97 GHz and more when the
    // clock is lower.
    const long long t0 = clock64();
    while (!mbarTry(b, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > (1ll << 33)) {
            *abort_flag = 1;
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tmaLoad2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smemU32(smem_dst)),
                 "l"(map), "r"(smemU32(bar)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcCommit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemU32(bar)) : "memory");
}
__device__ __forceinline__ void tcMma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
                 : "memory");
}
// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread = lane = row).
__device__ __forceinline__ void tmemLoad32(uint32_t addr, float (&v)[32]) {
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
}
// Waits for outstanding TMEM loads.  The registers are listed as read-write operands so that no
// use of them can be scheduled above the wait (the load instruction returns before its data).
__device__ __forceinline__ void tmemLoadWait(float (&v)[32]) {
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]),
                   "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]),
                   "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]),
                   "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// Shared-memory matrix descriptor for a K-major tile of 128-byte rows written by TMA with the
// 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the leading offset
// is unused for this layout, descriptor version 1 (sm_100), layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t smemDesc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);       // start address, bits [0,14)
    d |= static_cast<uint64_t>(1) << 16;                           // leading byte offset (ignored), bits [16,30)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                   // stride byte offset, bits [32,46)
    d |= static_cast<uint64_t>(1) << 46;                           // version, bits [46,48)
    d |= static_cast<uint64_t>(2) << 61;                           // layout type, bits [61,64)
    return d;
}

__device__ __forceinline__ uint64_t ldAcquireSys(const uint64_t *p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Epilogue store of a 32-row x 64-column bf16 block held one row per lane (64 fp32 per thread).
// Written row by row, every store instruction would touch 32 different 128-byte lines with 16
// bytes each.  Instead eight lanes exchange their 16-byte pieces (an 8 x 8 transpose in three
// butterfly steps), after which lane 8g + c holds piece c of rows 8g .. 8g + 7 and each
// instruction writes whole 128-byte runs.  `out` points at this lane group's first row, already
// advanced by (lane & 7) * 8 columns; rows_left counts the group's rows that may be written.
__device__ __forceinline__ void storeRows64(const float (&lo)[32], const float (&hi)[32], __nv_bfloat16 *out, long long row_stride, int rows_left,
                                            int lane) {
    uint4 piece[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float *src = i < 4 ? lo + 8 * i : hi + 8 * (i - 4);
        __nv_bfloat162 *hh = reinterpret_cast<__nv_bfloat162 *>(&piece[i]);
#pragma unroll
        for (int x = 0; x < 4; ++x) hh[x] = __floats2bfloat162_rn(src[2 * x], src[2 * x + 1]);
    }
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i & m) continue;
            const int j = i | m;
            const bool upper = (lane & m) != 0;
            const uint4 send = upper ? piece[i] : piece[j];
            uint4 recv;
            recv.x = __shfl_xor_sync(0xffffffffu, send.x, m);
            recv.y = __shfl_xor_sync(0xffffffffu, send.y, m);
            recv.z = __shfl_xor_sync(0xffffffffu, send.z, m);
            recv.w = __shfl_xor_sync(0xffffffffu, send.w, m);
            if (upper) piece[i] = recv; else piece[j] = recv;
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < rows_left) *reinterpret_cast<uint4 *>(out + static_cast<long long>(i) * row_stride) = piece[i];
}

} // namespace nixl_tc

#endif

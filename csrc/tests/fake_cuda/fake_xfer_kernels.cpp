// The copy kernels of the NVLINK backend (xfer_kernels.h) as host functions that run as stream tasks of the stand-in
// runtime.  They keep the contract the backend's host side relies on: the data moves, the "last CTA" counter is zero
// afterwards, the notification word is stored before the completion word, both with release semantics; the doorbell
// proxy reads the host ring in order from `start`, stores done[n % slots] = n + 1 per command, and leaves after its
// idle time or at the end of its life by storing (1 << 63) | next command to the exit word.
#include <atomic>
#include <chrono>
#include <cstring>
#include <thread>

#include "plugins/nvlink/xfer_kernels.h"

namespace nixl_nvlink {

namespace {
void storeRelease(uint64_t *p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }

uint64_t nowNs() {
    return static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count());
}

void copyAll(const XferDesc *descs, uint32_t n) {
    for (uint32_t i = 0; i < n; ++i)
        std::memmove(reinterpret_cast<void *>(descs[i].dst), reinterpret_cast<const void *>(descs[i].src), descs[i].len);
}
} // namespace

cudaError_t launchBatchCopy(const XferLaunch &params, int, CopyPath, cudaStream_t stream) {
    if (params.totalChunks == 0) return cudaErrorInvalidValue;
    if (fake_cuda::takeLaunchFailure(fake_cuda::LaunchKind::Copy)) return cudaErrorUnknown;
    const XferLaunch p = params; // by value, as kernel parameters are
    fake_cuda::enqueue(stream, [p] {
        // The table is read when the kernel runs, not when it is launched: an upload that has not landed, or a table
        // freed too early, shows as wrong bytes here just as it would on a GPU.
        const XferDesc *descs = p.table ? p.table : p.inl;
        copyAll(descs, p.nDescs);
        if (p.doneCounter) *p.doneCounter = 0;
        if (p.notifWord) storeRelease(p.notifWord, p.notifSeq);
        storeRelease(p.hostFlag, p.seq);
    });
    return cudaSuccess;
}

cudaError_t launchSignal(uint64_t *hostFlag, uint64_t seq, uint64_t *notifWord, uint64_t notifSeq, cudaStream_t stream) {
    if (fake_cuda::takeLaunchFailure(fake_cuda::LaunchKind::Signal)) return cudaErrorUnknown;
    fake_cuda::enqueue(stream, [=] {
        if (notifWord) storeRelease(notifWord, notifSeq);
        storeRelease(hostFlag, seq);
    });
    return cudaSuccess;
}

cudaError_t launchProxy(const ProxyLaunch &launch, int, cudaStream_t stream) {
    if (fake_cuda::takeLaunchFailure(fake_cuda::LaunchKind::Proxy)) return cudaErrorUnknown;
    const ProxyLaunch p = launch;
    fake_cuda::enqueue(stream, [p] {
        const uint64_t t_start = nowNs();
        uint64_t t_last = t_start, n = p.start;
        for (;;) {
            const ProxyCmd *slot = p.hostRing + (n % kProxySlots);
            const uint64_t seq = __atomic_load_n(&slot->seq, __ATOMIC_ACQUIRE);
            const uint64_t now = nowNs();
            // (The device reads the whole slot at once and tells a half-written one by the tag in c; here the
            // doorbell's release / acquire pair already orders the other three words.)
            const uint64_t a = seq == n + 1 ? slot->a : 0, b = seq == n + 1 ? slot->b : 0, c = seq == n + 1 ? slot->c : 0;
            if (seq == n + 1 && (c >> 48) == ((n + 1) & 0xffffull)) {
                t_last = now;
                const uint64_t kind = (c >> 44) & 15u, low = c & ((1ull << 38) - 1);
                if (kind == kProxyInline) {
                    std::memmove(reinterpret_cast<void *>(b), reinterpret_cast<const void *>(a), low);
                } else if (kind == kProxyTable) {
                    copyAll(reinterpret_cast<const XferDesc *>(a), static_cast<uint32_t>(low & 0xffffffull));
                }
                storeRelease(&p.done[n % kProxySlots], n + 1);
                ++n;
                if (now - t_start <= p.lifeNs) continue;
            } else if (now - t_last <= p.idleNs && now - t_start <= p.lifeNs) {
                std::this_thread::yield();
                continue;
            }
            storeRelease(p.exitWord, (1ull << 63) | n);
            return;
        }
    });
    return cudaSuccess;
}

int defaultGridCtas(int) { return 148 * 2 * 8; }

} // namespace nixl_nvlink

// nvlink_probe: what one NVLink direction between two GPUs of a machine delivers to each way of
// moving bytes - SM-issued stores into the peer (push), SM-issued loads from the peer (pull),
// the copy engine, and mixtures of them - one way and with the opposite direction busy.
//
// The NVLINK backend's copy kernel is tuned against these figures, and the ncu NVLink counters
// (nvltx__bytes_data_user / nvltx__bytes_data_protocol) are captured on this program's
// kernels: a small single-process two-GPU case.
//
// Usage: nvlink_probe [--mib N] [--iters K] [--case NAME] [--dev-a A] [--dev-b B]
//   cases: all (default), push, pull, ce, mix, bidir, grid
// Output: one line per measurement, "name  GB/s" (bytes that crossed A->B per second; for
// bidirectional cases the sum of both directions and the per-direction figure).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#define CK(x)                                                                                              \
    do {                                                                                                   \
        cudaError_t e_ = (x);                                                                              \
        if (e_ != cudaSuccess) {                                                                           \
            std::fprintf(stderr, "%s:%d %s: %s\n", __FILE__, __LINE__, #x, cudaGetErrorString(e_));        \
            std::exit(1);                                                                                  \
        }                                                                                                  \
    } while (0)

namespace {

struct V16 {
    unsigned x, y, z, w;
};
struct V32 {
    float v[8];
};

__device__ __forceinline__ V16 ld16(const void *p) {
    V16 r;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ void st16(void *p, const V16 &r) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w) : "memory");
}
__device__ __forceinline__ V32 ld32(const void *p) {
    V32 r;
    asm volatile("ld.global.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void st32(void *p, const V32 &r) {
    asm volatile("st.global.L1::no_allocate.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]),
                 "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]), "f"(r.v[7])
                 : "memory");
}

// Grid-stride copy: every CTA owns contiguous `chunk`-byte pieces (piece = blockIdx + k * grid),
// each thread keeps UNROLL vectors in flight.  The same kernel pushes (dst is the peer) or pulls
// (src is the peer); it only depends on which GPU launches it.
template<int VEC, int UNROLL> __global__ void __launch_bounds__(512) copyKernel(const char *__restrict__ src, char *__restrict__ dst, size_t bytes, size_t chunk) {
    const size_t pieces = (bytes + chunk - 1) / chunk;
    for (size_t pc = blockIdx.x; pc < pieces; pc += gridDim.x) {
        const size_t base = pc * chunk;
        const size_t n = (bytes - base < chunk ? bytes - base : chunk) / VEC;
        const char *s = src + base;
        char *d = dst + base;
        size_t i = threadIdx.x;
        for (; i + (UNROLL - 1) * blockDim.x < n; i += UNROLL * blockDim.x) {
            if constexpr (VEC == 16) {
                V16 v[UNROLL];
#pragma unroll
                for (int k = 0; k < UNROLL; ++k) v[k] = ld16(s + (i + k * blockDim.x) * 16);
#pragma unroll
                for (int k = 0; k < UNROLL; ++k) st16(d + (i + k * blockDim.x) * 16, v[k]);
            } else {
                V32 v[UNROLL];
#pragma unroll
                for (int k = 0; k < UNROLL; ++k) v[k] = ld32(s + (i + k * blockDim.x) * 32);
#pragma unroll
                for (int k = 0; k < UNROLL; ++k) st32(d + (i + k * blockDim.x) * 32, v[k]);
            }
        }
        for (; i < n; i += blockDim.x) {
            if constexpr (VEC == 16) st16(d + i * 16, ld16(s + i * 16));
            else st32(d + i * 32, ld32(s + i * 32));
        }
    }
}

struct Side {
    int dev;
    char *src;  // local source
    char *dst;  // local landing zone (written by the other side's push, or by this side's pull)
    cudaStream_t s0, s1;
};

enum Kind { PUSH16, PUSH32, PULL16, PULL32, CE_SRC, CE_DST };

struct Op {
    Kind kind;
    size_t off, bytes; // slice of the buffer this op moves
    int grid, threads, unroll;
    size_t chunk;
    int streamSel;     // 0 / 1: which stream of the launching side
};

void launchCopy(int vec, int unroll, int grid, int threads, cudaStream_t st, const char *s, char *d, size_t bytes, size_t chunk) {
    if (vec == 16) {
        if (unroll == 8) copyKernel<16, 8><<<grid, threads, 0, st>>>(s, d, bytes, chunk);
        else copyKernel<16, 4><<<grid, threads, 0, st>>>(s, d, bytes, chunk);
    } else {
        if (unroll == 8) copyKernel<32, 8><<<grid, threads, 0, st>>>(s, d, bytes, chunk);
        else if (unroll == 2) copyKernel<32, 2><<<grid, threads, 0, st>>>(s, d, bytes, chunk);
        else copyKernel<32, 4><<<grid, threads, 0, st>>>(s, d, bytes, chunk);
    }
    CK(cudaGetLastError());
}

// Moves from.src -> to.dst with the given method.
void issue(const Op &op, const Side &from, const Side &to) {
    const char *s = from.src + op.off;
    char *d = to.dst + op.off;
    switch (op.kind) {
    case PUSH16:
    case PUSH32:
        CK(cudaSetDevice(from.dev));
        launchCopy(op.kind == PUSH16 ? 16 : 32, op.unroll, op.grid, op.threads, op.streamSel ? from.s1 : from.s0, s, d, op.bytes, op.chunk);
        break;
    case PULL16:
    case PULL32:
        CK(cudaSetDevice(to.dev));
        launchCopy(op.kind == PULL16 ? 16 : 32, op.unroll, op.grid, op.threads, op.streamSel ? to.s1 : to.s0, s, d, op.bytes, op.chunk);
        break;
    case CE_SRC:
        CK(cudaSetDevice(from.dev));
        CK(cudaMemcpyAsync(d, s, op.bytes, cudaMemcpyDeviceToDevice, op.streamSel ? from.s1 : from.s0));
        break;
    case CE_DST:
        CK(cudaSetDevice(to.dev));
        CK(cudaMemcpyAsync(d, s, op.bytes, cudaMemcpyDeviceToDevice, op.streamSel ? to.s1 : to.s0));
        break;
    }
}

void syncBoth(const Side &a, const Side &b) {
    CK(cudaSetDevice(a.dev));
    CK(cudaDeviceSynchronize());
    CK(cudaSetDevice(b.dev));
    CK(cudaDeviceSynchronize());
}

// Runs `ab` (A -> B) and `ba` (B -> A) op lists `iters` times; device time between an event
// recorded on every used stream before and after (max of the stream times).
double run(const char *name, const std::vector<Op> &ab, const std::vector<Op> &ba, Side &a, Side &b, int iters, size_t bytes_ab, size_t bytes_ba) {
    struct Ev {
        int dev;
        cudaStream_t st;
        cudaEvent_t e0, e1;
    };
    std::vector<Ev> evs;
    auto add = [&](int dev, cudaStream_t st) {
        for (auto &e : evs)
            if (e.st == st) return;
        Ev e{dev, st, nullptr, nullptr};
        CK(cudaSetDevice(dev));
        CK(cudaEventCreate(&e.e0));
        CK(cudaEventCreate(&e.e1));
        evs.push_back(e);
    };
    auto streamOf = [&](const Op &op, const Side &from, const Side &to) {
        const bool on_src = op.kind == PUSH16 || op.kind == PUSH32 || op.kind == CE_SRC;
        const Side &sd = on_src ? from : to;
        add(sd.dev, op.streamSel ? sd.s1 : sd.s0);
    };
    for (auto &op : ab) streamOf(op, a, b);
    for (auto &op : ba) streamOf(op, b, a);
    // warm-up
    for (int w = 0; w < 2; ++w) {
        for (auto &op : ab) issue(op, a, b);
        for (auto &op : ba) issue(op, b, a);
    }
    syncBoth(a, b);
    const auto w0 = std::chrono::steady_clock::now();
    for (auto &e : evs) {
        CK(cudaSetDevice(e.dev));
        CK(cudaEventRecord(e.e0, e.st));
    }
    for (int it = 0; it < iters; ++it) {
        for (auto &op : ab) issue(op, a, b);
        for (auto &op : ba) issue(op, b, a);
    }
    for (auto &e : evs) {
        CK(cudaSetDevice(e.dev));
        CK(cudaEventRecord(e.e1, e.st));
    }
    syncBoth(a, b);
    const double wall_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - w0).count();
    float worst = 0;
    for (auto &e : evs) {
        float ms = 0;
        CK(cudaSetDevice(e.dev));
        CK(cudaEventElapsedTime(&ms, e.e0, e.e1));
        worst = ms > worst ? ms : worst;
        cudaEventDestroy(e.e0);
        cudaEventDestroy(e.e1);
    }
    const double total = double(bytes_ab + bytes_ba) * iters / (worst * 1e-3) / 1e9;
    // Events of different streams start their clocks when each stream starts: with several streams the
    // host's wall clock (issue + completion of everything) is the honest total.
    const double wall = double(bytes_ab + bytes_ba) * iters / (wall_ms * 1e-3) / 1e9;
    if (bytes_ba) std::printf("%-44s %8.1f GB/s both ways (%7.1f per direction)  %.3f ms/iter  [wall clock %.1f GB/s]\n", name, total, total / 2, worst / iters, wall);
    else std::printf("%-44s %8.1f GB/s  %.3f ms/iter  [wall clock %.1f GB/s]\n", name, total, worst / iters, wall);
    std::fflush(stdout);
    return total;
}

Op mk(Kind k, size_t off, size_t bytes, int grid = 296, int threads = 512, int unroll = 4, size_t chunk = 256 << 10, int streamSel = 0) {
    return Op{k, off, bytes, grid, threads, unroll, chunk, streamSel};
}

} // namespace

int main(int argc, char **argv) {
    size_t mib = 1024;
    int iters = 10, devA = 0, devB = 1;
    std::string which = "all";
    for (int i = 1; i < argc; ++i) {
        auto next = [&] { return i + 1 < argc ? argv[++i] : (char *)""; };
        if (!std::strcmp(argv[i], "--mib")) mib = std::strtoull(next(), nullptr, 0);
        else if (!std::strcmp(argv[i], "--iters")) iters = std::atoi(next());
        else if (!std::strcmp(argv[i], "--case")) which = next();
        else if (!std::strcmp(argv[i], "--dev-a")) devA = std::atoi(next());
        else if (!std::strcmp(argv[i], "--dev-b")) devB = std::atoi(next());
        else {
            std::fprintf(stderr, "usage: nvlink_probe [--mib N] [--iters K] [--case all|push|pull|ce|mix|bidir|grid] [--dev-a A] [--dev-b B]\n");
            return 2;
        }
    }
    int n = 0;
    CK(cudaGetDeviceCount(&n));
    if (n < 2 || devA >= n || devB >= n || devA == devB) {
        std::printf("nvlink_probe needs two GPUs (found %d)\n", n);
        return 0;
    }
    int can = 0;
    CK(cudaDeviceCanAccessPeer(&can, devA, devB));
    if (!can) {
        std::printf("GPU %d cannot access GPU %d\n", devA, devB);
        return 0;
    }
    const size_t bytes = mib << 20;
    Side a{devA, nullptr, nullptr, nullptr, nullptr}, b{devB, nullptr, nullptr, nullptr, nullptr};
    for (Side *s : {&a, &b}) {
        CK(cudaSetDevice(s->dev));
        CK(cudaDeviceEnablePeerAccess(s == &a ? devB : devA, 0));
        CK(cudaMalloc(&s->src, bytes));
        CK(cudaMalloc(&s->dst, bytes));
        CK(cudaMemset(s->src, s == &a ? 0x5a : 0xa5, bytes));
        CK(cudaMemset(s->dst, 0, bytes));
        CK(cudaStreamCreateWithFlags(&s->s0, cudaStreamNonBlocking));
        CK(cudaStreamCreateWithFlags(&s->s1, cudaStreamNonBlocking));
    }
    syncBoth(a, b);
    const bool all = which == "all";
    std::printf("# nvlink_probe: GPU %d <-> GPU %d, %zu MiB per direction, %d iterations\n", devA, devB, mib, iters);

    if (all || which == "push") {
        run("push  16B x4, 296 CTAs, 256K chunks", {mk(PUSH16, 0, bytes)}, {}, a, b, iters, bytes, 0);
        run("push  32B x4, 296 CTAs, 256K chunks", {mk(PUSH32, 0, bytes)}, {}, a, b, iters, bytes, 0);
        run("push  32B x8, 296 CTAs, 256K chunks", {mk(PUSH32, 0, bytes, 296, 512, 8)}, {}, a, b, iters, bytes, 0);
        run("push  32B x2, 592 CTAs x 256 thr", {mk(PUSH32, 0, bytes, 592, 256, 2)}, {}, a, b, iters, bytes, 0);
        run("push  32B x4, 2368 CTAs, 64K chunks", {mk(PUSH32, 0, bytes, 2368, 512, 4, 64 << 10)}, {}, a, b, iters, bytes, 0);
    }
    if (all || which == "pull") {
        run("pull  16B x4, 296 CTAs", {mk(PULL16, 0, bytes)}, {}, a, b, iters, bytes, 0);
        run("pull  32B x4, 296 CTAs", {mk(PULL32, 0, bytes)}, {}, a, b, iters, bytes, 0);
        run("pull  32B x8, 296 CTAs", {mk(PULL32, 0, bytes, 296, 512, 8)}, {}, a, b, iters, bytes, 0);
        run("pull  32B x8, 592 CTAs", {mk(PULL32, 0, bytes, 592, 512, 8)}, {}, a, b, iters, bytes, 0);
    }
    if (all || which == "ce") {
        run("copy engine, issued on the source GPU", {mk(CE_SRC, 0, bytes)}, {}, a, b, iters, bytes, 0);
        run("copy engine, issued on the destination GPU", {mk(CE_DST, 0, bytes)}, {}, a, b, iters, bytes, 0);
        run("copy engine x2 streams (halves), source GPU", {mk(CE_SRC, 0, bytes / 2), mk(CE_SRC, bytes / 2, bytes / 2, 296, 512, 4, 256 << 10, 1)}, {}, a, b, iters, bytes, 0);
        // The engine's shape: a request of 16 descriptors, one copy each.
        std::vector<Op> one, two, one_dst;
        for (int i = 0; i < 16; ++i) {
            one.push_back(mk(CE_SRC, bytes / 16 * i, bytes / 16));
            one_dst.push_back(mk(CE_DST, bytes / 16 * i, bytes / 16));
            two.push_back(mk(CE_SRC, bytes / 16 * i, bytes / 16, 296, 512, 4, 256 << 10, i & 1));
        }
        run("copy engine, 16 copies on one stream", one, {}, a, b, iters, bytes, 0);
        run("copy engine, 16 copies alternating 2 streams", two, {}, a, b, iters, bytes, 0);
        run("bidir copy engine, 16 copies on one stream", one, one, a, b, iters, bytes, bytes);
        run("bidir copy engine, 16 copies, 2 streams", two, two, a, b, iters, bytes, bytes);
        run("bidir copy engine, 16 copies, destination side", one_dst, one_dst, a, b, iters, bytes, bytes);
        run("bidir copy engine, 1 copy each way", {mk(CE_SRC, 0, bytes)}, {mk(CE_SRC, 0, bytes)}, a, b, iters, bytes, bytes);
        run("bidir push 32B (for comparison)", {mk(PUSH32, 0, bytes)}, {mk(PUSH32, 0, bytes)}, a, b, iters, bytes, bytes);
    }
    if (all || which == "grid") {
        for (int g : {32, 64, 96, 148, 296, 592}) {
            char nm[96];
            std::snprintf(nm, sizeof(nm), "push  32B x4, %d CTAs", g);
            run(nm, {mk(PUSH32, 0, bytes, g)}, {}, a, b, iters, bytes, 0);
        }
        for (int g : {32, 64, 96, 148, 296}) {
            char nm[96];
            std::snprintf(nm, sizeof(nm), "pull  32B x8, %d CTAs", g);
            run(nm, {mk(PULL32, 0, bytes, g, 512, 8)}, {}, a, b, iters, bytes, 0);
        }
    }
    if (all || which == "mix") {
        // One direction, two mechanisms side by side on disjoint halves / slices.
        for (int pct : {50, 70, 85}) {
            const size_t cut = (bytes / 100 * pct) & ~size_t(0xfffff);
            char nm[96];
            std::snprintf(nm, sizeof(nm), "push %d%% + pull %d%% (same direction)", pct, 100 - pct);
            run(nm, {mk(PUSH32, 0, cut), mk(PULL32, cut, bytes - cut, 148, 512, 8)}, {}, a, b, iters, bytes, 0);
            std::snprintf(nm, sizeof(nm), "push %d%% + copy engine %d%%", pct, 100 - pct);
            run(nm, {mk(PUSH32, 0, cut), mk(CE_SRC, cut, bytes - cut, 296, 512, 4, 256 << 10, 1)}, {}, a, b, iters, bytes, 0);
        }
        run("pull 50% + copy engine 50%", {mk(PULL32, 0, bytes / 2, 296, 512, 8), mk(CE_SRC, bytes / 2, bytes / 2, 296, 512, 4, 256 << 10, 1)}, {}, a, b, iters, bytes, 0);
    }
    if (all || which == "bidir") {
        run("bidir push 32B", {mk(PUSH32, 0, bytes)}, {mk(PUSH32, 0, bytes)}, a, b, iters, bytes, bytes);
        run("bidir push 16B", {mk(PUSH16, 0, bytes)}, {mk(PUSH16, 0, bytes)}, a, b, iters, bytes, bytes);
        run("bidir pull 32B x8", {mk(PULL32, 0, bytes, 296, 512, 8)}, {mk(PULL32, 0, bytes, 296, 512, 8)}, a, b, iters, bytes, bytes);
        run("bidir copy engine (source side)", {mk(CE_SRC, 0, bytes)}, {mk(CE_SRC, 0, bytes)}, a, b, iters, bytes, bytes);
        run("bidir copy engine (destination side)", {mk(CE_DST, 0, bytes)}, {mk(CE_DST, 0, bytes)}, a, b, iters, bytes, bytes);
        const size_t cut = (bytes / 100 * 70) & ~size_t(0xfffff);
        run("bidir push 70% + pull 30%", {mk(PUSH32, 0, cut), mk(PULL32, cut, bytes - cut, 148, 512, 8)},
            {mk(PUSH32, 0, cut), mk(PULL32, cut, bytes - cut, 148, 512, 8)}, a, b, iters, bytes, bytes);
        run("bidir push 70% + copy engine 30%", {mk(PUSH32, 0, cut), mk(CE_SRC, cut, bytes - cut, 296, 512, 4, 256 << 10, 1)},
            {mk(PUSH32, 0, cut), mk(CE_SRC, cut, bytes - cut, 296, 512, 4, 256 << 10, 1)}, a, b, iters, bytes, bytes);
    }
    // The bytes must have arrived: spot-check the landing zones.
    unsigned char probe[2] = {0, 0};
    CK(cudaSetDevice(b.dev));
    CK(cudaMemcpy(&probe[0], b.dst + bytes / 3, 1, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(&probe[1], b.dst + bytes - 1, 1, cudaMemcpyDeviceToHost));
    std::printf("# landing zone on GPU %d holds 0x%02x 0x%02x (expected 0x5a)\n", b.dev, probe[0], probe[1]);
    return (probe[0] == 0x5a && probe[1] == 0x5a) ? 0 : 1;
}

// Expert-parallel dispatch / combine and a fused KV-cache transfer driven from C++ (include/nixl_ep.h).
//
// One rank per GPU (up to four), all in this process; with one GPU a single rank talks to itself.
// Every rank dispatches its tokens (bf16, no quantisation) in throughput mode with the top-k weights,
// the "experts" are the identity (each rank copies what it received into its combine input), and the
// rank-reduced combine must hand every token back multiplied by the sum of its weights.  Then rank 0
// moves a small paged KV cache to the last rank with a head reshard, checked on the host.
//
//   make -C csrc -j8          builds nixl_b200/bin/ep_native_example from this file
//   NIXL_PLUGIN_DIR=nixl_b200/lib/plugins nixl_b200/bin/ep_native_example
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <random>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "nixl_ep.h"

#define REQUIRE(cond, what)                                       \
    do {                                                          \
        if (!(cond)) {                                            \
            std::fprintf(stderr, "FAILED: %s (%s)\n", what, #cond); \
            return 1;                                             \
        }                                                         \
    } while (0)

namespace {
float bf16ToFloat(uint16_t v) {
    uint32_t u = static_cast<uint32_t>(v) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
uint16_t floatToBf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u += 0x7fffu + ((u >> 16) & 1u); // round to nearest even
    return static_cast<uint16_t>(u >> 16);
}
} // namespace

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        std::printf("no GPU: nothing to show\n");
        return 0;
    }
    const int R = std::min(ndev, 4), El = 4, E = El * R, H = 1024, T = 64, K = 4;
    struct Rank {
        int dev;
        std::unique_ptr<nixlAgent> agent;
        std::unique_ptr<nixlEpBuffer> buf;
        void *x = nullptr, *out = nullptr;
        int64_t *idx = nullptr;
        float *w = nullptr;
        std::vector<uint16_t> hx;
        std::vector<int64_t> hidx;
        std::vector<float> hw;
        nixlEpHandle handle;
    };
    std::vector<Rank> ranks(R);
    std::mt19937 gen(7);
    std::normal_distribution<float> normal(0.f, 1.f);
    for (int r = 0; r < R; ++r) {
        Rank &k = ranks[r];
        k.dev = r % ndev;
        cudaSetDevice(k.dev);
        const std::string name = "ep_rank" + std::to_string(r);
        k.agent = std::make_unique<nixlAgent>(name, nixlAgentConfig(false));
        nixlBackendH *b = nullptr;
        REQUIRE(k.agent->createBackend("NVLINK", {}, b) == NIXL_SUCCESS, "NVLINK backend (is NIXL_PLUGIN_DIR set?)");
        nixlEpConfig cfg;
        cfg.agentName = name;
        cfg.rank = r;
        cfg.numRanks = R;
        cfg.numExperts = E;
        cfg.hidden = H;
        cfg.maxTokens = T;
        cfg.topk = K;
        cfg.device = k.dev;
        cfg.lowLatencyMode = false;
        cfg.timeoutMs = 20000;
        k.buf = std::make_unique<nixlEpBuffer>(*k.agent, cfg);
        REQUIRE(k.buf->ok(), "buffer construction");
        // inputs: tokens N(0,1); K distinct experts per token; weights that sum to about one
        k.hx.resize(size_t(T) * H);
        for (auto &v : k.hx) v = floatToBf16(normal(gen));
        k.hidx.resize(size_t(T) * K);
        k.hw.resize(size_t(T) * K);
        for (int t = 0; t < T; ++t) {
            std::vector<int> all(E);
            for (int e = 0; e < E; ++e) all[e] = e;
            std::shuffle(all.begin(), all.end(), gen);
            float sum = 0;
            for (int j = 0; j < K; ++j) {
                k.hidx[size_t(t) * K + j] = all[j];
                k.hw[size_t(t) * K + j] = 0.1f + std::fabs(normal(gen));
                sum += k.hw[size_t(t) * K + j];
            }
            for (int j = 0; j < K; ++j) k.hw[size_t(t) * K + j] /= sum * (1.f + 0.25f * (t % 3)); // not all sums equal
        }
        k.hidx[K - 1] = -1; // an unused slot must be skipped
        cudaMalloc(&k.x, k.hx.size() * 2);
        cudaMalloc(&k.out, k.hx.size() * 2);
        cudaMalloc(reinterpret_cast<void **>(&k.idx), k.hidx.size() * 8);
        cudaMalloc(reinterpret_cast<void **>(&k.w), k.hw.size() * 4);
        cudaMemcpy(k.x, k.hx.data(), k.hx.size() * 2, cudaMemcpyHostToDevice);
        cudaMemcpy(k.idx, k.hidx.data(), k.hidx.size() * 8, cudaMemcpyHostToDevice);
        cudaMemcpy(k.w, k.hw.data(), k.hw.size() * 4, cudaMemcpyHostToDevice);
    }
    std::vector<std::string> blobs(R);
    for (int r = 0; r < R; ++r) REQUIRE(ranks[r].buf->localMetadata(blobs[r]) == NIXL_SUCCESS, "metadata");
    for (int r = 0; r < R; ++r) REQUIRE(ranks[r].buf->connectRanks(blobs) == NIXL_SUCCESS, "connectRanks");

    for (int step = 0; step < 3; ++step) {
        // every rank launches before anyone waits: the kernels of different ranks wait for each other
        for (auto &k : ranks) {
            cudaSetDevice(k.dev);
            REQUIRE(k.buf->dispatch(k.x, k.idx, T, /*fp8=*/false, k.w, nullptr, k.handle) == NIXL_SUCCESS, "dispatch");
        }
        for (auto &k : ranks) {
            cudaSetDevice(k.dev);
            REQUIRE(cudaDeviceSynchronize() == cudaSuccess, "dispatch ran");
            REQUIRE(k.buf->status() == 0, "dispatch status");
            // identity experts: what arrived goes back
            cudaMemcpy(k.buf->combineInput(k.handle), k.handle.recvX, size_t(k.handle.rows) * H * 2, cudaMemcpyDeviceToDevice);
        }
        for (auto &k : ranks) {
            cudaSetDevice(k.dev);
            REQUIRE(k.buf->combine(k.buf->combineInput(k.handle), k.idx, k.w, k.handle, k.out, T, nullptr) == NIXL_SUCCESS, "combine");
        }
        for (auto &k : ranks) {
            cudaSetDevice(k.dev);
            REQUIRE(cudaDeviceSynchronize() == cudaSuccess, "combine ran");
            REQUIRE(k.buf->status() == 0, "combine status");
            std::vector<uint16_t> got(k.hx.size());
            cudaMemcpy(got.data(), k.out, got.size() * 2, cudaMemcpyDeviceToHost);
            double worst = 0;
            for (int t = 0; t < T; ++t) {
                float sum = 0;
                for (int j = 0; j < K; ++j)
                    if (k.hidx[size_t(t) * K + j] >= 0) sum += k.hw[size_t(t) * K + j];
                for (int c = 0; c < H; ++c) {
                    const float want = bf16ToFloat(k.hx[size_t(t) * H + c]) * sum;
                    const double err = std::fabs(bf16ToFloat(got[size_t(t) * H + c]) - want);
                    worst = std::max(worst, err - 0.02 * std::fabs(want));
                }
            }
            REQUIRE(worst <= 0.02, "combined tokens equal the tokens times their weight sums");
        }
    }
    std::printf("expert parallelism: %d rank(s) x %d tokens, top-%d of %d experts, 3 steps: combined output as expected\n", R, T, K, E);

    // ------------------------------------------------------------------ fused KV transfer, rank 0 -> last rank
    {
        Rank &src = ranks[0], &dst = ranks[R - 1];
        const int blocks = 24, tokens = 16, srcHeads = 2, dstHeads = 4, dim = 128, tensors = 3;
        const size_t srcElems = size_t(blocks) * tokens * srcHeads * dim, dstElems = size_t(blocks) * tokens * dstHeads * dim;
        std::vector<std::vector<uint16_t>> hsrc(tensors, std::vector<uint16_t>(srcElems));
        std::vector<void *> dsrc(tensors), ddst(tensors);
        nixl_reg_dlist_t regS(VRAM_SEG), regD(VRAM_SEG);
        std::vector<nixlBasicDesc> srcDescs, dstDescs;
        for (int t = 0; t < tensors; ++t) {
            for (auto &v : hsrc[t]) v = floatToBf16(normal(gen));
            cudaSetDevice(src.dev);
            cudaMalloc(&dsrc[t], srcElems * 2);
            cudaMemcpy(dsrc[t], hsrc[t].data(), srcElems * 2, cudaMemcpyHostToDevice);
            cudaSetDevice(dst.dev);
            cudaMalloc(&ddst[t], dstElems * 2);
            cudaMemset(ddst[t], 0, dstElems * 2);
            regS.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dsrc[t]), srcElems * 2, src.dev, ""));
            regD.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(ddst[t]), dstElems * 2, dst.dev, ""));
            srcDescs.emplace_back(reinterpret_cast<uintptr_t>(dsrc[t]), srcElems * 2, src.dev);
            dstDescs.emplace_back(reinterpret_cast<uintptr_t>(ddst[t]), dstElems * 2, dst.dev);
        }
        REQUIRE(src.agent->registerMem(regS) == NIXL_SUCCESS && dst.agent->registerMem(regD) == NIXL_SUCCESS, "KV registration");
        std::string dstName = "ep_rank" + std::to_string(R - 1);
        if (R > 1) { // the sender needs the receiver's new registrations
            nixl_blob_t md;
            dst.agent->getLocalMD(md);
            REQUIRE(src.agent->loadRemoteMD(md, dstName) == NIXL_SUCCESS, "KV metadata");
        }
        std::vector<int32_t> sb(blocks), db(blocks);
        for (int i = 0; i < blocks; ++i) sb[i] = i, db[i] = blocks - 1 - i;
        std::shuffle(sb.begin(), sb.end(), gen);
        cudaSetDevice(src.dev);
        int32_t *dsb = nullptr, *ddb = nullptr;
        cudaMalloc(reinterpret_cast<void **>(&dsb), blocks * 4);
        cudaMalloc(reinterpret_cast<void **>(&ddb), blocks * 4);
        cudaMemcpy(dsb, sb.data(), blocks * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(ddb, db.data(), blocks * 4, cudaMemcpyHostToDevice);
        {
            nixlKvTransfer xfer(*src.agent, srcDescs, nixlKvLayout{tokens, srcHeads, dim, false, 2}, dstName, dstDescs,
                                nixlKvLayout{tokens, dstHeads, dim, false, 2}, /*dstHeadOffset=*/2, /*castFp8=*/false);
            REQUIRE(xfer.ok(), "KV path");
            uint64_t ticket = 0;
            REQUIRE(xfer.post(dsb, ddb, blocks, nullptr, ticket) == NIXL_SUCCESS, "KV post");
            REQUIRE(xfer.wait(ticket) == NIXL_SUCCESS, "KV completion");
        }
        cudaSetDevice(dst.dev);
        cudaDeviceSynchronize();
        for (int t = 0; t < tensors; ++t) {
            std::vector<uint16_t> got(dstElems);
            cudaMemcpy(got.data(), ddst[t], dstElems * 2, cudaMemcpyDeviceToHost);
            for (int i = 0; i < blocks; ++i)
                for (int tok = 0; tok < tokens; ++tok)
                    for (int h = 0; h < dstHeads; ++h)
                        for (int c = 0; c < dim; ++c) {
                            const uint16_t g = got[((size_t(db[i]) * tokens + tok) * dstHeads + h) * dim + c];
                            const uint16_t want = h >= 2 ? hsrc[t][((size_t(sb[i]) * tokens + tok) * srcHeads + (h - 2)) * dim + c] : 0;
                            REQUIRE(g == want, "KV bytes at the receiver");
                        }
        }
        std::printf("KV transfer: %d tensors x %d blocks, 2 heads into head slots 2..3 of 4: bytes as expected\n", tensors, blocks);
        src.agent->deregisterMem(regS);
        dst.agent->deregisterMem(regD);
    }
    for (auto &k : ranks) {
        cudaSetDevice(k.dev);
        k.buf.reset();
    }
    return 0;
}

// Native host side of the fused paths: expert-parallel dispatch / combine and the paged KV-cache
// transfer, for serving engines written in C++.
//
// nixlEpBuffer plays the part of the reference's C++ `nixl_ep::Buffer`
// (examples/device/ep/csrc/nixl_ep.cpp: init :109, connect_ranks :463, dispatch :1031, combine
// :1146): one rank's symmetric communication buffer, registered with a nixlAgent, peers reached
// through a remote memory view, kernels from libnixl_kernels.so.  The layout of the buffer, the
// step counters and the launch parameters are the same as in the Python class
// nixl_b200.parallel.Buffer, so ranks driven from C++ and from Python can sit in one group.
//
// nixlKvTransfer is the prepared prefill -> decode path of the fused KV kernel
// (nixl_b200.ops.KVTransfer in Python).
//
// Everything here is host code; it links against libnixl, libnixl_kernels and the CUDA runtime.
#ifndef NIXL_B200_NIXL_EP_H
#define NIXL_B200_NIXL_EP_H

#include <cstdint>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "kernels/nixl_kernels.h"
#include "nixl.h"

struct nixlEpConfig {
    std::string agentName;     // name of the agent the buffer is built on (its own entry of the peer table carries it)
    int rank = 0, numRanks = 1;
    int numExperts = 0;        // global, divisible by numRanks
    int hidden = 0;            // multiple of 512
    int maxTokens = 0;         // upper bound of tokens a rank dispatches per call
    int topk = 0;
    int device = -1;           // CUDA device of this rank (-1: current)
    bool lowLatencyMode = true; // also size the buffer for the [local experts, ranks * maxTokens, hidden] layout
    long long compactRows = -1; // capacity of the throughput layout (-1: worst case)
    uint64_t timeoutMs = 30000; // bound of every in-kernel wait on a peer
};

// What a dispatch returns and the matching combine needs.  Pointers are device memory that
// belongs to the buffer; they stay valid until the dispatch after next.
struct nixlEpHandle {
    int parity = 0;
    uint64_t epoch = 0;
    int rowsPerExpert = 0;        // > 0: low-latency layout
    bool hasGroupRecords = false; // the dispatch was given weights: combine may reduce per rank
    void *recvX = nullptr;        // [rows][hidden] e4m3 or bf16
    float *recvScales = nullptr;  // [rows][hidden / 128] (fp8 only)
    long long rows = 0;           // capacity of recvX in rows
    int32_t *recvCount = nullptr;     // [local experts]
    int32_t *expertOffsets = nullptr; // [local experts + 1]
    int64_t *layoutRange = nullptr;   // [local experts][ranks]
    const uint32_t *srcInfo = nullptr; // [rows][2] {source rank, token * topk + k}
    int32_t *sendRow = nullptr;       // [maxTokens][topk]
};

enum class nixlEpCombineMode : int { AUTO = -1, PUSH = 0, PULL = 1, RANK_REDUCE = 2 };

class nixlEpBuffer {
public:
    // The agent must have the NVLINK backend and outlive the buffer.
    nixlEpBuffer(nixlAgent &agent, const nixlEpConfig &cfg);
    ~nixlEpBuffer();
    nixlEpBuffer(const nixlEpBuffer &) = delete;
    nixlEpBuffer &operator=(const nixlEpBuffer &) = delete;
    bool ok() const { return ok_; } // construction succeeded

    // What a peer needs to reach this rank (agent metadata, buffer descriptor, step counters).
    nixl_status_t localMetadata(std::string &blob) const;
    // Connects to the ranks whose metadata blobs are given (all ranks' blobs, in any order; this
    // rank's own may be among them).  Between steps only.
    nixl_status_t connectRanks(const std::vector<std::string> &blobs);
    nixl_status_t disconnectRanks(const std::vector<int> &ranks);

    // Throughput mode: compact layout.  x bf16 [tokens][hidden], topkIdx int64 [tokens][topk] (-1 = unused),
    // weights float [tokens][topk] or nullptr (given: the combine that follows may be rank-reduced).
    nixl_status_t dispatch(const void *x, const int64_t *topkIdx, int tokens, bool fp8, const float *weights, cudaStream_t stream,
                           nixlEpHandle &out);
    // Low-latency mode: expert-major layout [local experts][ranks * maxTokens][hidden].
    nixl_status_t lowLatencyDispatch(const void *x, const int64_t *topkIdx, int tokens, bool fp8, cudaStream_t stream, nixlEpHandle &out);
    // out[t] = sum_k weights[t][k] * y[row of (t, k)]; y bf16 in the row order the dispatch delivered.
    nixl_status_t combine(const void *y, const int64_t *topkIdx, const float *weights, const nixlEpHandle &h, void *out, int tokens,
                          cudaStream_t stream, nixlEpCombineMode mode = nixlEpCombineMode::AUTO);
    // The region pull-mode combine reads from (an expert GEMM that writes here makes combine copy-free).
    void *combineInput(const nixlEpHandle &h) const;

    nixl_status_t barrier(cudaStream_t stream);
    int status() const;                  // bit 0: a peer timed out, bit 1: a grid barrier timed out, bit 2: capacity exceeded
    std::vector<int> queryMask() const;  // non-zero: rank excluded
    void updateMask(int rank, bool masked);
    void cleanMask();
    uint64_t epoch() const { return epoch_; }
    int localExperts() const { return cfg_.numExperts / cfg_.numRanks; }
    const nixlEpConfig &config() const { return cfg_; }

private:
    NixlEpLayout layout(int parity) const;
    NixlEpScratch scratch() const;
    nixl_status_t rebuildView();
    nixl_status_t doDispatch(const void *x, const int64_t *topkIdx, int tokens, bool fp8, const float *weights, int rowsPerExpert,
                             cudaStream_t stream, nixlEpHandle &out);

    nixlAgent &agent_;
    nixlEpConfig cfg_;
    bool ok_ = false;
    long long llRows_ = 0, compactRows_ = 0, cap_ = 0;
    int64_t half_ = 0, barrierOff_ = 0, total_ = 0;
    NixlEpLayout lay_{}; // offsets of parity half 0
    char *buffer_ = nullptr;
    int32_t *cnt_ = nullptr;      // [3 * E]
    uint32_t *bar_ = nullptr;     // [4]
    int32_t *status_ = nullptr;   // [1]
    int32_t *mask_ = nullptr;     // [R]
    // per parity: outputs of the dispatch
    int32_t *recvCount_[2] = {nullptr, nullptr}, *expertOffsets_[2] = {nullptr, nullptr}, *sendRow_[2] = {nullptr, nullptr};
    int64_t *layoutRange_[2] = {nullptr, nullptr};
    nixlMemViewH peersView_ = nullptr;
    uint64_t epoch_ = 0, barrierEpoch_ = 0;
    struct Peer {
        std::string agent;
        uintptr_t addr = 0;
        size_t len = 0;
        int dev = 0;
        bool connected = false;
    };
    std::vector<Peer> peers_;
    bool registered_ = false;
};

// ------------------------------------------------------------------------------------------------ KV transfer

struct nixlKvLayout { // one cache tensor: [blocks][tokens][heads][headDim] ("NHD") or [blocks][heads][tokens][headDim] ("HND")
    int tokens = 0, heads = 0, headDim = 0;
    bool hnd = false;
    int elemBytes = 2; // 2: bf16, 1: fp8 e4m3
};

class nixlKvTransfer {
public:
    // srcTensors: this (sending) rank's registered cache tensors, one per (layer, K/V); dstTensors: the receiver's
    // registered tensors in the same order (addresses in the receiver's process), reached through `remoteAgent`.
    nixlKvTransfer(nixlAgent &agent, const std::vector<nixlBasicDesc> &srcTensors, const nixlKvLayout &srcLayout, const std::string &remoteAgent,
                   const std::vector<nixlBasicDesc> &dstTensors, const nixlKvLayout &dstLayout, int dstHeadOffset, bool castFp8, float scale = 1.f);
    ~nixlKvTransfer();
    nixlKvTransfer(const nixlKvTransfer &) = delete;
    nixlKvTransfer &operator=(const nixlKvTransfer &) = delete;
    bool ok() const { return ok_; }

    // Moves the block pairs (srcBlocks[i] -> dstBlocks[i], int32 device arrays on the sender's GPU) of every tensor in
    // one launch.  doneSignal: optional 64-bit counter in the receiver's registered memory (a device-visible peer
    // address), incremented by doneValue when everything landed.  Returns a ticket for done() / wait().
    nixl_status_t post(const int32_t *srcBlocks, const int32_t *dstBlocks, int pairs, cudaStream_t stream, uint64_t &ticket,
                       uint64_t *doneSignal = nullptr, uint64_t doneValue = 1);
    bool done(uint64_t ticket) const;
    nixl_status_t wait(uint64_t ticket, double timeoutSeconds = 30.0) const;

private:
    nixlAgent &agent_;
    bool ok_ = false;
    NixlKvXferParams p_{};
    nixlMemViewH srcView_ = nullptr, dstView_ = nullptr;
    uint32_t *counter_ = nullptr; // device
    uint64_t *flag_ = nullptr;    // pinned
    uint64_t seq_ = 0;
    int device_ = 0;
};

#endif

#include "nixl_ep.h"

#include <algorithm>
#include <chrono>
#include <cstring>

#include "serdes/serdes.h"
#include "utils/log.h"

namespace {

constexpr int64_t kAlign = 256;
int64_t up(int64_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

class DeviceGuard {
public:
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev_) != cudaSuccess) prev_ = -1;
        if (dev >= 0 && dev != prev_) {
            cudaSetDevice(dev);
            changed_ = true;
        }
    }
    ~DeviceGuard() {
        if (changed_ && prev_ >= 0) cudaSetDevice(prev_);
    }

private:
    int prev_ = -1;
    bool changed_ = false;
};

template<class T> bool devAlloc(T *&p, size_t count, bool zero = true) {
    void *v = nullptr;
    if (cudaMalloc(&v, count * sizeof(T)) != cudaSuccess) return false;
    if (zero && cudaMemset(v, 0, count * sizeof(T)) != cudaSuccess) {
        cudaFree(v);
        return false;
    }
    p = static_cast<T *>(v);
    return true;
}

} // namespace

// ================================================================================================ nixlEpBuffer

nixlEpBuffer::nixlEpBuffer(nixlAgent &agent, const nixlEpConfig &cfg) : agent_(agent), cfg_(cfg) {
    if (cfg_.numRanks <= 0 || cfg_.rank < 0 || cfg_.rank >= cfg_.numRanks || cfg_.numExperts <= 0 || cfg_.numExperts % cfg_.numRanks ||
        cfg_.agentName.empty() || cfg_.hidden <= 0 || cfg_.hidden % 512 || cfg_.maxTokens <= 0 || cfg_.topk <= 0 || cfg_.topk > 16) {
        NIXL_ERROR << "nixlEpBuffer: invalid shapes";
        return;
    }
    if (cfg_.device < 0 && cudaGetDevice(&cfg_.device) != cudaSuccess) return;
    DeviceGuard dg(cfg_.device);
    const int64_t R = cfg_.numRanks, E = cfg_.numExperts, El = E / R, H = cfg_.hidden, M = cfg_.maxTokens, K = cfg_.topk;
    llRows_ = El * R * M;
    compactRows_ = cfg_.compactRows >= 0 ? cfg_.compactRows : R * M * std::min<int64_t>(K, El);
    cap_ = cfg_.lowLatencyMode ? std::max(llRows_, compactRows_) : compactRows_;
    // One parity half; the same regions, in the same order, as nixl_b200.parallel.Buffer lays them out.
    int64_t off = 0;
    auto place = [&](int64_t &field, int64_t size) {
        field = off;
        off = up(off + size);
    };
    place(lay_.off_counts, R * E * 4);
    place(lay_.off_counts_flag, R * 8);
    place(lay_.off_disp_flag, El * R * 8);
    place(lay_.off_comb_flag, R * 8);
    place(lay_.off_recv_info, cap_ * 8);
    place(lay_.off_recv_scales, cap_ * (H / 128) * 4);
    place(lay_.off_recv_x, cap_ * H * 2);
    place(lay_.off_comb_x, M * std::max(K, R) * H * 2);
    place(lay_.off_comb_in, cap_ * H * 2);
    place(lay_.off_grp, R * M * static_cast<int64_t>(sizeof(NixlEpGroupRecord)));
    place(lay_.off_grp_tokens, R * 4);
    half_ = off;
    barrierOff_ = 2 * half_;
    total_ = 2 * half_ + up(R * 8);
    if (!devAlloc(buffer_, static_cast<size_t>(total_)) || !devAlloc(cnt_, static_cast<size_t>(3 * E)) || !devAlloc(bar_, 4) ||
        !devAlloc(status_, 1) || !devAlloc(mask_, static_cast<size_t>(R))) {
        NIXL_ERROR << "nixlEpBuffer: out of device memory (" << total_ << " bytes of symmetric buffer)";
        cudaGetLastError();
        return;
    }
    for (int p = 0; p < 2; ++p)
        if (!devAlloc(recvCount_[p], static_cast<size_t>(El)) || !devAlloc(expertOffsets_[p], static_cast<size_t>(El + 1)) ||
            !devAlloc(layoutRange_[p], static_cast<size_t>(El * R)) || !devAlloc(sendRow_[p], static_cast<size_t>(M * K)))
            return;
    nixl_reg_dlist_t reg(VRAM_SEG);
    reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buffer_), static_cast<size_t>(total_), cfg_.device, ""));
    if (agent_.registerMem(reg) != NIXL_SUCCESS) {
        NIXL_ERROR << "nixlEpBuffer: the agent could not register the communication buffer";
        return;
    }
    registered_ = true;
    peers_.resize(R);
    ok_ = true;
}

nixlEpBuffer::~nixlEpBuffer() {
    DeviceGuard dg(cfg_.device);
    if (peersView_) agent_.releaseMemView(peersView_);
    if (registered_) {
        cudaDeviceSynchronize();
        nixl_reg_dlist_t reg(VRAM_SEG);
        reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buffer_), static_cast<size_t>(total_), cfg_.device, ""));
        agent_.deregisterMem(reg);
    }
    for (void *p : {static_cast<void *>(buffer_), static_cast<void *>(cnt_), static_cast<void *>(bar_), static_cast<void *>(status_),
                    static_cast<void *>(mask_)})
        if (p) cudaFree(p);
    for (int p = 0; p < 2; ++p)
        for (void *q : {static_cast<void *>(recvCount_[p]), static_cast<void *>(expertOffsets_[p]), static_cast<void *>(layoutRange_[p]),
                        static_cast<void *>(sendRow_[p])})
            if (q) cudaFree(q);
}

NixlEpLayout nixlEpBuffer::layout(int parity) const {
    NixlEpLayout l = lay_;
    const int64_t shift = parity ? half_ : 0;
    for (int64_t *f : {&l.off_counts, &l.off_counts_flag, &l.off_disp_flag, &l.off_recv_x, &l.off_recv_scales, &l.off_recv_info, &l.off_comb_x,
                       &l.off_comb_flag, &l.off_comb_in, &l.off_grp, &l.off_grp_tokens})
        *f += shift;
    return l;
}

NixlEpScratch nixlEpBuffer::scratch() const {
    NixlEpScratch s{};
    s.cnt = cnt_;
    s.fill = cnt_ + cfg_.numExperts;
    s.sent = cnt_ + 2 * cfg_.numExperts;
    s.barrier = bar_;
    s.status = status_;
    s.mask = mask_;
    return s;
}

nixl_status_t nixlEpBuffer::localMetadata(std::string &blob) const {
    if (!ok_) return NIXL_ERR_BACKEND;
    nixl_blob_t md;
    if (const nixl_status_t st = agent_.getLocalMD(md); st != NIXL_SUCCESS) return st;
    std::string name;
    // the agent's name travels inside its metadata; peers learn it from loadRemoteMD
    nixlSerDes sd;
    const int64_t head[6] = {cfg_.rank, static_cast<int64_t>(reinterpret_cast<uintptr_t>(buffer_)), total_, cfg_.device,
                             static_cast<int64_t>(epoch_), static_cast<int64_t>(barrierEpoch_)};
    sd.addBuf("ep", head, sizeof(head));
    sd.addStr("md", md);
    blob = sd.exportStr();
    return NIXL_SUCCESS;
}

nixl_status_t nixlEpBuffer::connectRanks(const std::vector<std::string> &blobs) {
    if (!ok_) return NIXL_ERR_BACKEND;
    for (const std::string &blob : blobs) {
        nixlSerDes sd;
        int64_t head[6];
        if (sd.importStr(blob) != NIXL_SUCCESS || sd.getBuf("ep", head, sizeof(head)) != NIXL_SUCCESS) return NIXL_ERR_MISMATCH;
        const std::string md = sd.getStr("md");
        const int r = static_cast<int>(head[0]);
        if (r < 0 || r >= cfg_.numRanks || md.empty()) return NIXL_ERR_MISMATCH;
        if (r == cfg_.rank || peers_[r].connected) continue;
        std::string name;
        if (const nixl_status_t st = agent_.loadRemoteMD(md, name); st != NIXL_SUCCESS) return st;
        peers_[r] = Peer{name, static_cast<uintptr_t>(head[1]), static_cast<size_t>(head[2]), static_cast<int>(head[3]), true};
        // Flags carry the step number: a rank that missed steps catches up with the ranks it connects to.
        epoch_ = std::max<uint64_t>(epoch_, static_cast<uint64_t>(head[4]));
        barrierEpoch_ = std::max<uint64_t>(barrierEpoch_, static_cast<uint64_t>(head[5]));
        DeviceGuard dg(cfg_.device);
        const int zero = 0;
        cudaMemcpy(mask_ + r, &zero, sizeof(int), cudaMemcpyHostToDevice);
    }
    return rebuildView();
}

nixl_status_t nixlEpBuffer::disconnectRanks(const std::vector<int> &ranks) {
    if (!ok_) return NIXL_ERR_BACKEND;
    DeviceGuard dg(cfg_.device);
    for (int r : ranks) {
        if (r < 0 || r >= cfg_.numRanks || r == cfg_.rank) continue;
        if (peers_[r].connected) agent_.invalidateRemoteMD(peers_[r].agent);
        peers_[r] = Peer{};
        const int one = 1;
        cudaMemcpy(mask_ + r, &one, sizeof(int), cudaMemcpyHostToDevice);
    }
    return rebuildView();
}

nixl_status_t nixlEpBuffer::rebuildView() {
    DeviceGuard dg(cfg_.device);
    if (peersView_) {
        agent_.releaseMemView(peersView_);
        peersView_ = nullptr;
    }
    nixl_remote_dlist_t rows(VRAM_SEG);
    for (int r = 0; r < cfg_.numRanks; ++r) {
        if (r == cfg_.rank) rows.addDesc(nixlRemoteDesc(reinterpret_cast<uintptr_t>(buffer_), static_cast<size_t>(total_), cfg_.device, cfg_.agentName));
        else if (peers_[r].connected) rows.addDesc(nixlRemoteDesc(peers_[r].addr, peers_[r].len, peers_[r].dev, peers_[r].agent));
        else rows.addDesc(nixlRemoteDesc(0, 0, 0, nixl_null_agent)); // a hole keeps indices equal to rank numbers
    }
    return agent_.prepMemView(rows, peersView_);
}

nixl_status_t nixlEpBuffer::doDispatch(const void *x, const int64_t *topkIdx, int tokens, bool fp8, const float *weights, int rowsPerExpert,
                                       cudaStream_t stream, nixlEpHandle &out) {
    if (!ok_ || !x || !topkIdx || tokens < 0 || tokens > cfg_.maxTokens) return NIXL_ERR_INVALID_PARAM;
    if (rowsPerExpert && !cfg_.lowLatencyMode) return NIXL_ERR_INVALID_PARAM;
    if (!peersView_) {
        if (cfg_.numRanks != 1) return NIXL_ERR_NOT_FOUND; // connectRanks first
        if (const nixl_status_t st = rebuildView(); st != NIXL_SUCCESS) return st;
    }
    if (weights && (cfg_.topk > 8 || cfg_.numRanks > 32)) weights = nullptr; // a group record holds eight copies
    DeviceGuard dg(cfg_.device);
    ++epoch_;
    const int parity = static_cast<int>(epoch_ & 1);
    const int El = localExperts();
    NixlEpDispatchParams p{};
    p.x = x;
    p.topk_idx = topkIdx;
    p.T = tokens;
    p.K = cfg_.topk;
    p.H = cfg_.hidden;
    p.E = cfg_.numExperts;
    p.R = cfg_.numRanks;
    p.rank = cfg_.rank;
    p.use_fp8 = fp8 ? 1 : 0;
    p.rows_per_expert = rowsPerExpert;
    p.cap = static_cast<int32_t>(rowsPerExpert ? llRows_ : compactRows_);
    p.phases = 3;
    p.grid = 0;
    p.peers = peersView_;
    p.lay = layout(parity);
    p.epoch = epoch_;
    p.timeout_ns = cfg_.timeoutMs * 1000000ull;
    p.recv_count = recvCount_[parity];
    p.layout_range = layoutRange_[parity];
    p.expert_offsets = expertOffsets_[parity];
    p.scr = scratch();
    p.send_row = sendRow_[parity];
    p.topk_weights = weights;
    p.max_tokens = cfg_.maxTokens;
    if (const int e = nixl_ep_dispatch_launch(&p, stream); e != 0) {
        NIXL_ERROR << "nixlEpBuffer: dispatch launch failed: " << cudaGetErrorString(static_cast<cudaError_t>(e));
        return NIXL_ERR_BACKEND;
    }
    out = nixlEpHandle{};
    out.parity = parity;
    out.epoch = epoch_;
    out.rowsPerExpert = rowsPerExpert;
    out.hasGroupRecords = weights != nullptr;
    out.recvX = buffer_ + p.lay.off_recv_x;
    out.recvScales = fp8 ? reinterpret_cast<float *>(buffer_ + p.lay.off_recv_scales) : nullptr;
    out.rows = p.cap;
    out.recvCount = recvCount_[parity];
    out.expertOffsets = expertOffsets_[parity];
    out.layoutRange = layoutRange_[parity];
    out.srcInfo = reinterpret_cast<const uint32_t *>(buffer_ + p.lay.off_recv_info);
    out.sendRow = sendRow_[parity];
    (void)El;
    return NIXL_SUCCESS;
}

nixl_status_t nixlEpBuffer::dispatch(const void *x, const int64_t *topkIdx, int tokens, bool fp8, const float *weights, cudaStream_t stream,
                                     nixlEpHandle &out) {
    return doDispatch(x, topkIdx, tokens, fp8, weights, 0, stream, out);
}

nixl_status_t nixlEpBuffer::lowLatencyDispatch(const void *x, const int64_t *topkIdx, int tokens, bool fp8, cudaStream_t stream, nixlEpHandle &out) {
    return doDispatch(x, topkIdx, tokens, fp8, nullptr, cfg_.numRanks * cfg_.maxTokens, stream, out);
}

void *nixlEpBuffer::combineInput(const nixlEpHandle &h) const {
    return ok_ ? buffer_ + layout(h.parity).off_comb_in : nullptr;
}

nixl_status_t nixlEpBuffer::combine(const void *y, const int64_t *topkIdx, const float *weights, const nixlEpHandle &h, void *out, int tokens,
                                    cudaStream_t stream, nixlEpCombineMode mode) {
    if (!ok_ || !y || !topkIdx || !weights || !out || !peersView_) return NIXL_ERR_INVALID_PARAM;
    DeviceGuard dg(cfg_.device);
    const long long rows = h.rowsPerExpert ? llRows_ : compactRows_;
    void *staged = combineInput(h);
    if (mode == nixlEpCombineMode::AUTO) {
        // One row per (token, rank) when the expert ranks know which rows belong together; else pull when the
        // outputs already lie in the exposed region (nothing to copy), push when they live elsewhere.
        if (h.hasGroupRecords) mode = nixlEpCombineMode::RANK_REDUCE;
        else mode = y == staged ? nixlEpCombineMode::PULL : nixlEpCombineMode::PUSH;
    }
    if (mode == nixlEpCombineMode::RANK_REDUCE && !h.hasGroupRecords) return NIXL_ERR_INVALID_PARAM;
    if (mode == nixlEpCombineMode::PULL && y != staged) {
        if (cudaMemcpyAsync(staged, y, static_cast<size_t>(rows) * cfg_.hidden * 2, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return NIXL_ERR_BACKEND;
    }
    NixlEpCombineParams p{};
    p.x = y;
    p.recv_info = h.srcInfo;
    p.recv_count = h.recvCount;
    p.expert_offsets = h.expertOffsets;
    p.topk_idx = topkIdx;
    p.topk_weights = weights;
    p.out = out;
    p.T = tokens;
    p.K = cfg_.topk;
    p.H = cfg_.hidden;
    p.E = cfg_.numExperts;
    p.R = cfg_.numRanks;
    p.rank = cfg_.rank;
    p.phases = 3;
    p.grid = 0;
    p.peers = peersView_;
    p.lay = layout(h.parity);
    p.epoch = h.epoch;
    p.timeout_ns = cfg_.timeoutMs * 1000000ull;
    p.scr = scratch();
    p.pull = static_cast<int>(mode);
    p.send_row = h.sendRow;
    p.use_logfmt = 0;
    p.max_tokens = cfg_.maxTokens;
    if (const int e = nixl_ep_combine_launch(&p, stream); e != 0) {
        NIXL_ERROR << "nixlEpBuffer: combine launch failed: " << cudaGetErrorString(static_cast<cudaError_t>(e));
        return NIXL_ERR_BACKEND;
    }
    return NIXL_SUCCESS;
}

nixl_status_t nixlEpBuffer::barrier(cudaStream_t stream) {
    if (!ok_ || !peersView_) return NIXL_ERR_INVALID_PARAM;
    DeviceGuard dg(cfg_.device);
    ++barrierEpoch_;
    const int e = nixl_ep_barrier_launch(peersView_, barrierOff_, cfg_.numRanks, cfg_.rank, barrierEpoch_, cfg_.timeoutMs * 1000000ull, status_, mask_,
                                         stream);
    return e == 0 ? NIXL_SUCCESS : NIXL_ERR_BACKEND;
}

int nixlEpBuffer::status() const {
    if (!ok_) return -1;
    DeviceGuard dg(cfg_.device);
    int v = 0;
    cudaMemcpy(&v, status_, sizeof(int), cudaMemcpyDeviceToHost);
    return v;
}

std::vector<int> nixlEpBuffer::queryMask() const {
    std::vector<int> m(cfg_.numRanks, 0);
    if (!ok_) return m;
    DeviceGuard dg(cfg_.device);
    cudaMemcpy(m.data(), mask_, m.size() * sizeof(int), cudaMemcpyDeviceToHost);
    return m;
}

void nixlEpBuffer::updateMask(int rank, bool masked) {
    if (!ok_ || rank < 0 || rank >= cfg_.numRanks) return;
    DeviceGuard dg(cfg_.device);
    const int v = masked ? 1 : 0;
    cudaMemcpy(mask_ + rank, &v, sizeof(int), cudaMemcpyHostToDevice);
}

void nixlEpBuffer::cleanMask() {
    if (!ok_) return;
    DeviceGuard dg(cfg_.device);
    cudaMemset(mask_, 0, cfg_.numRanks * sizeof(int));
    cudaMemset(status_, 0, sizeof(int));
}

// ================================================================================================ nixlKvTransfer

namespace {
void kvStrides(const nixlKvLayout &l, int64_t &block, int64_t &token, int64_t &head) {
    const int64_t row = static_cast<int64_t>(l.headDim) * l.elemBytes;
    block = static_cast<int64_t>(l.tokens) * l.heads * row;
    if (l.hnd) {
        token = row;
        head = static_cast<int64_t>(l.tokens) * row;
    } else {
        token = static_cast<int64_t>(l.heads) * row;
        head = row;
    }
}
} // namespace

nixlKvTransfer::nixlKvTransfer(nixlAgent &agent, const std::vector<nixlBasicDesc> &srcTensors, const nixlKvLayout &srcLayout,
                               const std::string &remoteAgent, const std::vector<nixlBasicDesc> &dstTensors, const nixlKvLayout &dstLayout,
                               int dstHeadOffset, bool castFp8, float scale)
    : agent_(agent) {
    if (srcTensors.empty() || srcTensors.size() != dstTensors.size() || srcLayout.tokens != dstLayout.tokens || srcLayout.headDim != dstLayout.headDim ||
        dstHeadOffset < 0 || dstHeadOffset + srcLayout.heads > dstLayout.heads || srcLayout.elemBytes != 2 || castFp8 != (dstLayout.elemBytes == 1)) {
        NIXL_ERROR << "nixlKvTransfer: the two layouts do not fit together";
        return;
    }
    device_ = static_cast<int>(srcTensors.front().devId);
    DeviceGuard dg(device_);
    nixl_local_dlist_t local(VRAM_SEG);
    for (const auto &d : srcTensors) local.addDesc(d);
    nixl_remote_dlist_t remote(VRAM_SEG);
    for (const auto &d : dstTensors) remote.addDesc(nixlRemoteDesc(d, remoteAgent));
    if (agent_.prepMemView(local, srcView_) != NIXL_SUCCESS || agent_.prepMemView(remote, dstView_) != NIXL_SUCCESS) {
        NIXL_ERROR << "nixlKvTransfer: the agent could not prepare the memory views (are both sides registered and the peer's metadata loaded?)";
        return;
    }
    if (!devAlloc(counter_, 64) || cudaHostAlloc(reinterpret_cast<void **>(&flag_), 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return;
    flag_[0] = flag_[1] = 0;
    p_.status = reinterpret_cast<int32_t *>(flag_ + 1); // second word of the pinned block: set when a block id was out of range
    p_.src_view = srcView_;
    p_.dst_view = dstView_;
    p_.n_tensors = static_cast<int32_t>(srcTensors.size());
    p_.tokens = srcLayout.tokens;
    p_.heads = srcLayout.heads;
    p_.head_bytes = srcLayout.headDim * 2;
    p_.cast_fp8 = castFp8 ? 1 : 0;
    kvStrides(srcLayout, p_.src_block_stride, p_.src_token_stride, p_.src_head_stride);
    kvStrides(dstLayout, p_.dst_block_stride, p_.dst_token_stride, p_.dst_head_stride);
    p_.dst_head_offset = dstHeadOffset;
    p_.scale = scale;
    p_.done_counter = counter_;
    p_.host_flag = flag_;
    p_.grid = 0;
    ok_ = true;
}

nixlKvTransfer::~nixlKvTransfer() {
    DeviceGuard dg(device_);
    if (ok_ && seq_ > 0) wait(seq_, 10.0);
    if (srcView_) agent_.releaseMemView(srcView_);
    if (dstView_) agent_.releaseMemView(dstView_);
    if (counter_) cudaFree(counter_);
    if (flag_) cudaFreeHost(flag_);
}

nixl_status_t nixlKvTransfer::post(const int32_t *srcBlocks, const int32_t *dstBlocks, int pairs, cudaStream_t stream, uint64_t &ticket,
                                   uint64_t *doneSignal, uint64_t doneValue) {
    if (!ok_ || !srcBlocks || !dstBlocks || pairs <= 0) return NIXL_ERR_INVALID_PARAM;
    DeviceGuard dg(device_);
    p_.src_blocks = srcBlocks;
    p_.dst_blocks = dstBlocks;
    p_.n_pairs = pairs;
    p_.done_signal = doneSignal;
    p_.done_value = doneValue;
    p_.host_seq = ++seq_;
    if (const int e = nixl_kv_xfer_launch(&p_, stream); e != 0) {
        NIXL_ERROR << "nixlKvTransfer: launch failed: " << cudaGetErrorString(static_cast<cudaError_t>(e));
        return NIXL_ERR_BACKEND;
    }
    ticket = seq_;
    return NIXL_SUCCESS;
}

bool nixlKvTransfer::done(uint64_t ticket) const { return ok_ && *reinterpret_cast<volatile uint64_t *>(flag_) >= ticket; }

nixl_status_t nixlKvTransfer::wait(uint64_t ticket, double timeoutSeconds) const {
    if (!ok_) return NIXL_ERR_BACKEND;
    const auto t0 = std::chrono::steady_clock::now();
    for (uint32_t spins = 0; !done(ticket); ++spins)
        if ((spins & 0xfff) == 0xfff && std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeoutSeconds) return NIXL_IN_PROG;
    if (*reinterpret_cast<volatile uint64_t *>(flag_ + 1) != 0) { // the kernel skipped a block whose id pointed outside its cache tensor
        *reinterpret_cast<volatile uint64_t *>(flag_ + 1) = 0;
        NIXL_ERROR << "nixlKvTransfer: a block id pointed outside its cache tensor; that block was not transferred";
        return NIXL_ERR_INVALID_PARAM;
    }
    return NIXL_SUCCESS;
}

// NVLINK backend: intra-box transfers between registered DRAM and VRAM regions.
//
// This is the B200-native replacement for the reference's default UCX backend
// (src/plugins/ucx/ucx_backend.{h,cpp}); it fills the same south-bound interface:
//   * registration exports what a peer needs to reach the memory (CUDA IPC handle of the
//     enclosing allocation + offset for VRAM; pid + address for DRAM) in the public
//     metadata blob, the slot where UCX ships rkeys;
//   * loading remote metadata maps the peer's memory into this process (same process:
//     the pointer itself plus peer access; other process: cudaIpcOpenMemHandle);
//   * a transfer is ONE kernel launch per local GPU for the whole descriptor batch
//     (xfer_kernels.cu), which stores straight into the peer's HBM over NVLink (WRITE) or
//     loads from it (READ) and publishes completion to a host-mapped word;
//   * DRAM<->DRAM moves by memcpy (same process) or process_vm_readv/writev (other
//     process); pinned DRAM is visible to the copy kernel, so DRAM<->VRAM is the same kernel;
//   * notifications travel as datagrams on an abstract unix socket (other process) or a
//     direct queue push (same process), after the data is complete;
//   * a dead peer is detected on the host (registry / pid / socket) and reported as
//     NIXL_ERR_REMOTE_DISCONNECT; nothing on the GPU waits for a peer.
// Device-side memory views for GPU-initiated transfers are prepared here too
// (include/device/nixl_device.cuh).
#ifndef NIXL_B200_NVLINK_BACKEND_H
#define NIXL_B200_NVLINK_BACKEND_H

#include <atomic>
#include <condition_variable>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include <cuda_runtime.h>

#include "backend/backend_engine.h"
#include "plugins/nvlink/notif_ring.h"
#include "plugins/nvlink/vmm_share.h"
#include "plugins/nvlink/xfer_kernels.h"

namespace nixl_nvlink {

// Identity of an engine as published in its connection info.
struct PeerId {
    std::string agent;
    std::string host;
    int64_t pid = 0;
    uint64_t procTag = 0;   // random per process: tells "same pid number" from "same process"
    uint64_t engineTag = 0; // random per engine instance
    std::string sockName;   // abstract unix datagram socket receiving notifications
    std::string ringName;   // shared-memory notification ring (empty: none)
};

class Engine;

// Local registration.
class LocalMD : public nixlBackendMD {
public:
    LocalMD() : nixlBackendMD(true) {}
    nixl_mem_t mem = DRAM_SEG;
    uintptr_t addr = 0;
    size_t len = 0;
    int device = -1;           // VRAM: CUDA ordinal
    uintptr_t devVisible = 0;  // address usable by kernels (VRAM: addr; pinned DRAM: mapped address; else 0)
    bool pinnedByUs = false;   // we called cudaHostRegister
    bool hasIpc = false;
    cudaIpcMemHandle_t ipc{};
    uint64_t ipcOffset = 0;    // addr - base of the enclosing allocation
    std::vector<VmmChunk> vmm; // VMM memory (no IPC handle): its allocations, exported as file descriptors
};

// A peer's registration as seen from here.
class RemoteMD : public nixlBackendMD {
public:
    RemoteMD() : nixlBackendMD(false) {}
    std::string agent;
    nixl_mem_t mem = DRAM_SEG;
    uintptr_t addr = 0;        // address in the owner's address space
    size_t len = 0;
    int ownerDevice = -1;      // owner's CUDA ordinal in the owner's process (VRAM)
    int ownerLocalDevice = -1; // the same GPU's ordinal in THIS process (-1: unknown / not VRAM)
    bool sameProcess = false;
    uintptr_t devVisible = 0;  // kernel-usable address in THIS process covering [addr, addr+len); 0 if none
    int mapDevice = -1;        // local device the IPC mapping was opened on (other-process VRAM)
    int64_t ownerPid = 0;
    std::string ipcKey;        // key into the process-wide IPC mapping cache (empty: none)
    bool loopback = false;     // produced by loadLocalMD
    VmmMapping vmmMap;         // other-process VMM memory mapped here (va == 0: none)
};

// Simple first-fit sub-allocator over device slabs (tables and counters of requests).
class DeviceArena {
public:
    explicit DeviceArena(int device) : device_(device) {}
    ~DeviceArena();
    void *alloc(size_t bytes); // 256-byte aligned; nullptr on failure
    void free(void *p);

private:
    struct Slab { char *base; size_t size; std::map<size_t, size_t> freeByOff; std::map<size_t, size_t> used; };
    int device_;
    std::mutex mu_;
    std::vector<Slab> slabs_;
};

// Pinned, device-mapped completion words, handed out one per prepared request.  Grows by
// pages of kWordsPerPage words, so the number of prepared requests is bounded by host memory only.
class FlagPool {
public:
    ~FlagPool();
    uint64_t *acquire(); // zeroed word; nullptr when pinned memory cannot be had
    void release(uint64_t *w);
    size_t pages() const { return pages_.size(); }

private:
    static constexpr size_t kWordsPerPage = 4096;
    std::mutex mu_;
    std::vector<uint64_t *> pages_;
    std::vector<uint64_t *> free_;
};

// "Last CTA" counters of the copy kernel, one per prepared request.  A counter is zero whenever
// no kernel of its request runs (the last CTA resets it), so words go back to the pool as they
// are and the pool never has to clear one; they must not share an allocator with blocks that
// hold other data (a recycled descriptor table is not zero).
class CounterPool {
public:
    explicit CounterPool(int device) : device_(device) {}
    ~CounterPool();
    unsigned int *acquire(); // nullptr when device memory cannot be had
    void release(unsigned int *w);

private:
    static constexpr size_t kPerSlab = 4096, kStride = 64; // bytes between counters: no two share a 64-byte line
    int device_;
    std::mutex mu_;
    std::vector<char *> slabs_;
    std::vector<unsigned int *> free_;
};

// Host side of the doorbell proxy (xfer_kernels.h): the rings, and whether a kernel is alive.
struct Proxy {
    std::mutex mu;
    void *pinned = nullptr;         // one pinned, mapped block: ring | completion words | exit word
    ProxyCmd *hostRing = nullptr;
    uint64_t *done = nullptr;
    uint64_t *exitWord = nullptr;
    ProxyShared *shared = nullptr;  // device memory
    cudaStream_t stream = nullptr;  // proxy launches only: a new launch starts after the previous kernel has gone
    uint64_t posted = 0;            // number of commands written so far
    uint64_t nextStart = 0;         // first command the next launch takes
    uint64_t launches = 0;          // launches so far (the kernel tags its ring entries with it)
    bool launched = false;          // a kernel was launched and its exit word has not been seen yet
    std::atomic<bool> broken{false}; // set-up or a launch failed: the proxy is not used again, its pending commands fail
};

// Per-device resources of one engine.
struct DeviceCtx {
    int device = -1;
    std::vector<cudaStream_t> streams; // transfers: a request is bound to one of them when it is prepared
    std::atomic<uint32_t> nextStream{0};
    cudaStream_t prepStream = nullptr; // table uploads
    std::unique_ptr<DeviceArena> arena;
    std::unique_ptr<CounterPool> counters;
    FlagPool flags;
    std::unique_ptr<Proxy> proxy;      // created with the first small request
    int gridCtas = 0;
    int smCount = 148;
};

struct KernelBatch {
    int device = -1;
    std::vector<XferDesc> descs;   // copied by the kernel (dropped once they sit in the launch parameters / device table)
    std::vector<XferDesc> ceDescs; // large descriptors handed to the copy engines, one cudaMemcpyAsync each
    XferLaunch launch{};
    void *table = nullptr; // arena block holding table + chunk starts (nullptr when only inline)
    const XferDesc *tableDev = nullptr;   // the uploaded table and chunk starts inside `table`
    const uint32_t *startsDev = nullptr;
    bool proxyEligible = false; // small, kernel-only: may go through the doorbell proxy
    bool tableReady = false;    // the upload has been seen complete
    uint32_t uniformChunks = 0; // chunks per descriptor when every descriptor has the same number, else 0
    bool viaProxy = false;      // the post in flight went through the proxy
    uint64_t proxyCmd = 0;      // its command number
    struct Proxy *proxy = nullptr; // the proxy it went through
    XferDesc single{};          // the one descriptor of a one-descriptor batch
    unsigned int *counter = nullptr;
    uint64_t *flag = nullptr;      // completion word (FlagPool)
    cudaStream_t stream = nullptr; // engine stream this batch posts on unless the caller names one
    cudaEvent_t uploaded = nullptr;
    uint64_t seq = 0;
    bool inFlight = false;
    uint64_t *notifWord = nullptr; // host address of the notification slot this post claimed (nullptr: none)
    uint64_t notifSeq = 0;
};

struct HostCopy { void *dst; const void *src; size_t len; };
struct CmaCopy { uintptr_t local; uintptr_t remote; size_t len; };
struct AsyncCopy { void *dst; const void *src; size_t len; int device; };

class ReqH : public nixlBackendReqH {
public:
    nixl_xfer_op_t op = NIXL_WRITE;
    std::string remoteAgent;
    std::vector<KernelBatch> kernels;
    std::vector<HostCopy> hostCopies;
    std::vector<CmaCopy> cmaCopies;
    int64_t cmaPid = 0;
    std::vector<AsyncCopy> asyncCopies;
    std::vector<std::pair<int, cudaEvent_t>> asyncEvents; // device, event
    bool asyncInFlight = false;
    size_t totalBytes = 0;
    // notification to deliver once the data is complete
    bool notifPending = false;
    std::string notifMsg;
    std::mutex mu; // progress thread vs. user thread
    nixl_status_t last = NIXL_ERR_NOT_POSTED;
    // Peer identity looked up at prepare time; valid while peerGen equals the engine's generation.
    std::shared_ptr<const PeerId> peer;
    uint64_t peerGen = 0;
    int64_t lastAliveNs = 0; // steady-clock time of the last other-process liveness look
};

// Device-side view handle header (mirrors include/device/nixl_device.cuh).
struct MemViewHost {
    uint64_t magic;
    const Engine *owner;
    void *devBlock;
    int device;
};

class Engine : public nixlBackendEngine {
public:
    explicit Engine(const nixlBackendInitParams *init);
    ~Engine() override;

    bool supportsRemote() const override { return true; }
    bool supportsLocal() const override { return true; }
    bool supportsNotif() const override { return true; }
    nixl_mem_list_t getSupportedMems() const override { return {DRAM_SEG, VRAM_SEG}; }

    nixl_status_t registerMem(const nixlBlobDesc &mem, const nixl_mem_t &nixl_mem, nixlBackendMD *&out) override;
    nixl_status_t deregisterMem(nixlBackendMD *meta) override;
    nixl_status_t connect(const std::string &remote_agent) override;
    nixl_status_t disconnect(const std::string &remote_agent) override;
    nixl_status_t unloadMD(nixlBackendMD *input) override;

    nixl_status_t prepXfer(const nixl_xfer_op_t &operation, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote,
                           const std::string &remote_agent, nixlBackendReqH *&handle,
                           const nixl_opt_b_args_t *opt_args = nullptr) const override;
    nixl_status_t postXfer(const nixl_xfer_op_t &operation, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote,
                           const std::string &remote_agent, nixlBackendReqH *&handle,
                           const nixl_opt_b_args_t *opt_args = nullptr) const override;
    nixl_status_t checkXfer(nixlBackendReqH *handle) const override;
    nixl_status_t releaseReqH(nixlBackendReqH *handle) const override;

    nixl_status_t prepMemView(const nixl_remote_meta_dlist_t &, nixlMemViewH &, const nixl_opt_b_args_t * = nullptr) const override;
    nixl_status_t prepMemView(const nixl_meta_dlist_t &, nixlMemViewH &, const nixl_opt_b_args_t * = nullptr) const override;
    void releaseMemView(nixlMemViewH) const override;

    nixl_status_t getPublicData(const nixlBackendMD *meta, std::string &str) const override;
    nixl_status_t getConnInfo(std::string &str) const override;
    nixl_status_t loadRemoteConnInfo(const std::string &remote_agent, const std::string &remote_conn_info) override;
    nixl_status_t loadRemoteMD(const nixlBlobDesc &input, const nixl_mem_t &nixl_mem, const std::string &remote_agent,
                               nixlBackendMD *&output) override;
    nixl_status_t loadLocalMD(nixlBackendMD *input, nixlBackendMD *&output) override;

    nixl_status_t getNotifs(notif_list_t &notif_list) override;
    nixl_status_t genNotif(const std::string &remote_agent, const std::string &msg) const override;

    nixl_status_t estimateXferCost(const nixl_xfer_op_t &, const nixl_meta_dlist_t &, const nixl_meta_dlist_t &,
                                   const std::string &, nixlBackendReqH *const &, std::chrono::microseconds &,
                                   std::chrono::microseconds &, nixl_cost_t &, const nixl_opt_args_t * = nullptr) const override;

    // Used by peers in the same process.
    void pushNotif(const std::string &from, const std::string &msg);
    uint64_t engineTag() const { return self_.engineTag; }

private:
    DeviceCtx *ctx(int device) const;
    bool peerAlive(const PeerId &peer, bool force = false) const;
    std::shared_ptr<const PeerId> findPeer(const std::string &agent, uint64_t *gen = nullptr) const;
    void destroyReq(ReqH *req) const; // waits for launched work, frees device resources, deletes
    bool postViaProxy(DeviceCtx *c, KernelBatch &b) const; // false: take the launch path
    void proxyEnsureRunning(DeviceCtx *c, Proxy &px) const; // px.mu held
    int proxyDone(DeviceCtx *c, KernelBatch &b) const; // 1 complete, 0 in progress, -1 the proxy failed
    nixl_status_t sendNotif(const PeerId &peer, const std::string &msg) const;
    nixl_status_t finishIfDone(ReqH *req) const; // data complete -> deliver notification
    nixl_status_t pollData(ReqH *req) const;
    bool ensurePeerAccess(int from, int to) const;
    void progressLoop();
    void freeBatch(KernelBatch &b) const;

    PeerId self_;
    bool cuda_ = false;
    int deviceCount_ = 0;
    bool pinDram_ = true;
    CopyPath copyPath_ = CopyPath::VECTOR;
    int gridOverride_ = 0;
    int chunkShiftOverride_ = 0; // "chunk_shift" parameter: log2 of the bytes one CTA copies at a time (14..22); 0 = automatic
    // Descriptors between two GPUs of at least this many bytes go to the copy engines instead of
    // the copy kernel ("ce_threshold"; 0: never).  Measured on NVLink 5: SM-issued stores deliver
    // 714 GB/s one way and 703 GB/s with the opposite direction busy, because every 256 payload
    // bytes of a store carry 48 protocol bytes on the wire; copy-engine writes carry 32 and deliver
    // 779 / 774 GB/s, but each copy costs about 7.5 us to start and drain.
    size_t ceThreshold_ = size_t(96) << 20;
    bool coalesce_ = true; // "coalesce": merge descriptors that continue their predecessor on both sides
    bool livenessPing_ = false;

    int numStreams_ = 4;
    // Doorbell proxy for small requests ("proxy", "proxy_max_bytes", "proxy_workers", "proxy_idle_us", "proxy_life_us").
    bool proxyEnabled_ = true;
    size_t proxyMaxBytes_ = size_t(2) << 20;
    int proxyWorkers_ = 24;
    uint64_t proxyIdleNs_ = 100000;
    uint64_t proxyLifeNs_ = 2000000;

    mutable std::mutex peersMu_;
    std::unordered_map<std::string, std::shared_ptr<const PeerId>> peers_;
    mutable std::atomic<uint64_t> peersGen_{1}; // bumped whenever peers_ changes

    mutable std::mutex ctxMu_;
    mutable std::vector<std::unique_ptr<DeviceCtx>> ctxs_;
    mutable std::atomic<int> primaryDevice_{-1};

    VmmFdServer fdServer_; // hands exported VMM descriptors to importing processes (started with the first VMM registration)
    int notifFd_ = -1;
    bool notifRingEnabled_ = true; // "notif_ring": notifications of kernel-path requests are released by the copy kernel itself
    NotifRingOwner notifRing_;     // the ring peers write into
    mutable std::mutex ringMu_;
    mutable std::unordered_map<std::string, std::shared_ptr<NotifRingWriter>> peerRings_; // by ring name
    std::shared_ptr<NotifRingWriter> ringOf(const PeerId &peer) const; // mapped and registered with CUDA, or nullptr
    mutable std::mutex notifMu_;
    notif_list_t inbox_; // same-process deliveries
    std::vector<char> notifBuf_; // receive buffer of getNotifs, kept between polls

    // progress thread
    bool progThread_ = false;
    uint64_t progDelayUs_ = 0;
    mutable std::mutex progMu_;
    mutable std::condition_variable progCv_;
    mutable std::vector<ReqH *> progWatch_;
    std::atomic<bool> progStop_{false};
    std::thread progTh_;
};

uint64_t kernelLaunches(); // process-wide count of kernels launched by the backend

} // namespace nixl_nvlink

#endif

#include "plugins/nvlink/nvlink_backend.h"

#include <cerrno>
#include <csignal>
#include <cstring>
#include <random>
#include <sys/socket.h>
#include <sys/uio.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>

#include "backend/backend_plugin.h"
#include "device/nixl_device_layout.h"
#include "serdes/serdes.h"
#include "utils/hw_info.h"
#include "utils/log.h"
#include "utils/misc.h"

namespace nixl_nvlink {
namespace {

// ---------------------------------------------------------------- process-wide state

using nixl_util::hostName;
using nixl_util::random64;

// Words in pinned host memory that a GPU (or the doorbell proxy) writes with release semantics at system scope and
// this side polls: read them with an acquire load, so that everything the writer did before is visible afterwards.
inline uint64_t loadWord(const uint64_t *p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline void storeWord(uint64_t *p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }

uint64_t processTag() {
    static const uint64_t tag = random64() | 1;
    return tag;
}

// Engines alive in this process, by agent name: same-process peers talk directly.
std::mutex g_regMu;
std::unordered_map<std::string, Engine *> g_registry;

// CUDA IPC mappings are per process, not per engine: two agents (or two registrations that
// share one allocation) must not open the same handle twice.
struct IpcMapping {
    void *base = nullptr;
    int refs = 0;
    int device = -1;     // device that was current when the handle was opened
    int ownerLocal = -1; // local ordinal of the GPU that owns the memory
};
std::mutex g_ipcMu;
std::unordered_map<std::string, IpcMapping> g_ipc;

// Kernels this library launched in this process (copy kernels and completion kernels), for
// tools that report how much of a run went through them.
std::atomic<uint64_t> g_kernelLaunches{0};

std::mutex g_peerAccessMu;
std::vector<std::pair<int, int>> g_peerAccess;

// RAII: run a block with a given current device, then restore the caller's.
class DeviceScope {
public:
    explicit DeviceScope(int dev) {
        if (cudaGetDevice(&prev_) != cudaSuccess) prev_ = -1;
        if (dev >= 0 && dev != prev_) {
            cudaSetDevice(dev);
            changed_ = true;
        }
    }
    ~DeviceScope() {
        if (changed_ && prev_ >= 0) cudaSetDevice(prev_);
    }

private:
    int prev_ = -1;
    bool changed_ = false;
};

bool cudaOk(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return true;
    NIXL_ERROR << "NVLINK backend: " << what << " failed: " << cudaGetErrorString(e);
    cudaGetLastError(); // clear the sticky-less error so later calls are not blamed
    return false;
}

// cuMemGetAddressRange through the runtime's driver entry point (no link against libcuda).
bool allocationRange(uintptr_t ptr, uintptr_t &base, size_t &size) {
    using fn_t = int (*)(unsigned long long *, size_t *, unsigned long long);
    static fn_t fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<fn_t>(p);
    }();
    if (!fn) return false;
    unsigned long long b = 0;
    size_t s = 0;
    if (fn(&b, &s, ptr) != 0) return false;
    base = b;
    size = s;
    return true;
}

// UUID of a local GPU, looked up once per ordinal.
struct GpuUuid {
    unsigned char b[16];
};
const GpuUuid *deviceUuid(int dev) {
    static std::mutex mu;
    static std::vector<std::unique_ptr<GpuUuid>> cache;
    if (dev < 0) return nullptr;
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() <= static_cast<size_t>(dev)) cache.resize(dev + 1);
    if (!cache[dev]) {
        cudaDeviceProp prop{};
        if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cache[dev] = std::make_unique<GpuUuid>();
        std::memcpy(cache[dev]->b, prop.uuid.bytes, 16);
    }
    return cache[dev].get();
}

// Local ordinal of the GPU with that UUID, or -1 when this process does not see it.
int ordinalOfUuid(const unsigned char *uuid, int device_count) {
    for (int d = 0; d < device_count; ++d) {
        const GpuUuid *u = deviceUuid(d);
        if (u && std::memcmp(u->b, uuid, 16) == 0) return d;
    }
    return -1;
}

// ---------------------------------------------------------------- wire structs

constexpr uint8_t kPubVersion = 2;

#pragma pack(push, 1)
struct PubReg {
    uint8_t version;
    uint8_t mem; // nixl_mem_t
    uint8_t hasIpc;
    uint8_t pad;
    int32_t device;
    uint64_t addr;
    uint64_t len;
    uint64_t ipcOffset;
    uint64_t engineTag;
    unsigned char ipc[sizeof(cudaIpcMemHandle_t)];
    unsigned char gpuUuid[16]; // VRAM: which physical GPU holds the memory (ordinals differ between processes)
};
struct PubVmmChunk {
    uint64_t base;
    uint64_t size;
    int32_t fd;
    int32_t pad;
};
#pragma pack(pop)

std::string encodePeer(const PeerId &p) {
    nixlSerDes sd;
    sd.addStr("agent", p.agent);
    sd.addStr("host", p.host);
    sd.addBuf("pid", &p.pid, sizeof(p.pid));
    sd.addBuf("ptag", &p.procTag, sizeof(p.procTag));
    sd.addBuf("etag", &p.engineTag, sizeof(p.engineTag));
    sd.addStr("sock", p.sockName);
    if (!p.ringName.empty()) sd.addStr("ring", p.ringName);
    return sd.exportStr();
}

bool decodePeer(const std::string &blob, PeerId &p) {
    nixlSerDes sd;
    if (sd.importStr(blob) != NIXL_SUCCESS) return false;
    p.agent = sd.getStr("agent");
    p.host = sd.getStr("host");
    if (sd.getBuf("pid", &p.pid, sizeof(p.pid)) != NIXL_SUCCESS) return false;
    if (sd.getBuf("ptag", &p.procTag, sizeof(p.procTag)) != NIXL_SUCCESS) return false;
    if (sd.getBuf("etag", &p.engineTag, sizeof(p.engineTag)) != NIXL_SUCCESS) return false;
    p.sockName = sd.getStr("sock");
    p.ringName = sd.remaining() > 0 && sd.getBufLen("ring") > 0 ? sd.getStr("ring") : std::string(); // optional last field
    return !p.agent.empty() && !p.sockName.empty();
}

sockaddr_un abstractAddr(const std::string &name, socklen_t &len) {
    sockaddr_un a{};
    a.sun_family = AF_UNIX;
    const size_t n = std::min(name.size(), sizeof(a.sun_path) - 2);
    std::memcpy(a.sun_path + 1, name.data(), n); // leading NUL = abstract namespace
    len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
    return a;
}

uint32_t log2Ceil(uint64_t v) {
    uint32_t s = 0;
    while ((uint64_t(1) << s) < v) ++s;
    return s;
}

bool paramBool(const nixl_b_params_t &p, const char *key, bool dflt) {
    auto it = p.find(key);
    if (it == p.end()) return dflt;
    const std::string &v = it->second;
    return v == "1" || v == "true" || v == "yes" || v == "on" || v == "y";
}

long paramLong(const nixl_b_params_t &p, const char *key, long dflt) {
    auto it = p.find(key);
    if (it == p.end() || it->second.empty()) return dflt;
    char *end = nullptr;
    const long v = std::strtol(it->second.c_str(), &end, 0);
    return end && *end == 0 ? v : dflt;
}

} // namespace

uint64_t kernelLaunches() { return g_kernelLaunches.load(std::memory_order_relaxed); }

// ================================================================ DeviceArena

DeviceArena::~DeviceArena() {
    DeviceScope ds(device_);
    for (auto &s : slabs_) cudaFree(s.base);
}

void *DeviceArena::alloc(size_t bytes) {
    bytes = (bytes + 255) & ~size_t(255);
    std::lock_guard<std::mutex> g(mu_);
    for (int pass = 0; pass < 2; ++pass) {
        for (auto &s : slabs_) {
            for (auto it = s.freeByOff.begin(); it != s.freeByOff.end(); ++it) {
                if (it->second < bytes) continue;
                const size_t off = it->first, sz = it->second;
                s.freeByOff.erase(it);
                if (sz > bytes) s.freeByOff[off + bytes] = sz - bytes;
                s.used[off] = bytes;
                return s.base + off;
            }
        }
        if (pass == 1) break;
        const size_t slab = std::max<size_t>(bytes, size_t(8) << 20);
        DeviceScope ds(device_);
        void *p = nullptr;
        if (!cudaOk(cudaMalloc(&p, slab), "cudaMalloc(arena)")) return nullptr;
        cudaMemset(p, 0, slab);
        Slab s{static_cast<char *>(p), slab, {}, {}};
        s.freeByOff[0] = slab;
        slabs_.push_back(std::move(s));
    }
    return nullptr;
}

void DeviceArena::free(void *p) {
    if (!p) return;
    std::lock_guard<std::mutex> g(mu_);
    for (auto &s : slabs_) {
        char *c = static_cast<char *>(p);
        if (c < s.base || c >= s.base + s.size) continue;
        size_t off = static_cast<size_t>(c - s.base);
        auto u = s.used.find(off);
        if (u == s.used.end()) return;
        size_t sz = u->second;
        s.used.erase(u);
        // coalesce with neighbours
        auto next = s.freeByOff.find(off + sz);
        if (next != s.freeByOff.end()) {
            sz += next->second;
            s.freeByOff.erase(next);
        }
        auto prev = s.freeByOff.lower_bound(off);
        if (prev != s.freeByOff.begin()) {
            --prev;
            if (prev->first + prev->second == off) {
                off = prev->first;
                sz += prev->second;
                s.freeByOff.erase(prev);
            }
        }
        s.freeByOff[off] = sz;
        return;
    }
}

// ================================================================ CounterPool

CounterPool::~CounterPool() {
    DeviceScope ds(device_);
    for (char *p : slabs_) cudaFree(p);
}

unsigned int *CounterPool::acquire() {
    std::lock_guard<std::mutex> g(mu_);
    if (free_.empty()) {
        DeviceScope ds(device_);
        void *p = nullptr;
        if (!cudaOk(cudaMalloc(&p, kPerSlab * kStride), "cudaMalloc(counters)")) return nullptr;
        if (!cudaOk(cudaMemset(p, 0, kPerSlab * kStride), "cudaMemset(counters)")) {
            cudaFree(p);
            return nullptr;
        }
        slabs_.push_back(static_cast<char *>(p));
        for (size_t i = kPerSlab; i-- > 0;) free_.push_back(reinterpret_cast<unsigned int *>(static_cast<char *>(p) + i * kStride));
    }
    unsigned int *w = free_.back();
    free_.pop_back();
    return w;
}

void CounterPool::release(unsigned int *w) {
    if (!w) return;
    std::lock_guard<std::mutex> g(mu_);
    free_.push_back(w);
}

// ================================================================ FlagPool

FlagPool::~FlagPool() {
    for (uint64_t *p : pages_) cudaFreeHost(p);
}

uint64_t *FlagPool::acquire() {
    std::lock_guard<std::mutex> g(mu_);
    if (free_.empty()) {
        void *page = nullptr;
        if (!cudaOk(cudaHostAlloc(&page, kWordsPerPage * sizeof(uint64_t), cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc(flags)"))
            return nullptr;
        std::memset(page, 0, kWordsPerPage * sizeof(uint64_t));
        auto *w = static_cast<uint64_t *>(page);
        pages_.push_back(w);
        free_.reserve(free_.size() + kWordsPerPage);
        for (size_t i = kWordsPerPage; i-- > 0;) free_.push_back(w + i);
    }
    uint64_t *w = free_.back();
    free_.pop_back();
    *w = 0;
    return w;
}

void FlagPool::release(uint64_t *w) {
    if (!w) return;
    std::lock_guard<std::mutex> g(mu_);
    free_.push_back(w);
}

// ================================================================ Engine: lifecycle

Engine::Engine(const nixlBackendInitParams *init) : nixlBackendEngine(init) {
    const nixl_b_params_t &params = getCustomParams();
    self_.agent = localAgent;
    self_.host = hostName();
    // "host_id": what this engine takes for "the same NVLink box" instead of the host name.  Engines only reach peers
    // that name the same one, so containers with their own host names on one box can be told that they share it (they
    // must also share the IPC and pid name spaces), and a test can play two hosts on one machine.
    if (auto it = params.find("host_id"); it != params.end() && !it->second.empty()) self_.host = it->second;
    self_.pid = ::getpid();
    self_.procTag = processTag();
    self_.engineTag = random64() | 1;

    int n = 0;
    const bool want_cuda = paramBool(params, "use_cuda", true);
    if (want_cuda && cudaGetDeviceCount(&n) == cudaSuccess && n > 0) {
        cuda_ = true;
        deviceCount_ = n;
    } else {
        cudaGetLastError();
        // GPUs on the PCI bus that CUDA cannot open usually mean a driver / container set-up problem:
        // say so once instead of silently moving host memory only.
        const nixl::hwInfo &hw = nixl::hwInfo::instance();
        if (want_cuda && hw.numNvidiaGpus > 0)
            NIXL_WARN << "NVLINK backend: " << hw.numNvidiaGpus << " NVIDIA GPU(s) on the PCI bus but CUDA reports none; VRAM transfers are unavailable";
    }
    pinDram_ = paramBool(params, "pin_dram", true);
    auto cp = params.find("copy_path");
    if (cp != params.end() && (cp->second == "bulk" || cp->second == "tma")) copyPath_ = CopyPath::BULK;
    ceThreshold_ = static_cast<size_t>(std::max<long>(0, paramLong(params, "ce_threshold", static_cast<long>(ceThreshold_))));
    if (cp != params.end() && (cp->second == "ce" || cp->second == "copy_engine")) {
        copyPath_ = CopyPath::COPY_ENGINE; // every descriptor, whatever its size
        ceThreshold_ = 1;
    }
    gridOverride_ = static_cast<int>(paramLong(params, "grid_ctas", 0));
    chunkShiftOverride_ = static_cast<int>(paramLong(params, "chunk_shift", 0));
    livenessPing_ = paramBool(params, "liveness_ping", false);
    coalesce_ = paramBool(params, "coalesce", true);
    proxyEnabled_ = paramBool(params, "proxy", true);
    proxyMaxBytes_ = static_cast<size_t>(std::max<long>(0, paramLong(params, "proxy_max_bytes", static_cast<long>(proxyMaxBytes_))));
    proxyWorkers_ = static_cast<int>(std::min<long>(kProxyMaxWorkers, std::max<long>(1, paramLong(params, "proxy_workers", proxyWorkers_))));
    proxyIdleNs_ = static_cast<uint64_t>(std::max<long>(1, paramLong(params, "proxy_idle_us", 100))) * 1000;
    proxyLifeNs_ = static_cast<uint64_t>(std::max<long>(10, paramLong(params, "proxy_life_us", 2000))) * 1000;
    numStreams_ = static_cast<int>(std::min<long>(32, std::max<long>(1, paramLong(params, "num_streams", 4))));
    const long dev = paramLong(params, "device_id", -1);
    if (dev >= 0) primaryDevice_ = static_cast<int>(dev);

    // Notification endpoint.
    notifFd_ = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
    if (notifFd_ < 0) {
        NIXL_ERROR << "NVLINK backend: cannot create the notification socket: " << std::strerror(errno);
        initErr = true;
        return;
    }
    char name[96];
    std::snprintf(name, sizeof(name), "nixl_b200.%lld.%016llx", static_cast<long long>(self_.pid),
                  static_cast<unsigned long long>(self_.engineTag));
    self_.sockName = name;
    socklen_t alen = 0;
    sockaddr_un addr = abstractAddr(self_.sockName, alen);
    if (::bind(notifFd_, reinterpret_cast<sockaddr *>(&addr), alen) != 0) {
        NIXL_ERROR << "NVLINK backend: cannot bind the notification socket: " << std::strerror(errno);
        initErr = true;
        return;
    }
    int big = 8 << 20;
    setsockopt(notifFd_, SOL_SOCKET, SO_RCVBUF, &big, sizeof(big));
    setsockopt(notifFd_, SOL_SOCKET, SO_SNDBUF, &big, sizeof(big));

    notifRingEnabled_ = paramBool(params, "notif_ring", true);
    if (notifRingEnabled_ && cuda_) {
        char ring[96];
        std::snprintf(ring, sizeof(ring), "/nixl_b200.%lld.%016llx", static_cast<long long>(self_.pid), static_cast<unsigned long long>(self_.engineTag));
        if (notifRing_.create(ring)) self_.ringName = ring;
        else NIXL_DEBUG << "NVLINK backend: no shared-memory notification ring (" << std::strerror(errno) << "); notifications use datagrams";
    }

    {
        std::lock_guard<std::mutex> g(g_regMu);
        g_registry[self_.agent] = this;
    }
    progThread_ = init->enableProgTh;
    progDelayUs_ = init->pthrDelay;
    if (progThread_) progTh_ = std::thread([this] { progressLoop(); });
}

Engine::~Engine() {
    progStop_ = true;
    progCv_.notify_all();
    if (progTh_.joinable()) progTh_.join();
    {
        std::lock_guard<std::mutex> g(g_regMu);
        auto it = g_registry.find(self_.agent);
        if (it != g_registry.end() && it->second == this) g_registry.erase(it);
    }
    if (notifFd_ >= 0) ::close(notifFd_);
    for (auto &c : ctxs_) {
        if (!c) continue;
        DeviceScope ds(c->device);
        for (cudaStream_t st : c->streams) {
            cudaStreamSynchronize(st);
            cudaStreamDestroy(st);
        }
        if (c->prepStream) cudaStreamDestroy(c->prepStream);
        if (c->proxy) {
            Proxy &px = *c->proxy;
            if (px.stream) {
                cudaStreamSynchronize(px.stream); // the kernel leaves by itself once idle
                cudaStreamDestroy(px.stream);
            }
            if (px.shared) cudaFree(px.shared);
            if (px.pinned) cudaFreeHost(px.pinned);
        }
        c->arena.reset();
        c->counters.reset();
    }
}

DeviceCtx *Engine::ctx(int device) const {
    if (!cuda_ || device < 0 || device >= deviceCount_) return nullptr;
    std::lock_guard<std::mutex> g(ctxMu_);
    if (ctxs_.size() < static_cast<size_t>(deviceCount_)) ctxs_.resize(deviceCount_);
    if (ctxs_[device]) return ctxs_[device].get();
    DeviceScope ds(device);
    auto c = std::make_unique<DeviceCtx>();
    c->device = device;
    // Independent requests of one agent run side by side: each prepared request is bound to one
    // of numStreams_ streams (the role of the reference's worker split, ucx_backend.cpp:653-754).
    for (int i = 0; i < numStreams_; ++i) {
        cudaStream_t st = nullptr;
        if (!cudaOk(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking), "cudaStreamCreate")) return nullptr;
        c->streams.push_back(st);
    }
    if (!cudaOk(cudaStreamCreateWithFlags(&c->prepStream, cudaStreamNonBlocking), "cudaStreamCreate")) return nullptr;
    c->arena = std::make_unique<DeviceArena>(device);
    c->counters = std::make_unique<CounterPool>(device);
    c->gridCtas = gridOverride_ > 0 ? gridOverride_ : defaultGridCtas(device);
    c->smCount = 148;
    if (cudaDeviceGetAttribute(&c->smCount, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || c->smCount <= 0) c->smCount = 148;
    ctxs_[device] = std::move(c);
    return ctxs_[device].get();
}

bool Engine::ensurePeerAccess(int from, int to) const {
    if (from == to) return true;
    std::lock_guard<std::mutex> g(g_peerAccessMu);
    if (std::find(g_peerAccess.begin(), g_peerAccess.end(), std::make_pair(from, to)) != g_peerAccess.end()) return true;
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, from, to) != cudaSuccess || !can) {
        cudaGetLastError();
        return false;
    }
    DeviceScope ds(from);
    const cudaError_t e = cudaDeviceEnablePeerAccess(to, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
        cudaOk(e, "cudaDeviceEnablePeerAccess");
        return false;
    }
    cudaGetLastError();
    g_peerAccess.emplace_back(from, to);
    return true;
}

// ================================================================ registration

nixl_status_t Engine::registerMem(const nixlBlobDesc &mem, const nixl_mem_t &nixl_mem, nixlBackendMD *&out) {
    if (mem.len == 0) return NIXL_ERR_INVALID_PARAM;
    auto md = std::make_unique<LocalMD>();
    md->mem = nixl_mem;
    md->addr = mem.addr;
    md->len = mem.len;
    if (nixl_mem == VRAM_SEG) {
        if (!cuda_) return NIXL_ERR_NOT_SUPPORTED;
        if (mem.devId >= static_cast<uint64_t>(deviceCount_)) return NIXL_ERR_INVALID_PARAM;
        md->device = static_cast<int>(mem.devId);
        md->devVisible = mem.addr;
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, reinterpret_cast<void *>(mem.addr)) != cudaSuccess ||
            (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)) {
            cudaGetLastError();
            NIXL_ERROR << "NVLINK backend: address " << reinterpret_cast<void *>(mem.addr) << " is not device memory";
            return NIXL_ERR_INVALID_PARAM;
        }
        if (attr.device != md->device) {
            NIXL_ERROR << "NVLINK backend: descriptor says device " << md->device << " but the memory lives on " << attr.device;
            return NIXL_ERR_INVALID_PARAM;
        }
        int expected = -1;
        primaryDevice_.compare_exchange_strong(expected, md->device);
        // Export for other processes.  Memory that CUDA IPC cannot export (VMM, pools) stays
        // reachable from this process only.
        DeviceScope ds(md->device);
        uintptr_t base = 0;
        size_t size = 0;
        if (allocationRange(mem.addr, base, size) && mem.addr + mem.len <= base + size &&
            cudaIpcGetMemHandle(&md->ipc, reinterpret_cast<void *>(base)) == cudaSuccess) {
            md->hasIpc = true;
            md->ipcOffset = mem.addr - base;
        } else {
            cudaGetLastError();
            // Not cudaMalloc memory.  Memory from the virtual memory management API (PyTorch's expandable
            // segments, engines' own pools) is exported allocation by allocation as file descriptors.
            if (vmmExportRange(mem.addr, mem.len, md->vmm) && fdServer_.start(self_.sockName + ".fd")) {
                for (const auto &c : md->vmm) fdServer_.allow(c.fd);
                NIXL_DEBUG << "NVLINK backend: " << reinterpret_cast<void *>(mem.addr) << " exported as " << md->vmm.size() << " VMM allocation(s)";
            } else {
                vmmCloseChunks(md->vmm);
                NIXL_DEBUG << "NVLINK backend: no IPC handle for " << reinterpret_cast<void *>(mem.addr) << "; same-process use only";
            }
        }
    } else if (nixl_mem == DRAM_SEG) {
        if (cuda_ && pinDram_) {
            const int dev = primaryDevice_.load() >= 0 ? primaryDevice_.load() : 0;
            DeviceScope ds(dev);
            cudaError_t e = cudaHostRegister(reinterpret_cast<void *>(mem.addr), mem.len, cudaHostRegisterPortable | cudaHostRegisterMapped);
            if (e == cudaSuccess) md->pinnedByUs = true;
            if (e == cudaSuccess || e == cudaErrorHostMemoryAlreadyRegistered) {
                cudaGetLastError();
                void *dp = nullptr;
                if (cudaHostGetDevicePointer(&dp, reinterpret_cast<void *>(mem.addr), 0) == cudaSuccess)
                    md->devVisible = reinterpret_cast<uintptr_t>(dp);
                else cudaGetLastError();
            } else {
                cudaGetLastError();
                NIXL_DEBUG << "NVLINK backend: DRAM region not pinned (" << cudaGetErrorString(e) << "); staged copies will be used";
            }
        }
    } else {
        return NIXL_ERR_NOT_SUPPORTED;
    }
    out = md.release();
    return NIXL_SUCCESS;
}

nixl_status_t Engine::deregisterMem(nixlBackendMD *meta) {
    auto *md = dynamic_cast<LocalMD *>(meta);
    if (!md) return NIXL_ERR_INVALID_PARAM;
    if (md->pinnedByUs) {
        if (cudaHostUnregister(reinterpret_cast<void *>(md->addr)) != cudaSuccess) cudaGetLastError();
    }
    for (const auto &c : md->vmm) fdServer_.revoke(c.fd);
    vmmCloseChunks(md->vmm);
    delete md;
    return NIXL_SUCCESS;
}

nixl_status_t Engine::getPublicData(const nixlBackendMD *meta, std::string &str) const {
    auto *md = dynamic_cast<const LocalMD *>(meta);
    if (!md) return NIXL_ERR_INVALID_PARAM;
    PubReg pub{};
    pub.version = kPubVersion;
    pub.mem = static_cast<uint8_t>(md->mem);
    pub.hasIpc = md->hasIpc ? 1 : (md->vmm.empty() ? 0 : 2);
    pub.device = md->device;
    pub.addr = md->addr;
    pub.len = md->len;
    pub.ipcOffset = md->ipcOffset;
    pub.engineTag = self_.engineTag;
    std::memcpy(pub.ipc, &md->ipc, sizeof(md->ipc));
    if (md->mem == VRAM_SEG)
        if (const GpuUuid *u = deviceUuid(md->device)) std::memcpy(pub.gpuUuid, u->b, 16);
    str.assign(reinterpret_cast<const char *>(&pub), sizeof(pub));
    if (pub.hasIpc == 2) { // tail: allocation count, then (base, size, descriptor number) of each
        const uint32_t n = static_cast<uint32_t>(md->vmm.size());
        str.append(reinterpret_cast<const char *>(&n), sizeof(n));
        for (const auto &c : md->vmm) {
            PubVmmChunk w{c.base, c.size, c.fd, 0};
            str.append(reinterpret_cast<const char *>(&w), sizeof(w));
        }
    }
    return NIXL_SUCCESS;
}

nixl_status_t Engine::getConnInfo(std::string &str) const {
    str = encodePeer(self_);
    return NIXL_SUCCESS;
}

nixl_status_t Engine::loadRemoteConnInfo(const std::string &remote_agent, const std::string &remote_conn_info) {
    PeerId p;
    if (!decodePeer(remote_conn_info, p) || p.agent != remote_agent) return NIXL_ERR_MISMATCH;
    if (p.host != self_.host) {
        // Not an error of the deployment: with the TCP backend created next to this one the agent reaches that peer there.
        NIXL_WARN << "NVLINK backend: agent " << remote_agent << " runs on host " << p.host
                  << "; this backend reaches peers of one NVLink box only (the TCP backend reaches other hosts)";
        return NIXL_ERR_NOT_SUPPORTED;
    }
    std::lock_guard<std::mutex> g(peersMu_);
    peers_[remote_agent] = std::make_shared<const PeerId>(std::move(p));
    ++peersGen_;
    return NIXL_SUCCESS;
}

std::shared_ptr<const PeerId> Engine::findPeer(const std::string &agent, uint64_t *gen) const {
    std::lock_guard<std::mutex> g(peersMu_);
    if (gen) *gen = peersGen_.load(std::memory_order_relaxed);
    auto it = peers_.find(agent);
    return it == peers_.end() ? nullptr : it->second;
}

nixl_status_t Engine::connect(const std::string &remote_agent) {
    if (remote_agent == self_.agent) {
        std::lock_guard<std::mutex> g(peersMu_);
        peers_[remote_agent] = std::make_shared<const PeerId>(self_);
        ++peersGen_;
        return NIXL_SUCCESS;
    }
    auto p = findPeer(remote_agent);
    if (!p) return NIXL_ERR_NOT_FOUND;
    return peerAlive(*p, true) ? NIXL_SUCCESS : NIXL_ERR_REMOTE_DISCONNECT;
}

nixl_status_t Engine::disconnect(const std::string &remote_agent) {
    std::lock_guard<std::mutex> g(peersMu_);
    ++peersGen_;
    return peers_.erase(remote_agent) ? NIXL_SUCCESS : NIXL_ERR_NOT_FOUND;
}

nixl_status_t Engine::loadRemoteMD(const nixlBlobDesc &input, const nixl_mem_t &nixl_mem, const std::string &remote_agent,
                                   nixlBackendMD *&output) {
    if (input.metaInfo.size() < sizeof(PubReg)) return NIXL_ERR_MISMATCH;
    PubReg pub;
    std::memcpy(&pub, input.metaInfo.data(), sizeof(pub));
    if (pub.version != kPubVersion || pub.mem != static_cast<uint8_t>(nixl_mem)) return NIXL_ERR_MISMATCH;
    auto peerp = findPeer(remote_agent);
    if (!peerp) return NIXL_ERR_NOT_FOUND;
    const PeerId &peer = *peerp;
    auto md = std::make_unique<RemoteMD>();
    md->agent = remote_agent;
    md->mem = nixl_mem;
    md->addr = pub.addr;
    md->len = pub.len;
    md->ownerDevice = pub.device;
    md->ownerPid = peer.pid;
    md->sameProcess = peer.pid == self_.pid && peer.procTag == self_.procTag;
    if (md->sameProcess) {
        if (nixl_mem == VRAM_SEG) {
            md->devVisible = pub.addr;
            md->ownerLocalDevice = pub.device;
        } else if (cuda_) {
            void *dp = nullptr; // pinned by its owner? then kernels can touch it
            if (cudaHostGetDevicePointer(&dp, reinterpret_cast<void *>(pub.addr), 0) == cudaSuccess)
                md->devVisible = reinterpret_cast<uintptr_t>(dp);
            else cudaGetLastError();
        }
    } else if (nixl_mem == VRAM_SEG && cuda_ && pub.hasIpc == 1) {
        const std::string key(reinterpret_cast<const char *>(pub.ipc), sizeof(pub.ipc));
        std::lock_guard<std::mutex> g(g_ipcMu);
        IpcMapping &m = g_ipc[key];
        if (!m.base) {
            int dev = primaryDevice_.load();
            if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) dev = 0;
            DeviceScope ds(dev);
            cudaIpcMemHandle_t h;
            std::memcpy(&h, pub.ipc, sizeof(h));
            void *base = nullptr;
            if (!cudaOk(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) {
                g_ipc.erase(key);
                return NIXL_ERR_BACKEND;
            }
            m.base = base;
            m.device = dev;
            // Which of THIS process's ordinals owns the memory (the exporter may number its GPUs
            // differently): kernels launched from any other local GPU need peer access to it, and
            // a copy between two GPUs is routed differently from one inside a GPU.
            m.ownerLocal = ordinalOfUuid(pub.gpuUuid, deviceCount_);
        }
        ++m.refs;
        md->ipcKey = key;
        md->mapDevice = m.device;
        md->ownerLocalDevice = m.ownerLocal;
        md->devVisible = reinterpret_cast<uintptr_t>(m.base) + pub.ipcOffset;
    } else if (nixl_mem == VRAM_SEG && cuda_ && pub.hasIpc == 2) {
        // VMM memory of another process: fetch its allocations' descriptors and map them here.
        const char *tail = input.metaInfo.data() + sizeof(PubReg);
        const size_t left = input.metaInfo.size() - sizeof(PubReg);
        uint32_t n = 0;
        if (left < sizeof(n)) return NIXL_ERR_MISMATCH;
        std::memcpy(&n, tail, sizeof(n));
        if (n == 0 || left < sizeof(n) + size_t(n) * sizeof(PubVmmChunk)) return NIXL_ERR_MISMATCH;
        std::vector<VmmChunk> chunks(n);
        std::vector<int> numbers(n);
        for (uint32_t i = 0; i < n; ++i) {
            PubVmmChunk w;
            std::memcpy(&w, tail + sizeof(n) + size_t(i) * sizeof(w), sizeof(w));
            chunks[i] = {w.base, w.size, -1};
            numbers[i] = w.fd;
        }
        int dev = primaryDevice_.load();
        if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) dev = 0;
        DeviceScope ds(dev);
        cudaFree(nullptr); // make sure the device has a context before driver calls
        const int owner_local = ordinalOfUuid(pub.gpuUuid, deviceCount_);
        const std::vector<int> fds = vmmFetchFds(peer.sockName + ".fd", numbers);
        if (fds.size() != n || !vmmMap(chunks, fds, deviceCount_, owner_local, md->vmmMap)) {
            NIXL_ERROR << "NVLINK backend: cannot map the VMM memory of agent " << remote_agent
                       << " (its allocations must be created with the POSIX file-descriptor handle type)";
            return NIXL_ERR_BACKEND;
        }
        md->mapDevice = dev;
        md->ownerLocalDevice = owner_local;
        md->devVisible = static_cast<uintptr_t>(md->vmmMap.va) + static_cast<uintptr_t>(pub.addr - chunks.front().base);
    }
    output = md.release();
    return NIXL_SUCCESS;
}

nixl_status_t Engine::loadLocalMD(nixlBackendMD *input, nixlBackendMD *&output) {
    auto *l = dynamic_cast<LocalMD *>(input);
    if (!l) return NIXL_ERR_INVALID_PARAM;
    auto md = std::make_unique<RemoteMD>();
    md->agent = self_.agent;
    md->mem = l->mem;
    md->addr = l->addr;
    md->len = l->len;
    md->ownerDevice = l->device;
    md->ownerLocalDevice = l->device; // the agent's own memory: copies between two of its buffers on one GPU stay on the copy kernel
    md->ownerPid = self_.pid;
    md->sameProcess = true;
    md->devVisible = l->devVisible;
    md->loopback = true;
    output = md.release();
    return NIXL_SUCCESS;
}

nixl_status_t Engine::unloadMD(nixlBackendMD *input) {
    auto *md = dynamic_cast<RemoteMD *>(input);
    if (!md) return NIXL_ERR_INVALID_PARAM;
    if (md->vmmMap.va != 0) {
        DeviceScope ds(md->mapDevice);
        vmmUnmap(md->vmmMap);
    }
    if (!md->ipcKey.empty()) {
        std::lock_guard<std::mutex> g(g_ipcMu);
        auto it = g_ipc.find(md->ipcKey);
        if (it != g_ipc.end() && --it->second.refs == 0) {
            DeviceScope ds(it->second.device);
            if (cudaIpcCloseMemHandle(it->second.base) != cudaSuccess) cudaGetLastError();
            g_ipc.erase(it);
        }
    }
    delete md;
    return NIXL_SUCCESS;
}

// ================================================================ transfers

void Engine::freeBatch(KernelBatch &b) const {
    DeviceCtx *c = ctx(b.device);
    if (!c) return;
    if (b.table) c->arena->free(b.table);
    c->counters->release(b.counter);
    if (b.uploaded) {
        DeviceScope ds(b.device);
        cudaEventDestroy(b.uploaded);
    }
    c->flags.release(b.flag);
    b.table = nullptr;
    b.counter = nullptr;
    b.uploaded = nullptr;
    b.flag = nullptr;
}

// Frees a request whatever state it is in.  A launched copy kernel still reads the request's
// descriptor table and writes its counter and completion word, on whichever stream it was
// posted (the engine's or the caller's), so the completion word itself is what is waited on;
// only if it does not turn within ten seconds is the whole device synchronised instead.
void Engine::destroyReq(ReqH *req) const {
    {
        std::lock_guard<std::mutex> g(req->mu);
        for (auto &b : req->kernels) {
            if (b.inFlight && b.flag) {
                const auto t0 = std::chrono::steady_clock::now();
                bool done = false;
                for (uint32_t spins = 0;; ++spins) {
                    const uint64_t v = loadWord(b.flag);
                    if (b.viaProxy ? proxyDone(nullptr, b) != 0 : (v & 0x7fffffffffffffffull) == b.seq) {
                        done = true;
                        break;
                    }
                    if ((spins & 1023u) == 1023u) {
                        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(10)) break;
                        std::this_thread::yield();
                    }
                }
                if (!done) {
                    NIXL_ERROR << "NVLINK backend: a released request's copy on GPU " << b.device << " did not complete within 10 s ("
                               << (b.viaProxy ? "doorbell proxy" : "copy kernel") << "); waiting for the whole device";
                    DeviceScope ds(b.device);
                    const cudaError_t e = cudaDeviceSynchronize();
                    if (e != cudaSuccess) {
                        NIXL_ERROR << "NVLINK backend: cudaDeviceSynchronize: " << cudaGetErrorString(e);
                        cudaGetLastError();
                    }
                }
                b.inFlight = false;
            }
            freeBatch(b);
        }
        for (auto &e : req->asyncEvents) {
            DeviceScope ds(e.first);
            if (req->asyncInFlight) cudaEventSynchronize(e.second);
            cudaEventDestroy(e.second);
        }
    }
    delete req;
}

nixl_status_t Engine::prepXfer(const nixl_xfer_op_t &operation, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote,
                               const std::string &remote_agent, nixlBackendReqH *&handle, const nixl_opt_b_args_t *) const {
    if (local.descCount() != remote.descCount() || local.isEmpty()) return NIXL_ERR_INVALID_PARAM;
    ReqH *req = new ReqH();
    // Every early return hands back what the request already holds (completion words, arena blocks, events).
    auto fail = [&](nixl_status_t st) {
        destroyReq(req);
        return st;
    };
    req->op = operation;
    req->remoteAgent = remote_agent;
    req->peer = findPeer(remote_agent, &req->peerGen);
    struct Item {
        XferDesc d;
        uint64_t klass; // 1: both ends are VRAM of different GPUs
    };
    std::map<int, std::vector<Item>> perDevice;

    for (int i = 0; i < local.descCount(); ++i) {
        auto *l = dynamic_cast<LocalMD *>(local[i].metadataP);
        auto *r = dynamic_cast<RemoteMD *>(remote[i].metadataP);
        if (!l || !r || local[i].len != remote[i].len) return fail(NIXL_ERR_INVALID_PARAM);
        const size_t len = local[i].len;
        if (len == 0) continue;
        req->totalBytes += len;
        const uintptr_t laddr = local[i].addr, raddr = remote[i].addr;
        // Kernel-visible addresses of both ends, when they exist.
        const uintptr_t lvis = l->devVisible ? l->devVisible + (laddr - l->addr) : 0;
        const uintptr_t rvis = r->devVisible ? r->devVisible + (raddr - r->addr) : 0;
        const bool any_vram = l->mem == VRAM_SEG || r->mem == VRAM_SEG;

        if (!any_vram) { // DRAM <-> DRAM: the CPU moves it
            if (r->sameProcess) {
                if (operation == NIXL_WRITE) req->hostCopies.push_back({reinterpret_cast<void *>(raddr), reinterpret_cast<void *>(laddr), len});
                else req->hostCopies.push_back({reinterpret_cast<void *>(laddr), reinterpret_cast<void *>(raddr), len});
            } else {
                req->cmaCopies.push_back({laddr, raddr, len});
                req->cmaPid = r->ownerPid;
            }
            continue;
        }
        if (!cuda_) return fail(NIXL_ERR_NOT_SUPPORTED);
        if (lvis && rvis) { // the copy kernel can see both ends
            int dev;
            if (l->mem == VRAM_SEG) dev = l->device;
            else dev = r->sameProcess ? r->ownerDevice : r->mapDevice;
            if (dev < 0) return fail(NIXL_ERR_BACKEND);
            // The launching GPU needs peer access to the GPU that owns the remote memory.  For
            // another process's memory the IPC mapping enabled it for the device that opened the
            // handle only; a process driving several GPUs launches from others too.
            if (r->mem == VRAM_SEG && r->ownerLocalDevice >= 0 && !ensurePeerAccess(dev, r->ownerLocalDevice)) {
                NIXL_ERROR << "NVLINK backend: GPU " << dev << " cannot access GPU " << r->ownerLocalDevice;
                return fail(NIXL_ERR_NOT_SUPPORTED);
            }
            XferDesc d;
            d.src = operation == NIXL_WRITE ? lvis : rvis;
            d.dst = operation == NIXL_WRITE ? rvis : lvis;
            d.len = len;
            // Neighbours in the list that continue each other on both sides become one descriptor
            // (a buffer posted as consecutive blocks is one long copy: fewer table entries for
            // the kernel, one copy instead of many for the copy engines).
            // (A GPU this process cannot name is certainly not the local one.)
            const bool cross_gpu = l->mem == VRAM_SEG && r->mem == VRAM_SEG && r->ownerLocalDevice != l->device;
            auto &list = perDevice[dev];
            const uint64_t klass = cross_gpu ? 1 : 0; // never merge across kinds of path
            if (coalesce_ && !list.empty() && list.back().d.src + list.back().d.len == d.src && list.back().d.dst + list.back().d.len == d.dst &&
                list.back().klass == klass)
                list.back().d.len += d.len;
            else list.push_back({d, klass});
            continue;
        }
        // One end is pageable host memory: let the runtime stage it.
        if (l->mem == DRAM_SEG && rvis) {
            const int dev = r->sameProcess ? r->ownerDevice : r->mapDevice;
            if (operation == NIXL_WRITE) req->asyncCopies.push_back({reinterpret_cast<void *>(rvis), reinterpret_cast<void *>(laddr), len, dev});
            else req->asyncCopies.push_back({reinterpret_cast<void *>(laddr), reinterpret_cast<void *>(rvis), len, dev});
            continue;
        }
        if (l->mem == VRAM_SEG && r->mem == DRAM_SEG && r->sameProcess) {
            if (operation == NIXL_WRITE) req->asyncCopies.push_back({reinterpret_cast<void *>(raddr), reinterpret_cast<void *>(lvis), len, l->device});
            else req->asyncCopies.push_back({reinterpret_cast<void *>(lvis), reinterpret_cast<void *>(raddr), len, l->device});
            continue;
        }
        NIXL_ERROR << "NVLINK backend: no path between local " << nixlEnumStrings::memTypeStr(l->mem) << " and remote "
                   << nixlEnumStrings::memTypeStr(r->mem) << " of agent " << remote_agent
                   << (r->sameProcess ? "" : " (other process; its VRAM must be exportable device memory, its DRAM is reachable from DRAM only)");
        return fail(NIXL_ERR_NOT_SUPPORTED);
    }

    for (auto &kv : perDevice) {
        DeviceCtx *c = ctx(kv.first);
        if (!c) return fail(NIXL_ERR_BACKEND);
        req->kernels.emplace_back();
        KernelBatch &b = req->kernels.back(); // owned by the request from here on: fail() frees it
        b.device = kv.first;
        // Copy engines only where they beat the kernel: long copies between two GPUs.  Measured on
        // NVLink 5 with both directions busy: one copy-engine copy runs at 774 GB/s but costs about
        // 7.5 us to start and drain, the kernel moves a whole batch in one launch at 703 GB/s; they
        // break even near 64 MiB per descriptor.  Inside one GPU's HBM the kernel is faster
        // (3.2 against 2.6 TB/s).
        for (const Item &it : kv.second) {
            const bool ce = ceThreshold_ > 0 && it.d.len >= ceThreshold_ && (it.klass == 1 || copyPath_ == CopyPath::COPY_ENGINE);
            (ce ? b.ceDescs : b.descs).push_back(it.d);
        }
        b.stream = c->streams[c->nextStream.fetch_add(1, std::memory_order_relaxed) % c->streams.size()];
        uint64_t total = 0, longest = 0;
        for (auto &d : b.descs) {
            total += d.len;
            longest = std::max<uint64_t>(longest, d.len);
        }
        // Chunk size: aim at ~2 chunks per CTA that can be resident at once (two per SM), between
        // 16 KiB and 256 KiB.  The grid itself may be several times larger (see defaultGridCtas): a
        // large copy then runs as many short-lived CTAs whose tail balances itself.
        const uint64_t resident = std::min<uint64_t>(static_cast<uint64_t>(c->gridCtas), 2 * static_cast<uint64_t>(c->smCount));
        uint32_t shift = log2Ceil(std::max<uint64_t>(1, total / (2 * std::max<uint64_t>(1, resident))));
        shift = std::min<uint32_t>(18, std::max<uint32_t>(14, shift));
        const size_t n = b.descs.size();
        // Small kernel-only batches may go through the doorbell proxy, whose unit of work is a warp: 4 KiB chunks.
        b.proxyEligible = proxyEnabled_ && copyPath_ == CopyPath::VECTOR && b.ceDescs.empty() && n >= 1 && n <= kProxyMaxDescs && total <= proxyMaxBytes_;
        if (b.proxyEligible) shift = 12;
        if (chunkShiftOverride_ >= 12 && chunkShiftOverride_ <= 22) shift = static_cast<uint32_t>(chunkShiftOverride_);
        std::vector<uint32_t> starts(n + 1);
        uint64_t chunks = 0;
        uint64_t per = 0; // chunks per descriptor when all descriptors have the same number, else 0
        for (size_t i = 0; i < n; ++i) {
            starts[i] = static_cast<uint32_t>(chunks);
            const uint64_t mine = (b.descs[i].len + (uint64_t(1) << shift) - 1) >> shift;
            per = i == 0 ? mine : (per == mine ? per : 0);
            chunks += mine;
            if (chunks > 0x7fffffffull) return fail(NIXL_ERR_INVALID_PARAM); // cannot happen below 2^31 * 16 KiB, but stay safe
        }
        b.uniformChunks = per <= kProxyMaxPer ? static_cast<uint32_t>(per) : 0;
        starts[n] = static_cast<uint32_t>(chunks);
        b.launch.nDescs = static_cast<uint32_t>(n);
        b.launch.totalChunks = static_cast<uint32_t>(chunks);
        b.launch.chunkShift = shift;
        b.flag = c->flags.acquire();
        if (!b.flag) return fail(NIXL_ERR_BACKEND);
        b.launch.hostFlag = b.flag; // UVA: the pinned allocation's host address is device-visible
        b.counter = c->counters->acquire();
        if (!b.counter) return fail(NIXL_ERR_BACKEND);
        b.launch.doneCounter = b.counter;
        if (n == 1) b.single = b.descs[0];
        const bool inline_ok = n <= static_cast<size_t>(kInlineDescs);
        if (inline_ok) {
            b.launch.table = nullptr;
            b.launch.chunkStart = nullptr;
            for (size_t i = 0; i < n; ++i) b.launch.inl[i] = b.descs[i];
            for (size_t i = 0; i <= n; ++i) b.launch.inlStart[i] = starts[i];
        }
        // A device table for batches too long for the launch parameters, and for any batch of
        // several descriptors that may go through the proxy (a proxy command has room for one).
        if (!inline_ok || (b.proxyEligible && n > 1)) {
            const size_t tbytes = n * sizeof(XferDesc), sbytes = (n + 1) * sizeof(uint32_t);
            const size_t toff = 0, soff = (tbytes + 15) & ~size_t(15);
            b.table = c->arena->alloc(soff + sbytes);
            if (!b.table) return fail(NIXL_ERR_BACKEND);
            DeviceScope ds(b.device);
            char *base = static_cast<char *>(b.table);
            // Pageable source: the runtime copies it out before returning, so the vectors may die.
            bool ok = cudaOk(cudaMemcpyAsync(base + toff, b.descs.data(), tbytes, cudaMemcpyHostToDevice, c->prepStream), "table upload");
            ok = ok && cudaOk(cudaMemcpyAsync(base + soff, starts.data(), sbytes, cudaMemcpyHostToDevice, c->prepStream), "table upload");
            ok = ok && cudaOk(cudaEventCreateWithFlags(&b.uploaded, cudaEventDisableTiming), "cudaEventCreate");
            ok = ok && cudaOk(cudaEventRecord(b.uploaded, c->prepStream), "cudaEventRecord");
            if (!ok) return fail(NIXL_ERR_BACKEND);
            b.tableDev = reinterpret_cast<const XferDesc *>(base + toff);
            b.startsDev = reinterpret_cast<const uint32_t *>(base + soff);
            if (!inline_ok) {
                b.launch.table = b.tableDev;
                b.launch.chunkStart = b.startsDev;
            }
        }
        NIXL_DEBUG << "NVLINK backend: request to " << remote_agent << " on GPU " << b.device << ": " << n << " descriptor(s) for the copy kernel ("
                   << chunks << " chunks of " << (1u << shift) << " bytes), " << b.ceDescs.size() << " for the copy engines";
        // The host copy of the kernel's descriptors has served its purpose (they sit in the launch
        // parameters or in the device table).
        std::vector<XferDesc>().swap(b.descs);
    }
    for (auto &a : req->asyncCopies) {
        bool have = false;
        for (auto &e : req->asyncEvents) have |= e.first == a.device;
        if (have) continue;
        if (!ctx(a.device)) return fail(NIXL_ERR_BACKEND);
        DeviceScope ds(a.device);
        cudaEvent_t ev = nullptr;
        if (!cudaOk(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate")) return fail(NIXL_ERR_BACKEND);
        req->asyncEvents.emplace_back(a.device, ev);
    }
    handle = req;
    return NIXL_SUCCESS;
}

// ---------------------------------------------------------------- doorbell proxy, host side

// Starts the proxy kernel when commands are pending and none is alive.  `launched` stays true until
// this side has SEEN the exit word; a kernel that has just left is therefore noticed by the next
// post or poll, and the new launch queues behind it on the proxy's stream.
void Engine::proxyEnsureRunning(DeviceCtx *c, Proxy &px) const {
    if (px.broken) return;
    if (px.launched) {
        const uint64_t w = loadWord(px.exitWord);
        if (w == 0) return;
        px.launched = false;
        px.nextStart = w & ~(1ull << 63);
    }
    if (px.nextStart >= px.posted) return; // nothing pending
    storeWord(px.exitWord, 0);
    ProxyLaunch pl{};
    pl.hostRing = px.hostRing;
    pl.shared = px.shared;
    pl.done = px.done;
    pl.exitWord = px.exitWord;
    pl.start = px.nextStart;
    pl.gen = ++px.launches;
    pl.idleNs = proxyIdleNs_;
    pl.lifeNs = proxyLifeNs_;
    DeviceScope ds(c->device);
    if (!cudaOk(launchProxy(pl, proxyWorkers_, px.stream), "proxy kernel launch")) {
        // Commands already written stay unserved: mark them so that their requests fail over.
        px.broken = true;
        return;
    }
    g_kernelLaunches.fetch_add(1, std::memory_order_relaxed);
    px.launched = true;
}

bool Engine::postViaProxy(DeviceCtx *c, KernelBatch &b) const {
    if (b.launch.nDescs > 1) {
        if (!b.tableDev) return false;
        if (!b.tableReady) { // the table upload of prepXfer must have landed; seen once, remembered
            if (b.uploaded && cudaEventQuery(b.uploaded) != cudaSuccess) {
                cudaGetLastError();
                return false;
            }
            b.tableReady = true;
        }
    }
    if (!c->proxy) {
        std::lock_guard<std::mutex> g(ctxMu_);
        if (!c->proxy) {
            auto px = std::make_unique<Proxy>();
            DeviceScope ds(c->device);
            const size_t ring_bytes = kProxySlots * sizeof(ProxyCmd), done_bytes = kProxySlots * sizeof(uint64_t);
            bool ok = cudaOk(cudaHostAlloc(&px->pinned, ring_bytes + done_bytes + 64, cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc(proxy)");
            ok = ok && cudaOk(cudaMalloc(reinterpret_cast<void **>(&px->shared), sizeof(ProxyShared)), "cudaMalloc(proxy)");
            ok = ok && cudaOk(cudaMemset(px->shared, 0, sizeof(ProxyShared)), "cudaMemset(proxy)");
            ok = ok && cudaOk(cudaStreamCreateWithFlags(&px->stream, cudaStreamNonBlocking), "cudaStreamCreate(proxy)");
            if (ok) {
                std::memset(px->pinned, 0, ring_bytes + done_bytes + 64);
                px->hostRing = static_cast<ProxyCmd *>(px->pinned);
                px->done = reinterpret_cast<uint64_t *>(static_cast<char *>(px->pinned) + ring_bytes);
                px->exitWord = reinterpret_cast<uint64_t *>(static_cast<char *>(px->pinned) + ring_bytes + done_bytes);
            } else {
                px->broken = true;
            }
            c->proxy = std::move(px);
        }
    }
    Proxy &px = *c->proxy;
    std::lock_guard<std::mutex> g(px.mu);
    if (px.broken) return false;
    const uint64_t n = px.posted;
    const uint32_t slot = static_cast<uint32_t>(n % kProxySlots);
    // The slot's previous command (one ring ago) must be complete: its workers are past it.
    if (n >= kProxySlots && loadWord(px.done + slot) < n - kProxySlots + 1) return false;
    ProxyCmd *h = px.hostRing + slot;
    if (b.launch.nDescs == 1) {
        h->b = b.single.dst;
        h->c = proxyPackC(n + 1, kProxyInline, b.launch.chunkShift, b.single.len);
        h->a = b.single.src;
    } else {
        h->b = reinterpret_cast<uint64_t>(b.startsDev);
        h->c = proxyPackC(n + 1, kProxyTable, b.launch.chunkShift, (uint64_t(b.uniformChunks) << 24) | b.launch.nDescs);
        h->a = reinterpret_cast<uint64_t>(b.tableDev);
    }
    __atomic_store_n(&h->seq, n + 1, __ATOMIC_RELEASE); // the doorbell: written last
    px.posted = n + 1;
    b.viaProxy = true;
    b.proxy = &px;
    b.proxyCmd = n;
    b.inFlight = true;
    proxyEnsureRunning(c, px); // a failed launch marks the proxy broken; the request then reports it when polled
    return true;
}

int Engine::proxyDone(DeviceCtx *c, KernelBatch &b) const {
    Proxy &px = *b.proxy;
    const uint64_t v = loadWord(px.done + (b.proxyCmd % kProxySlots));
    if (v >= b.proxyCmd + 1) {
        std::atomic_thread_fence(std::memory_order_acquire);
        return 1;
    }
    if (px.broken.load(std::memory_order_relaxed)) return -1;
    // Not done: if the kernel has left (idle or end of life) with this command pending, start it again.
    if (loadWord(px.exitWord) != 0) {
        if (!c) c = ctx(b.device);
        std::lock_guard<std::mutex> g(px.mu);
        proxyEnsureRunning(c, px);
    }
    return 0;
}

// Liveness of a peer, host side only.  Same process: the engine registry.  Other process:
// kill(pid, 0); callers on the post path pass force = false unless their last look is older
// than a millisecond, so a stream of small posts does not pay a system call each.
bool Engine::peerAlive(const PeerId &peer, bool force) const {
    if (peer.engineTag == self_.engineTag) return true;
    if (peer.pid == self_.pid && peer.procTag == self_.procTag) {
        std::lock_guard<std::mutex> g(g_regMu);
        auto it = g_registry.find(peer.agent);
        return it != g_registry.end() && it->second->engineTag() == peer.engineTag;
    }
    if (!force) return true;
    if (::kill(static_cast<pid_t>(peer.pid), 0) != 0 && errno == ESRCH) return false;
    if (livenessPing_) {
        socklen_t alen = 0;
        sockaddr_un addr = abstractAddr(peer.sockName, alen);
        if (::sendto(notifFd_, "", 0, MSG_DONTWAIT | MSG_NOSIGNAL, reinterpret_cast<sockaddr *>(&addr), alen) != 0 &&
            (errno == ECONNREFUSED || errno == ENOENT))
            return false;
    }
    return true;
}

nixl_status_t Engine::postXfer(const nixl_xfer_op_t &operation, const nixl_meta_dlist_t &, const nixl_meta_dlist_t &,
                               const std::string &remote_agent, nixlBackendReqH *&handle, const nixl_opt_b_args_t *opt_args) const {
    auto *req = dynamic_cast<ReqH *>(handle);
    if (!req || req->op != operation) return NIXL_ERR_INVALID_PARAM;

    std::unique_lock<std::mutex> lk(req->mu);
    // Whatever goes wrong below, the request records it: kernels launched before the failure
    // stay marked in flight and are waited for when the request is released.
    auto fail = [&](nixl_status_t st) {
        req->last = st;
        return st;
    };
    if (!req->peer || req->peerGen != peersGen_.load(std::memory_order_acquire)) {
        req->peer = findPeer(remote_agent, &req->peerGen);
        if (!req->peer) return fail(NIXL_ERR_NOT_FOUND);
    }
    const int64_t now_ns = static_cast<int64_t>(nixl_util::FastClock::ns()); // one stamp per post: the cycle counter
    const bool look = livenessPing_ || now_ns - req->lastAliveNs > 1000000;
    if (look) req->lastAliveNs = now_ns;
    if (!peerAlive(*req->peer, look)) return fail(NIXL_ERR_REMOTE_DISCONNECT);

    req->notifPending = opt_args && opt_args->hasNotif;
    if (req->notifPending) req->notifMsg = opt_args->notifMsg;

    // Optional stream-ordered posting: customParam "stream=<address of a cudaStream_t value>".
    cudaStream_t user_stream = nullptr;
    bool has_user_stream = false;
    if (opt_args && opt_args->customParam.rfind("stream=", 0) == 0) {
        user_stream = reinterpret_cast<cudaStream_t>(std::strtoull(opt_args->customParam.c_str() + 7, nullptr, 0));
        has_user_stream = true;
    }

    for (auto &h : req->hostCopies) std::memcpy(h.dst, h.src, h.len);

    if (!req->cmaCopies.empty()) {
        constexpr size_t kBatch = 512;
        iovec liov[kBatch], riov[kBatch];
        size_t i = 0;
        while (i < req->cmaCopies.size()) {
            size_t n = 0, want = 0;
            for (; n < kBatch && i + n < req->cmaCopies.size(); ++n) {
                const CmaCopy &cc = req->cmaCopies[i + n];
                liov[n] = {reinterpret_cast<void *>(cc.local), cc.len};
                riov[n] = {reinterpret_cast<void *>(cc.remote), cc.len};
                want += cc.len;
            }
            const ssize_t got = operation == NIXL_WRITE
                ? ::process_vm_writev(static_cast<pid_t>(req->cmaPid), liov, n, riov, n, 0)
                : ::process_vm_readv(static_cast<pid_t>(req->cmaPid), liov, n, riov, n, 0);
            if (got < 0 || static_cast<size_t>(got) != want) {
                if (errno == ESRCH) return fail(NIXL_ERR_REMOTE_DISCONNECT);
                NIXL_ERROR << "NVLINK backend: cross-process DRAM copy failed: " << std::strerror(errno);
                return fail(NIXL_ERR_BACKEND);
            }
            i += n;
        }
    }

    if (!req->kernels.empty() || !req->asyncCopies.empty()) {
        int cur = -1;
        if (cudaGetDevice(&cur) != cudaSuccess) cur = -1;
        int active = cur;
        auto use = [&](int dev) {
            if (dev != active) {
                cudaSetDevice(dev);
                active = dev;
            }
        };
        nixl_status_t err = NIXL_SUCCESS;
        for (auto &b : req->kernels) {
            DeviceCtx *c = ctx(b.device);
            if (!c) {
                err = NIXL_ERR_BACKEND;
                break;
            }
            b.viaProxy = false;
            // A request that is one kernel batch and nothing else lets the kernel's tail release the
            // notification itself (notif_ring.h); such a request skips the doorbell proxy, whose
            // commands have no room for it.
            std::shared_ptr<NotifRingWriter> ring;
            b.notifWord = nullptr;
            b.launch.notifWord = nullptr;
            if (req->notifPending && req->kernels.size() == 1 && req->hostCopies.empty() && req->cmaCopies.empty() && req->asyncCopies.empty() &&
                (ring = ringOf(*req->peer)) && ring->claim(self_.agent, req->notifMsg, &b.notifWord, &b.notifSeq)) {
                b.launch.notifWord = ring->deviceWord(b.notifWord);
                b.launch.notifSeq = b.notifSeq;
            }
            if (!b.notifWord && b.proxyEligible && !has_user_stream && postViaProxy(c, b)) continue; // no CUDA call on this path
            use(b.device);
            cudaStream_t s = has_user_stream ? user_stream : b.stream;
            if (b.uploaded && !b.tableReady && b.launch.table && !cudaOk(cudaStreamWaitEvent(s, b.uploaded, 0), "cudaStreamWaitEvent")) {
                if (b.notifWord) NotifRingWriter::complete(b.notifWord, b.notifSeq, false); // claimed above, never to be released by a kernel
                b.notifWord = nullptr;
                err = NIXL_ERR_BACKEND;
                break;
            }
            uint64_t seq = (b.seq + 1) & 0x7fffffffffffffffull;
            if (seq == 0) seq = 1;
            b.launch.seq = seq;
            // Large descriptors first, on the copy engines; then the kernel for the rest, whose tail
            // publishes the completion word (stream order puts it behind the copies).  Without
            // kernel work a one-thread kernel publishes it.
            bool ok = true;
            for (const XferDesc &d : b.ceDescs)
                ok = ok && cudaOk(cudaMemcpyAsync(reinterpret_cast<void *>(d.dst), reinterpret_cast<const void *>(d.src), d.len, cudaMemcpyDefault, s),
                                  "cudaMemcpyAsync");
            const cudaError_t le = b.launch.totalChunks > 0 ? launchBatchCopy(b.launch, c->gridCtas, copyPath_, s)
                                                            : launchSignal(b.launch.hostFlag, seq, b.launch.notifWord, b.launch.notifSeq, s);
            if (!cudaOk(le, "copy kernel launch")) {
                if (b.notifWord) NotifRingWriter::complete(b.notifWord, b.notifSeq, false); // nothing will release the slot: void it
                b.notifWord = nullptr;
                err = NIXL_ERR_BACKEND; // copies queued before stay unreported: the stream is in an error state anyway
                break;
            }
            g_kernelLaunches.fetch_add(1, std::memory_order_relaxed);
            b.seq = seq;
            b.inFlight = true;
            if (b.notifWord) req->notifPending = false; // the kernel delivers it
            if (!ok) {
                err = NIXL_ERR_BACKEND;
                break;
            }
        }
        if (err == NIXL_SUCCESS && !req->asyncCopies.empty()) {
            for (auto &a : req->asyncCopies) {
                DeviceCtx *c = ctx(a.device);
                use(a.device);
                cudaStream_t s = has_user_stream ? user_stream : c->streams[0];
                if (!cudaOk(cudaMemcpyAsync(a.dst, a.src, a.len, cudaMemcpyDefault, s), "cudaMemcpyAsync")) {
                    err = NIXL_ERR_BACKEND;
                    break;
                }
            }
            // Everything queued so far is covered by the events, also after a failed copy.
            for (auto &e : req->asyncEvents) {
                DeviceCtx *c = ctx(e.first);
                use(e.first);
                if (!cudaOk(cudaEventRecord(e.second, has_user_stream ? user_stream : c->streams[0]), "cudaEventRecord")) err = NIXL_ERR_BACKEND;
            }
            req->asyncInFlight = true;
        }
        if (active != cur && cur >= 0) cudaSetDevice(cur);
        if (err != NIXL_SUCCESS) return fail(err);
    }

    nixl_status_t st = pollData(req);
    if (st == NIXL_SUCCESS) st = finishIfDone(req);
    req->last = st;
    const bool watch = st == NIXL_IN_PROG && progThread_ && req->notifPending;
    lk.unlock();
    if (watch) {
        std::lock_guard<std::mutex> g(progMu_);
        progWatch_.push_back(req);
        progCv_.notify_one();
    }
    return st;
}

// Data state only: SUCCESS when every launched piece has completed.
nixl_status_t Engine::pollData(ReqH *req) const {
    for (auto &b : req->kernels) {
        if (!b.inFlight) continue;
        if (b.viaProxy) {
            const int st = proxyDone(nullptr, b);
            if (st == 0) return NIXL_IN_PROG;
            b.inFlight = false;
            if (st < 0) {
                NIXL_ERROR << "NVLINK backend: the doorbell proxy kernel could not be launched";
                return NIXL_ERR_BACKEND;
            }
            continue;
        }
        const uint64_t v = loadWord(b.flag);
        if ((v & 0x7fffffffffffffffull) != b.seq) return NIXL_IN_PROG;
        b.inFlight = false;
        if (v >> 63) {
            NIXL_ERROR << "NVLINK backend: copy kernel reported a lost bulk copy";
            if (b.notifWord) NotifRingWriter::complete(b.notifWord, b.notifSeq, false); // the kernel left the slot alone
            b.notifWord = nullptr;
            return NIXL_ERR_BACKEND;
        }
        b.notifWord = nullptr;
    }
    if (req->asyncInFlight) {
        for (auto &e : req->asyncEvents) {
            const cudaError_t q = cudaEventQuery(e.second);
            if (q == cudaErrorNotReady) {
                cudaGetLastError();
                return NIXL_IN_PROG;
            }
            if (q != cudaSuccess) {
                cudaOk(q, "cudaEventQuery");
                return NIXL_ERR_BACKEND;
            }
        }
        req->asyncInFlight = false;
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    return NIXL_SUCCESS;
}

nixl_status_t Engine::finishIfDone(ReqH *req) const {
    if (!req->notifPending) return NIXL_SUCCESS;
    std::shared_ptr<const PeerId> peer = req->peer;
    if (!peer || req->peerGen != peersGen_.load(std::memory_order_acquire)) {
        peer = findPeer(req->remoteAgent);
        if (!peer) return NIXL_ERR_NOT_FOUND;
    }
    req->notifPending = false;
    return sendNotif(*peer, req->notifMsg);
}

nixl_status_t Engine::checkXfer(nixlBackendReqH *handle) const {
    auto *req = dynamic_cast<ReqH *>(handle);
    if (!req) return NIXL_ERR_INVALID_PARAM;
    std::lock_guard<std::mutex> g(req->mu);
    if (req->last != NIXL_IN_PROG) return req->last;
    nixl_status_t st = pollData(req);
    if (st == NIXL_SUCCESS) st = finishIfDone(req);
    req->last = st;
    return st;
}

nixl_status_t Engine::releaseReqH(nixlBackendReqH *handle) const {
    auto *req = dynamic_cast<ReqH *>(handle);
    if (!req) return NIXL_ERR_INVALID_PARAM;
    {
        std::lock_guard<std::mutex> g(progMu_);
        progWatch_.erase(std::remove(progWatch_.begin(), progWatch_.end(), req), progWatch_.end());
    }
    destroyReq(req);
    return NIXL_SUCCESS;
}

void Engine::progressLoop() {
    std::unique_lock<std::mutex> lk(progMu_);
    while (!progStop_) {
        if (progWatch_.empty()) {
            progCv_.wait_for(lk, std::chrono::milliseconds(50));
            continue;
        }
        for (size_t i = 0; i < progWatch_.size();) {
            ReqH *req = progWatch_[i];
            nixl_status_t st;
            {
                std::lock_guard<std::mutex> g(req->mu);
                st = req->last;
                if (st == NIXL_IN_PROG) {
                    st = pollData(req);
                    if (st == NIXL_SUCCESS) st = finishIfDone(req);
                    req->last = st;
                }
            }
            if (st != NIXL_IN_PROG) progWatch_.erase(progWatch_.begin() + i);
            else ++i;
        }
        lk.unlock();
        if (progDelayUs_) std::this_thread::sleep_for(std::chrono::microseconds(progDelayUs_));
        else std::this_thread::yield();
        lk.lock();
    }
}

nixl_status_t Engine::estimateXferCost(const nixl_xfer_op_t &, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote,
                                       const std::string &, nixlBackendReqH *const &handle, std::chrono::microseconds &duration,
                                       std::chrono::microseconds &err_margin, nixl_cost_t &method, const nixl_opt_args_t *) const {
    // Analytical model: fixed launch/poll latency plus bytes over the slowest link involved.
    double bytes = 0;
    for (const auto &d : local) bytes += static_cast<double>(d.len);
    double gbps = 20.0; // host memcpy
    if (local.getType() == VRAM_SEG && remote.getType() == VRAM_SEG) {
        gbps = 700.0; // NVLink 5, one direction
        if (auto *req = dynamic_cast<ReqH *>(handle))
            if (!req->kernels.empty() && local.descCount() > 0) {
                auto *r = dynamic_cast<RemoteMD *>(remote[0].metadataP);
                if (r && r->sameProcess && r->ownerDevice == req->kernels[0].device) gbps = 2800.0; // same-GPU HBM copy
            }
    } else if (local.getType() == VRAM_SEG || remote.getType() == VRAM_SEG) {
        gbps = 50.0; // PCIe Gen5 x16
    }
    const double us = 6.0 + bytes / (gbps * 1e3);
    duration = std::chrono::microseconds(static_cast<int64_t>(us + 0.5));
    err_margin = std::chrono::microseconds(static_cast<int64_t>(us * 0.25 + 1.0));
    method = nixl_cost_t::ANALYTICAL_BACKEND;
    return NIXL_SUCCESS;
}

// ================================================================ notifications

namespace {
void unregisterRingMapping(void *base) {
    if (cudaHostUnregister(base) != cudaSuccess) cudaGetLastError();
}
} // namespace

// The peer's notification ring, mapped into this process and registered with CUDA so that a
// kernel can store into it.  nullptr: the peer has none, or it cannot be mapped here (the
// datagram path serves then).
std::shared_ptr<NotifRingWriter> Engine::ringOf(const PeerId &peer) const {
    if (!notifRingEnabled_ || !cuda_ || peer.ringName.empty()) return nullptr;
    std::lock_guard<std::mutex> g(ringMu_);
    auto it = peerRings_.find(peer.ringName);
    if (it != peerRings_.end()) return it->second->devBase.load(std::memory_order_acquire) ? it->second : nullptr;
    std::shared_ptr<NotifRingWriter> w = NotifRingWriter::open(peer.ringName);
    if (!w) {
        NIXL_DEBUG << "NVLINK backend: cannot map the notification ring " << peer.ringName << " of " << peer.agent;
        return nullptr;
    }
    peerRings_[peer.ringName] = w; // also remembers a failed registration: it is not tried again
    if (!w->devBase.load(std::memory_order_acquire) && !w->registerFailed.load(std::memory_order_acquire)) {
        NotifRingWriter::unregisterHook.store(&unregisterRingMapping, std::memory_order_release);
        void *dev = nullptr;
        if (cudaHostRegister(w->base(), w->bytes(), cudaHostRegisterMapped | cudaHostRegisterPortable) == cudaSuccess &&
            cudaHostGetDevicePointer(&dev, w->base(), 0) == cudaSuccess && dev) {
            w->devBase.store(static_cast<char *>(dev), std::memory_order_release);
        } else {
            cudaGetLastError();
            w->registerFailed.store(true, std::memory_order_release);
            NIXL_DEBUG << "NVLINK backend: cannot register the notification ring of " << peer.agent << " with CUDA";
        }
    }
    return w->devBase.load(std::memory_order_acquire) ? w : nullptr;
}

void Engine::pushNotif(const std::string &from, const std::string &msg) {
    std::lock_guard<std::mutex> g(notifMu_);
    inbox_.emplace_back(from, msg);
}

nixl_status_t Engine::sendNotif(const PeerId &peer, const std::string &msg) const {
    if (peer.pid == self_.pid && peer.procTag == self_.procTag) {
        std::lock_guard<std::mutex> g(g_regMu);
        auto it = g_registry.find(peer.agent);
        if (it == g_registry.end() || it->second->engineTag() != peer.engineTag) return NIXL_ERR_REMOTE_DISCONNECT;
        it->second->pushNotif(self_.agent, msg);
        return NIXL_SUCCESS;
    }
    // Payload layout follows the reference's UCX notification (ucx_backend.cpp:1376): name + msg.
    nixlSerDes sd;
    sd.addStr("name", self_.agent);
    sd.addStr("msg", msg);
    const std::string wire = sd.exportStr();
    socklen_t alen = 0;
    sockaddr_un addr = abstractAddr(peer.sockName, alen);
    for (int attempt = 0; attempt < 2000; ++attempt) {
        if (::sendto(notifFd_, wire.data(), wire.size(), MSG_DONTWAIT | MSG_NOSIGNAL, reinterpret_cast<sockaddr *>(&addr), alen) >= 0)
            return NIXL_SUCCESS;
        if (errno == EAGAIN || errno == EWOULDBLOCK || errno == ENOBUFS) { // receiver's queue is full: give it a moment
            std::this_thread::sleep_for(std::chrono::microseconds(100));
            continue;
        }
        if (errno == ECONNREFUSED || errno == ENOENT) return NIXL_ERR_REMOTE_DISCONNECT;
        if (errno == EMSGSIZE) return NIXL_ERR_INVALID_PARAM;
        NIXL_ERROR << "NVLINK backend: notification send failed: " << std::strerror(errno);
        return NIXL_ERR_BACKEND;
    }
    return NIXL_ERR_BACKEND;
}

nixl_status_t Engine::genNotif(const std::string &remote_agent, const std::string &msg) const {
    auto peer = findPeer(remote_agent);
    if (!peer) return NIXL_ERR_NOT_FOUND;
    return sendNotif(*peer, msg);
}

nixl_status_t Engine::getNotifs(notif_list_t &notif_list) {
    std::lock_guard<std::mutex> g(notifMu_);
    for (auto &n : inbox_) notif_list.push_back(std::move(n));
    inbox_.clear();
    if (notifRing_.ok()) notifRing_.poll(notif_list);
    // The receive buffer lives in the engine: this is the target's polling path.
    std::vector<char> &buf = notifBuf_;
    if (buf.empty()) buf.resize(256 * 1024);
    for (;;) {
        const ssize_t n = ::recv(notifFd_, buf.data(), buf.size(), MSG_DONTWAIT | MSG_TRUNC);
        if (n < 0) break;
        if (n == 0) continue; // liveness ping
        if (static_cast<size_t>(n) > buf.size()) { // truncated: grow for the next one, this one is lost
            NIXL_ERROR << "NVLINK backend: dropped an oversized notification (" << n << " bytes)";
            buf.resize(static_cast<size_t>(n));
            continue;
        }
        nixlSerDes sd;
        if (sd.importStr(std::string(buf.data(), static_cast<size_t>(n))) != NIXL_SUCCESS) continue;
        std::string from = sd.getStr("name");
        std::string msg = sd.getStr("msg");
        if (!from.empty()) notif_list.emplace_back(std::move(from), std::move(msg));
    }
    return NIXL_SUCCESS;
}

// ================================================================ memory views

namespace {
std::mutex g_viewMu;
std::unordered_map<void *, MemViewHost> g_views;

nixl_status_t buildView(const Engine *owner, const std::vector<nixlMemViewEntry> &entries, uint32_t kind, nixlMemViewH &mvh) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return NIXL_ERR_BACKEND;
    }
    const size_t bytes = sizeof(nixlMemViewHeader) + entries.size() * sizeof(nixlMemViewEntry);
    std::vector<char> host(bytes);
    auto *hdr = reinterpret_cast<nixlMemViewHeader *>(host.data());
    hdr->magic = NIXL_MEMVIEW_MAGIC;
    hdr->count = static_cast<uint32_t>(entries.size());
    hdr->kind = kind;
    std::memcpy(host.data() + sizeof(nixlMemViewHeader), entries.data(), entries.size() * sizeof(nixlMemViewEntry));
    void *d = nullptr;
    if (!cudaOk(cudaMalloc(&d, bytes), "cudaMalloc(view)")) return NIXL_ERR_BACKEND;
    if (!cudaOk(cudaMemcpy(d, host.data(), bytes, cudaMemcpyHostToDevice), "view upload")) {
        cudaFree(d);
        return NIXL_ERR_BACKEND;
    }
    std::lock_guard<std::mutex> g(g_viewMu);
    g_views[d] = MemViewHost{NIXL_MEMVIEW_MAGIC, owner, d, dev};
    mvh = d;
    return NIXL_SUCCESS;
}
} // namespace

nixl_status_t Engine::prepMemView(const nixl_remote_meta_dlist_t &dlist, nixlMemViewH &mvh, const nixl_opt_b_args_t *) const {
    if (!cuda_) return NIXL_ERR_NOT_SUPPORTED;
    int dev = 0;
    cudaGetDevice(&dev);
    std::vector<nixlMemViewEntry> entries;
    for (const auto &d : dlist) {
        nixlMemViewEntry e{0, 0};
        if (d.remoteAgent != nixl_null_agent) {
            auto *r = dynamic_cast<RemoteMD *>(d.metadataP);
            if (!r || !r->devVisible) return NIXL_ERR_NOT_SUPPORTED;
            if (r->mem == VRAM_SEG && r->ownerLocalDevice >= 0 && !ensurePeerAccess(dev, r->ownerLocalDevice)) return NIXL_ERR_NOT_SUPPORTED;
            e.ptr = r->devVisible + (d.addr - r->addr);
            e.len = d.len;
        }
        entries.push_back(e);
    }
    return buildView(this, entries, NIXL_MEMVIEW_REMOTE, mvh);
}

nixl_status_t Engine::prepMemView(const nixl_meta_dlist_t &dlist, nixlMemViewH &mvh, const nixl_opt_b_args_t *) const {
    if (!cuda_) return NIXL_ERR_NOT_SUPPORTED;
    std::vector<nixlMemViewEntry> entries;
    for (const auto &d : dlist) {
        auto *l = dynamic_cast<LocalMD *>(d.metadataP);
        if (!l || !l->devVisible) return NIXL_ERR_NOT_SUPPORTED;
        entries.push_back({l->devVisible + (d.addr - l->addr), d.len});
    }
    return buildView(this, entries, NIXL_MEMVIEW_LOCAL, mvh);
}

void Engine::releaseMemView(nixlMemViewH mvh) const {
    MemViewHost v{};
    {
        std::lock_guard<std::mutex> g(g_viewMu);
        auto it = g_views.find(mvh);
        if (it == g_views.end() || it->second.owner != this) return;
        v = it->second;
        g_views.erase(it);
    }
    DeviceScope ds(v.device);
    cudaFree(v.devBlock);
}

} // namespace nixl_nvlink

// ================================================================ plugin entry points

namespace {
nixl_b_params_t nvlinkDefaults() {
    return {
        {"use_cuda", "true"},      // false: host-only operation (DRAM transfers)
        {"pin_dram", "true"},      // cudaHostRegister DRAM registrations so kernels can reach them
        {"copy_path", "vector"},   // kernel for descriptors below ce_threshold: "vector" (SIMT) or "bulk" (TMA 1-D through shared memory); "ce": copy engines for everything
        {"ce_threshold", "100663296"}, // descriptors between GPUs of at least this many bytes (96 MiB) go to the copy engines; 0: never
        {"coalesce", "true"},      // merge descriptors that continue their predecessor on both sides
        {"grid_ctas", "0"},        // 0: two CTAs per SM
        {"device_id", "-1"},       // GPU that maps other processes' memory; -1: first registered / current
        {"liveness_ping", "false"},// probe the peer's socket at every post
        {"host_id", ""},           // name of the NVLink box (default: the host name); peers that name another one are left to other backends
        {"num_streams", "4"},      // streams per GPU that independent requests are spread over
        {"proxy", "true"},         // small requests go through a persistent doorbell kernel instead of one launch each
        {"proxy_max_bytes", "2097152"}, // largest request (all descriptors) the proxy takes
        {"proxy_workers", "24"},   // worker CTAs of the proxy kernel
        {"proxy_idle_us", "100"},  // the proxy kernel leaves after this long without a request
        {"proxy_life_us", "2000"}  // and after this long in any case (the next request starts it again)
    };
}
} // namespace

extern "C" NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init() {
    return nixlBackendPluginCreator<nixl_nvlink::Engine>::create(NIXL_PLUGIN_API_VERSION, "NVLINK", "1.0.0", nvlinkDefaults(),
                                                                 {DRAM_SEG, VRAM_SEG});
}

extern "C" NIXL_PLUGIN_EXPORT void nixl_plugin_fini() {}

// Number of kernels the NVLINK backend has launched in this process so far.
extern "C" NIXL_PLUGIN_EXPORT uint64_t nixl_nvlink_kernel_launches() { return nixl_nvlink::kernelLaunches(); }

// The stand-in CUDA runtime (contract: cuda_runtime.h beside this file).
#include "cuda_runtime.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <signal.h>
#include <dirent.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

// ---------------------------------------------------------------- streams and events

struct FakeCudaStream {
    int device = 0;
    std::mutex mu;
    std::condition_variable cv, idleCv;
    std::deque<std::function<void()>> tasks;
    bool busy = false, stop = false;
    std::thread worker;

    explicit FakeCudaStream(int dev) : device(dev) {
        worker = std::thread([this] { run(); });
    }
    ~FakeCudaStream() {
        {
            std::lock_guard<std::mutex> g(mu);
            stop = true;
        }
        cv.notify_all();
        worker.join();
    }
    void push(std::function<void()> t) {
        {
            std::lock_guard<std::mutex> g(mu);
            tasks.push_back(std::move(t));
        }
        cv.notify_one();
    }
    void drain() {
        std::unique_lock<std::mutex> lk(mu);
        idleCv.wait(lk, [this] { return tasks.empty() && !busy; });
    }
    void run();
};

struct FakeCudaEvent {
    std::mutex mu;
    std::condition_variable cv;
    uint64_t recorded = 0;  // times cudaEventRecord was called
    uint64_t completed = 0; // records whose marker has run
};

namespace {

std::atomic<uint64_t> g_tasksRun{0};
thread_local int t_device = 0;
thread_local cudaError_t t_lastError = cudaSuccess;

cudaError_t fail(cudaError_t e) {
    t_lastError = e;
    return e;
}

struct Allocation {
    size_t size;
    int device;
    std::string shm; // name of the shared-memory object behind it (device memory another process can map), or empty
    int vmmFd = -1;  // >= 0: one physical allocation of a virtual-memory range (its memory object); CUDA IPC refuses it
    bool mapped = false; // a mapping of an imported allocation (cuMemMap)
};
struct HostRange {
    size_t size;
    bool ours; // cudaHostAlloc (freed by cudaFreeHost) or cudaHostRegister
};

struct Runtime {
    std::mutex mu;
    int devices = 2;
    std::map<uintptr_t, Allocation> device; // base -> allocation
    std::map<uintptr_t, HostRange> pinned;  // base -> range
    std::vector<std::unique_ptr<FakeCudaStream>> defaults;
    std::vector<FakeCudaStream *> streams; // every live stream (default ones included)
    std::map<std::pair<int, int>, bool> peer;

    Runtime() {
        reapLeftovers();
        if (const char *e = std::getenv("FAKE_CUDA_DEVICES")) devices = std::max(0, std::atoi(e));
        for (int d = 0; d < devices; ++d) {
            defaults.push_back(std::make_unique<FakeCudaStream>(d));
            streams.push_back(defaults.back().get());
        }
    }
    ~Runtime() {
        // Streams the program never destroyed: let their workers finish what is queued.
        for (auto &s : defaults) s->drain();
    }
    // "Device memory" the program never freed: the objects behind it go with the process, as a GPU's memory would.
    // (Run from atexit: the runtime object itself is never destroyed.)
    void unlinkOwnObjects() {
        std::vector<std::string> names;
        {
            std::lock_guard<std::mutex> g(mu);
            const std::string mine = "." + std::to_string(::getpid()) + ".";
            for (const auto &kv : device)
                if (!kv.second.shm.empty() && kv.second.shm.find(mine) != std::string::npos) names.push_back(kv.second.shm);
        }
        for (const auto &n : names) ::shm_unlink(n.c_str());
    }
    // Objects of processes that ended without running the destructor above (a crash, _exit) would pile up in /dev/shm,
    // and one of them would take the name of a later process that draws the same pid: remove those whose owner is gone.
    static void reapLeftovers() {
        DIR *d = ::opendir("/dev/shm");
        if (!d) return;
        while (dirent *e = ::readdir(d)) {
            long pid = 0;
            if (std::sscanf(e->d_name, "fakecuda.%ld.", &pid) != 1 || pid <= 0) continue;
            if (pid == ::getpid() || (::kill(static_cast<pid_t>(pid), 0) != 0 && errno == ESRCH)) ::shm_unlink((std::string("/") + e->d_name).c_str());
        }
        ::closedir(d);
    }
    const Allocation *findDevice(uintptr_t p, uintptr_t *base = nullptr) {
        auto it = device.upper_bound(p);
        if (it == device.begin()) return nullptr;
        --it;
        if (p >= it->first + it->second.size) return nullptr;
        if (base) *base = it->first;
        return &it->second;
    }
    bool isPinned(uintptr_t p) {
        auto it = pinned.upper_bound(p);
        if (it == pinned.begin()) return false;
        --it;
        return p < it->first + it->second.size;
    }
};

Runtime &rt() {
    static Runtime *r = [] {
        auto *x = new Runtime(); // leaked on purpose: worker threads may outlive static destruction
        std::atexit([] { rt().unlinkOwnObjects(); });
        return x;
    }();
    return *r;
}

FakeCudaStream *resolve(cudaStream_t s) {
    if (s) return s;
    Runtime &r = rt();
    if (t_device < 0 || t_device >= r.devices) return nullptr;
    return r.defaults[t_device].get();
}

} // namespace

void FakeCudaStream::run() {
    std::unique_lock<std::mutex> lk(mu);
    for (;;) {
        cv.wait(lk, [this] { return stop || !tasks.empty(); });
        if (tasks.empty()) {
            if (stop) return;
            continue;
        }
        std::function<void()> t = std::move(tasks.front());
        tasks.pop_front();
        busy = true;
        lk.unlock();
        t();
        g_tasksRun.fetch_add(1, std::memory_order_relaxed);
        lk.lock();
        busy = false;
        if (tasks.empty()) idleCv.notify_all();
    }
}

namespace fake_cuda {
void enqueue(cudaStream_t stream, std::function<void()> task) {
    if (FakeCudaStream *s = resolve(stream)) s->push(std::move(task));
}
void enqueueDelay(cudaStream_t stream, unsigned microseconds) {
    enqueue(stream, [microseconds] { std::this_thread::sleep_for(std::chrono::microseconds(microseconds)); });
}
int deviceCount() { return rt().devices; }
uint64_t tasksRun() { return g_tasksRun.load(); }
void *mallocVmm(size_t chunk_bytes, int chunks, int device) {
    if (chunk_bytes == 0 || chunk_bytes % 4096 || chunks <= 0) return nullptr;
    const size_t total = chunk_bytes * static_cast<size_t>(chunks);
    char *va = static_cast<char *>(::mmap(nullptr, total, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0));
    if (va == MAP_FAILED) return nullptr;
    for (int i = 0; i < chunks; ++i) {
        const int fd = ::memfd_create("fakecuda-vmm", MFD_CLOEXEC);
        if (fd < 0 || ::ftruncate(fd, static_cast<off_t>(chunk_bytes)) != 0 ||
            ::mmap(va + i * chunk_bytes, chunk_bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, 0) == MAP_FAILED)
            return nullptr;
        std::lock_guard<std::mutex> g(rt().mu);
        Allocation a{chunk_bytes, device, std::string()};
        a.vmmFd = fd;
        rt().device[reinterpret_cast<uintptr_t>(va + i * chunk_bytes)] = a;
    }
    std::memset(va, 0xcd, total);
    return va;
}
void freeVmm(void *ptr) {
    // every chunk that starts at or behind ptr and continues the range
    uintptr_t p = reinterpret_cast<uintptr_t>(ptr);
    for (;;) {
        Allocation a;
        {
            std::lock_guard<std::mutex> g(rt().mu);
            auto it = rt().device.find(p);
            if (it == rt().device.end() || it->second.vmmFd < 0) return;
            a = it->second;
            rt().device.erase(it);
        }
        ::close(a.vmmFd);
        ::munmap(reinterpret_cast<void *>(p), a.size);
        p += a.size;
    }
}
static std::atomic<int> g_failLaunches[3];
void failLaunches(LaunchKind kind, int count) { g_failLaunches[static_cast<int>(kind)].store(count); }
bool takeLaunchFailure(LaunchKind kind) {
    std::atomic<int> &c = g_failLaunches[static_cast<int>(kind)];
    int left = c.load();
    while (left > 0)
        if (c.compare_exchange_weak(left, left - 1)) return true;
    return false;
}
} // namespace fake_cuda

extern "C" {

cudaError_t cudaGetLastError(void) {
    const cudaError_t e = t_lastError;
    t_lastError = cudaSuccess;
    return e;
}
cudaError_t cudaPeekAtLastError(void) { return t_lastError; }
const char *cudaGetErrorString(cudaError_t e) {
    switch (e) {
    case cudaSuccess: return "no error";
    case cudaErrorInvalidValue: return "invalid argument";
    case cudaErrorMemoryAllocation: return "out of memory";
    case cudaErrorInvalidDevice: return "invalid device ordinal";
    case cudaErrorInvalidResourceHandle: return "invalid resource handle";
    case cudaErrorNotReady: return "device not ready";
    case cudaErrorPeerAccessAlreadyEnabled: return "peer access is already enabled";
    case cudaErrorHostMemoryAlreadyRegistered: return "part or all of the requested memory range is already mapped";
    case cudaErrorHostMemoryNotRegistered: return "pointer does not correspond to a registered memory region";
    case cudaErrorNotSupported: return "operation not supported";
    default: return "unknown error";
    }
}

cudaError_t cudaGetDeviceCount(int *count) {
    if (!count) return fail(cudaErrorInvalidValue);
    *count = rt().devices;
    return cudaSuccess;
}
cudaError_t cudaGetDevice(int *device) {
    if (!device) return fail(cudaErrorInvalidValue);
    *device = t_device;
    return cudaSuccess;
}
cudaError_t cudaSetDevice(int device) {
    if (device < 0 || device >= rt().devices) return fail(cudaErrorInvalidDevice);
    t_device = device;
    return cudaSuccess;
}
cudaError_t cudaDeviceGetAttribute(int *value, enum cudaDeviceAttr attr, int device) {
    if (!value || device < 0 || device >= rt().devices) return fail(cudaErrorInvalidValue);
    if (attr == cudaDevAttrMultiProcessorCount) {
        *value = 148;
        return cudaSuccess;
    }
    return fail(cudaErrorInvalidValue);
}
cudaError_t cudaGetDeviceProperties(struct cudaDeviceProp *prop, int device) {
    if (!prop || device < 0 || device >= rt().devices) return fail(cudaErrorInvalidDevice);
    std::memset(prop, 0, sizeof(*prop));
    std::snprintf(prop->name, sizeof(prop->name), "stand-in GPU %d", device);
    std::memset(prop->uuid.bytes, 0xa0 + device, sizeof(prop->uuid.bytes));
    prop->uuid.bytes[0] = static_cast<char>(device);
    prop->totalGlobalMem = size_t(16) << 30;
    prop->multiProcessorCount = 148;
    prop->major = 10;
    prop->pciBusID = device + 1;
    return cudaSuccess;
}
cudaError_t cudaDeviceSynchronize(void) {
    std::vector<FakeCudaStream *> snap;
    {
        std::lock_guard<std::mutex> g(rt().mu);
        for (FakeCudaStream *s : rt().streams)
            if (s->device == t_device) snap.push_back(s);
    }
    // A stream may be destroyed by another thread while this one waits: only a program that already races does that.
    for (FakeCudaStream *s : snap) s->drain();
    return cudaSuccess;
}
cudaError_t cudaDeviceCanAccessPeer(int *can, int device, int peer) {
    if (!can || device < 0 || peer < 0 || device >= rt().devices || peer >= rt().devices) return fail(cudaErrorInvalidDevice);
    *can = device != peer;
    return cudaSuccess;
}
cudaError_t cudaDeviceEnablePeerAccess(int peer, unsigned int) {
    if (peer < 0 || peer >= rt().devices || peer == t_device) return fail(cudaErrorInvalidDevice);
    std::lock_guard<std::mutex> g(rt().mu);
    bool &on = rt().peer[{t_device, peer}];
    if (on) return fail(cudaErrorPeerAccessAlreadyEnabled);
    on = true;
    return cudaSuccess;
}

// "Device memory" lives in shared-memory objects, so that another process can map it through an IPC handle the way a
// second process maps a real GPU allocation (at an address of its own).  Allocations of less than a page stay on the heap
// (an IPC handle for them works inside the process only).
cudaError_t cudaMalloc(void **ptr, size_t size) {
    if (!ptr) return fail(cudaErrorInvalidValue);
    static std::atomic<uint64_t> serial{0};
    void *p = nullptr;
    std::string name;
    if (size >= 4096) {
        name = "/fakecuda." + std::to_string(::getpid()) + "." + std::to_string(serial.fetch_add(1));
        int fd = ::shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR | O_CLOEXEC, 0600);
        if (fd < 0 && errno == EEXIST) { // the name carries this process's pid: whatever has it is a dead process's leftover
            ::shm_unlink(name.c_str());
            fd = ::shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR | O_CLOEXEC, 0600);
        }
        if (fd >= 0 && ::ftruncate(fd, static_cast<off_t>(size)) == 0) p = ::mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        if (fd >= 0) ::close(fd);
        if (p == nullptr || p == MAP_FAILED) {
            if (fd >= 0) ::shm_unlink(name.c_str());
            return fail(cudaErrorMemoryAllocation);
        }
    } else if (posix_memalign(&p, 512, size ? size : 1) != 0) {
        return fail(cudaErrorMemoryAllocation);
    }
    std::memset(p, 0xcd, size); // fresh device memory is not zero
    std::lock_guard<std::mutex> g(rt().mu);
    rt().device[reinterpret_cast<uintptr_t>(p)] = {size, t_device, name};
    *ptr = p;
    return cudaSuccess;
}
cudaError_t cudaFree(void *ptr) {
    if (!ptr) return cudaSuccess;
    Allocation a;
    {
        std::lock_guard<std::mutex> g(rt().mu);
        auto it = rt().device.find(reinterpret_cast<uintptr_t>(ptr));
        if (it == rt().device.end()) return fail(cudaErrorInvalidValue);
        a = it->second;
        rt().device.erase(it);
    }
    cudaDeviceSynchronize(); // as the real call: the device is idle before memory goes away
    if (a.shm.empty()) {
        std::free(ptr);
    } else {
        ::munmap(ptr, a.size);
        ::shm_unlink(a.shm.c_str()); // processes that mapped it keep their mappings, as with a real handle
    }
    return cudaSuccess;
}
cudaError_t cudaHostAlloc(void **ptr, size_t size, unsigned int) {
    if (!ptr) return fail(cudaErrorInvalidValue);
    void *p = nullptr;
    if (posix_memalign(&p, 4096, size ? size : 1) != 0) return fail(cudaErrorMemoryAllocation);
    std::lock_guard<std::mutex> g(rt().mu);
    rt().pinned[reinterpret_cast<uintptr_t>(p)] = {size, true};
    *ptr = p;
    return cudaSuccess;
}
cudaError_t cudaFreeHost(void *ptr) {
    if (!ptr) return cudaSuccess;
    {
        std::lock_guard<std::mutex> g(rt().mu);
        auto it = rt().pinned.find(reinterpret_cast<uintptr_t>(ptr));
        if (it == rt().pinned.end() || !it->second.ours) return fail(cudaErrorInvalidValue);
        rt().pinned.erase(it);
    }
    std::free(ptr);
    return cudaSuccess;
}
cudaError_t cudaHostRegister(void *ptr, size_t size, unsigned int) {
    if (!ptr || size == 0) return fail(cudaErrorInvalidValue);
    const uintptr_t p = reinterpret_cast<uintptr_t>(ptr);
    std::lock_guard<std::mutex> g(rt().mu);
    for (auto &kv : rt().pinned)
        if (p < kv.first + kv.second.size && kv.first < p + size) return fail(cudaErrorHostMemoryAlreadyRegistered);
    rt().pinned[p] = {size, false};
    return cudaSuccess;
}
cudaError_t cudaHostUnregister(void *ptr) {
    std::lock_guard<std::mutex> g(rt().mu);
    auto it = rt().pinned.find(reinterpret_cast<uintptr_t>(ptr));
    if (it == rt().pinned.end() || it->second.ours) return fail(cudaErrorHostMemoryNotRegistered);
    rt().pinned.erase(it);
    return cudaSuccess;
}
cudaError_t cudaHostGetDevicePointer(void **dev, void *host, unsigned int) {
    if (!dev) return fail(cudaErrorInvalidValue);
    std::lock_guard<std::mutex> g(rt().mu);
    if (!rt().isPinned(reinterpret_cast<uintptr_t>(host))) return fail(cudaErrorInvalidValue);
    *dev = host;
    return cudaSuccess;
}
cudaError_t cudaPointerGetAttributes(struct cudaPointerAttributes *attr, const void *ptr) {
    if (!attr) return fail(cudaErrorInvalidValue);
    std::lock_guard<std::mutex> g(rt().mu);
    const uintptr_t p = reinterpret_cast<uintptr_t>(ptr);
    if (const Allocation *a = rt().findDevice(p)) {
        *attr = {cudaMemoryTypeDevice, a->device, const_cast<void *>(ptr), nullptr};
    } else if (rt().isPinned(p)) {
        *attr = {cudaMemoryTypeHost, 0, const_cast<void *>(ptr), const_cast<void *>(ptr)};
    } else {
        *attr = {cudaMemoryTypeUnregistered, -1, nullptr, const_cast<void *>(ptr)};
    }
    return cudaSuccess;
}

cudaError_t cudaMemset(void *ptr, int value, size_t count) {
    if (!ptr && count) return fail(cudaErrorInvalidValue);
    if (FakeCudaStream *s = resolve(nullptr)) s->drain(); // the default stream's order
    std::memset(ptr, value, count);
    return cudaSuccess;
}
cudaError_t cudaMemcpy(void *dst, const void *src, size_t count, enum cudaMemcpyKind) {
    if ((!dst || !src) && count) return fail(cudaErrorInvalidValue);
    if (FakeCudaStream *s = resolve(nullptr)) s->drain();
    std::memmove(dst, src, count);
    return cudaSuccess;
}
cudaError_t cudaMemcpyAsync(void *dst, const void *src, size_t count, enum cudaMemcpyKind, cudaStream_t stream) {
    if ((!dst || !src) && count) return fail(cudaErrorInvalidValue);
    FakeCudaStream *s = resolve(stream);
    if (!s) return fail(cudaErrorInvalidResourceHandle);
    bool pageable_source;
    {
        std::lock_guard<std::mutex> g(rt().mu);
        const uintptr_t p = reinterpret_cast<uintptr_t>(src);
        pageable_source = !rt().findDevice(p) && !rt().isPinned(p);
    }
    if (pageable_source) {
        // As the real runtime: a pageable source is taken now (the caller may free it when the call returns).
        auto staged = std::make_shared<std::vector<char>>(static_cast<const char *>(src), static_cast<const char *>(src) + count);
        s->push([dst, staged] { std::memcpy(dst, staged->data(), staged->size()); });
    } else {
        s->push([dst, src, count] { std::memmove(dst, src, count); });
    }
    return cudaSuccess;
}

cudaError_t cudaStreamCreateWithFlags(cudaStream_t *stream, unsigned int) {
    if (!stream) return fail(cudaErrorInvalidValue);
    auto *s = new FakeCudaStream(t_device);
    std::lock_guard<std::mutex> g(rt().mu);
    rt().streams.push_back(s);
    *stream = s;
    return cudaSuccess;
}
cudaError_t cudaStreamCreate(cudaStream_t *stream) { return cudaStreamCreateWithFlags(stream, cudaStreamDefault); }
cudaError_t cudaStreamDestroy(cudaStream_t stream) {
    if (!stream) return fail(cudaErrorInvalidResourceHandle);
    stream->drain(); // the real call lets queued work finish
    {
        std::lock_guard<std::mutex> g(rt().mu);
        auto &v = rt().streams;
        v.erase(std::remove(v.begin(), v.end(), stream), v.end());
    }
    delete stream;
    return cudaSuccess;
}
cudaError_t cudaStreamSynchronize(cudaStream_t stream) {
    FakeCudaStream *s = resolve(stream);
    if (!s) return fail(cudaErrorInvalidResourceHandle);
    s->drain();
    return cudaSuccess;
}
cudaError_t cudaStreamWaitEvent(cudaStream_t stream, cudaEvent_t event, unsigned int) {
    FakeCudaStream *s = resolve(stream);
    if (!s || !event) return fail(cudaErrorInvalidResourceHandle);
    uint64_t want;
    {
        std::lock_guard<std::mutex> g(event->mu);
        want = event->recorded; // the work captured by the latest record
    }
    s->push([event, want] {
        std::unique_lock<std::mutex> lk(event->mu);
        event->cv.wait(lk, [&] { return event->completed >= want; });
    });
    return cudaSuccess;
}

cudaError_t cudaEventCreateWithFlags(cudaEvent_t *event, unsigned int) {
    if (!event) return fail(cudaErrorInvalidValue);
    *event = new FakeCudaEvent();
    return cudaSuccess;
}
cudaError_t cudaEventCreate(cudaEvent_t *event) { return cudaEventCreateWithFlags(event, cudaEventDefault); }
cudaError_t cudaEventDestroy(cudaEvent_t event) {
    if (!event) return fail(cudaErrorInvalidResourceHandle);
    // The real call defers the release until the event has completed; waiting here has the same effect.
    {
        std::unique_lock<std::mutex> lk(event->mu);
        event->cv.wait(lk, [&] { return event->completed >= event->recorded; });
    }
    delete event;
    return cudaSuccess;
}
cudaError_t cudaEventRecord(cudaEvent_t event, cudaStream_t stream) {
    FakeCudaStream *s = resolve(stream);
    if (!s || !event) return fail(cudaErrorInvalidResourceHandle);
    uint64_t mine;
    {
        std::lock_guard<std::mutex> g(event->mu);
        mine = ++event->recorded;
    }
    s->push([event, mine] {
        std::lock_guard<std::mutex> g(event->mu); // notified under the lock: cudaEventDestroy may free the event right after
        if (event->completed < mine) event->completed = mine;
        event->cv.notify_all();
    });
    return cudaSuccess;
}
cudaError_t cudaEventQuery(cudaEvent_t event) {
    if (!event) return fail(cudaErrorInvalidResourceHandle);
    std::lock_guard<std::mutex> g(event->mu);
    if (event->completed >= event->recorded) return cudaSuccess;
    return fail(cudaErrorNotReady); // recorded as the last error, as the real runtime does
}
cudaError_t cudaEventSynchronize(cudaEvent_t event) {
    if (!event) return fail(cudaErrorInvalidResourceHandle);
    std::unique_lock<std::mutex> lk(event->mu);
    event->cv.wait(lk, [&] { return event->completed >= event->recorded; });
    return cudaSuccess;
}

// The handle carries the owner's process id, the base address there, the size and the name of the shared-memory object.
// Opened in the owner's process it gives the allocation itself; in another process a mapping of the same memory.
namespace {
struct IpcPayload {
    uint64_t base, pid, size;
    char name[40];
};
static_assert(sizeof(IpcPayload) <= sizeof(cudaIpcMemHandle_t), "payload fits the handle");
std::map<uintptr_t, size_t> g_ipcMappings; // mappings of other processes' allocations (under rt().mu)
} // namespace

cudaError_t cudaIpcGetMemHandle(cudaIpcMemHandle_t *handle, void *ptr) {
    if (!handle) return fail(cudaErrorInvalidValue);
    std::lock_guard<std::mutex> g(rt().mu);
    auto it = rt().device.find(reinterpret_cast<uintptr_t>(ptr));
    if (it == rt().device.end() || it->second.vmmFd >= 0 || it->second.mapped) return fail(cudaErrorInvalidValue); // the base of a cudaMalloc allocation only
    IpcPayload pl{};
    pl.base = reinterpret_cast<uintptr_t>(ptr);
    pl.pid = static_cast<uint64_t>(::getpid());
    pl.size = it->second.size;
    std::snprintf(pl.name, sizeof(pl.name), "%s", it->second.shm.c_str());
    std::memset(handle, 0, sizeof(*handle));
    std::memcpy(handle->reserved, &pl, sizeof(pl));
    return cudaSuccess;
}
cudaError_t cudaIpcOpenMemHandle(void **ptr, cudaIpcMemHandle_t handle, unsigned int) {
    if (!ptr) return fail(cudaErrorInvalidValue);
    IpcPayload pl;
    std::memcpy(&pl, handle.reserved, sizeof(pl));
    pl.name[sizeof(pl.name) - 1] = 0;
    if (pl.pid == static_cast<uint64_t>(::getpid())) { // (the real runtime refuses this; the backend never asks for it)
        *ptr = reinterpret_cast<void *>(pl.base);
        return cudaSuccess;
    }
    if (pl.name[0] == 0) return fail(cudaErrorNotSupported);
    const int fd = ::shm_open(pl.name, O_RDWR | O_CLOEXEC, 0);
    if (fd < 0) return fail(cudaErrorInvalidValue);
    void *p = ::mmap(nullptr, pl.size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) return fail(cudaErrorMemoryAllocation);
    std::lock_guard<std::mutex> g(rt().mu);
    g_ipcMappings[reinterpret_cast<uintptr_t>(p)] = pl.size;
    // kernels of this process address it like device memory of the GPU that opened it
    rt().device[reinterpret_cast<uintptr_t>(p)] = {pl.size, t_device, std::string()};
    *ptr = p;
    return cudaSuccess;
}
cudaError_t cudaIpcCloseMemHandle(void *ptr) {
    std::lock_guard<std::mutex> g(rt().mu);
    auto it = g_ipcMappings.find(reinterpret_cast<uintptr_t>(ptr));
    if (it == g_ipcMappings.end()) return cudaSuccess; // an allocation of this process: nothing was mapped
    ::munmap(ptr, it->second);
    rt().device.erase(reinterpret_cast<uintptr_t>(ptr));
    g_ipcMappings.erase(it);
    return cudaSuccess;
}

static int fakeGetAddressRange(unsigned long long *base, size_t *size, unsigned long long ptr) {
    std::lock_guard<std::mutex> g(rt().mu);
    uintptr_t b = 0;
    const Allocation *a = rt().findDevice(static_cast<uintptr_t>(ptr), &b);
    if (!a) return 1;
    if (base) *base = b;
    if (size) *size = a->size;
    return 0;
}

// ---- the driver's virtual-memory calls (signatures as the backend's function-pointer types) ----
namespace {
struct VmmHandle {
    int fd;
    size_t size;
};
int vmmRetain(unsigned long long *handle, void *addr) {
    std::lock_guard<std::mutex> g(rt().mu);
    uintptr_t base = 0;
    const Allocation *a = rt().findDevice(reinterpret_cast<uintptr_t>(addr), &base);
    if (!a || a->vmmFd < 0) return 1; // not memory of that kind
    *handle = reinterpret_cast<uintptr_t>(new VmmHandle{::dup(a->vmmFd), a->size});
    return 0;
}
int vmmExport(void *out, unsigned long long handle, int, unsigned long long) {
    auto *h = reinterpret_cast<VmmHandle *>(static_cast<uintptr_t>(handle));
    const int fd = ::dup(h->fd);
    if (fd < 0) return 1;
    *static_cast<int *>(out) = fd;
    return 0;
}
int vmmImport(unsigned long long *handle, void *os_handle, int) {
    const int fd = static_cast<int>(reinterpret_cast<uintptr_t>(os_handle));
    struct stat st{};
    if (::fstat(fd, &st) != 0) return 1;
    *handle = reinterpret_cast<uintptr_t>(new VmmHandle{::dup(fd), static_cast<size_t>(st.st_size)});
    return 0;
}
int vmmRelease(unsigned long long handle) {
    auto *h = reinterpret_cast<VmmHandle *>(static_cast<uintptr_t>(handle));
    ::close(h->fd);
    delete h;
    return 0;
}
int vmmReserve(unsigned long long *ptr, size_t size, size_t, unsigned long long, unsigned long long) {
    void *p = ::mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (p == MAP_FAILED) return 2;
    *ptr = reinterpret_cast<uintptr_t>(p);
    return 0;
}
int vmmAddressFree(unsigned long long ptr, size_t size) { return ::munmap(reinterpret_cast<void *>(static_cast<uintptr_t>(ptr)), size) == 0 ? 0 : 1; }
int vmmMapCall(unsigned long long ptr, size_t size, size_t offset, unsigned long long handle, unsigned long long) {
    auto *h = reinterpret_cast<VmmHandle *>(static_cast<uintptr_t>(handle));
    if (offset + size > h->size) return 1;
    void *p = ::mmap(reinterpret_cast<void *>(static_cast<uintptr_t>(ptr)), size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, h->fd, static_cast<off_t>(offset));
    if (p == MAP_FAILED) return 1;
    std::lock_guard<std::mutex> g(rt().mu);
    Allocation a{size, t_device, std::string()};
    a.mapped = true;
    rt().device[static_cast<uintptr_t>(ptr)] = a;
    return 0;
}
int vmmUnmapCall(unsigned long long ptr, size_t size) {
    {
        std::lock_guard<std::mutex> g(rt().mu);
        rt().device.erase(static_cast<uintptr_t>(ptr));
    }
    void *p = ::mmap(reinterpret_cast<void *>(static_cast<uintptr_t>(ptr)), size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_FIXED | MAP_NORESERVE, -1, 0);
    return p == MAP_FAILED ? 1 : 0;
}
int vmmSetAccess(unsigned long long, size_t, const void *, size_t) { return 0; }
} // namespace

cudaError_t cudaGetDriverEntryPoint(const char *symbol, void **fn, unsigned long long, enum cudaDriverEntryPointQueryResult *result) {
    if (!symbol || !fn) return fail(cudaErrorInvalidValue);
    static const struct {
        const char *name;
        void *fn;
    } table[] = {
        {"cuMemGetAddressRange", reinterpret_cast<void *>(&fakeGetAddressRange)},
        {"cuMemRetainAllocationHandle", reinterpret_cast<void *>(&vmmRetain)},
        {"cuMemExportToShareableHandle", reinterpret_cast<void *>(&vmmExport)},
        {"cuMemImportFromShareableHandle", reinterpret_cast<void *>(&vmmImport)},
        {"cuMemRelease", reinterpret_cast<void *>(&vmmRelease)},
        {"cuMemAddressReserve", reinterpret_cast<void *>(&vmmReserve)},
        {"cuMemAddressFree", reinterpret_cast<void *>(&vmmAddressFree)},
        {"cuMemMap", reinterpret_cast<void *>(&vmmMapCall)},
        {"cuMemUnmap", reinterpret_cast<void *>(&vmmUnmapCall)},
        {"cuMemSetAccess", reinterpret_cast<void *>(&vmmSetAccess)},
    };
    for (const auto &e : table)
        if (std::strcmp(symbol, e.name) == 0) {
            *fn = e.fn;
            if (result) *result = cudaDriverEntryPointSuccess;
            return cudaSuccess;
        }
    *fn = nullptr;
    if (result) *result = cudaDriverEntryPointSymbolNotFound;
    return cudaSuccess;
}

} // extern "C"

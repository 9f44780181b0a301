#include "plugins/nvlink/vmm_share.h"

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cuda.h>
#include <cuda_runtime.h>

#include "utils/log.h"

namespace nixl_nvlink {
namespace {

// Driver entry points through the runtime (the plug-in does not link libcuda).
template<class Fn> Fn driverFn(const char *name) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return reinterpret_cast<Fn>(p);
}

struct Driver {
    CUresult (*getAddressRange)(CUdeviceptr *, size_t *, CUdeviceptr) = nullptr;
    CUresult (*retainHandle)(CUmemGenericAllocationHandle *, void *) = nullptr;
    CUresult (*exportHandle)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*importHandle)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType) = nullptr;
    CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*reserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*addressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*setAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t) = nullptr;
    bool ok = false;
};

const Driver &driver() {
    static const Driver d = [] {
        Driver x;
        x.getAddressRange = driverFn<decltype(x.getAddressRange)>("cuMemGetAddressRange");
        x.retainHandle = driverFn<decltype(x.retainHandle)>("cuMemRetainAllocationHandle");
        x.exportHandle = driverFn<decltype(x.exportHandle)>("cuMemExportToShareableHandle");
        x.importHandle = driverFn<decltype(x.importHandle)>("cuMemImportFromShareableHandle");
        x.release = driverFn<decltype(x.release)>("cuMemRelease");
        x.reserve = driverFn<decltype(x.reserve)>("cuMemAddressReserve");
        x.addressFree = driverFn<decltype(x.addressFree)>("cuMemAddressFree");
        x.map = driverFn<decltype(x.map)>("cuMemMap");
        x.unmap = driverFn<decltype(x.unmap)>("cuMemUnmap");
        x.setAccess = driverFn<decltype(x.setAccess)>("cuMemSetAccess");
        x.ok = x.getAddressRange && x.retainHandle && x.exportHandle && x.importHandle && x.release && x.reserve && x.addressFree && x.map &&
            x.unmap && x.setAccess;
        return x;
    }();
    return d;
}

sockaddr_un abstractAddr(const std::string &name, socklen_t &len) {
    sockaddr_un a{};
    a.sun_family = AF_UNIX;
    const size_t n = std::min(name.size(), sizeof(a.sun_path) - 2);
    std::memcpy(a.sun_path + 1, name.data(), n); // leading NUL = abstract namespace
    len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
    return a;
}

constexpr char kMagic[6] = {'N', 'I', 'X', 'L', 'F', 'D'};
constexpr size_t kMaxPerMessage = 128; // descriptors per datagram (the kernel allows 253)

struct Wire {
    char magic[6];
    uint16_t pad;
    uint32_t count;
    int32_t numbers[kMaxPerMessage];
};

} // namespace

// ================================================================ export

bool vmmExportRange(uintptr_t addr, size_t len, std::vector<VmmChunk> &out) {
    const Driver &d = driver();
    if (!d.ok || len == 0) return false;
    std::vector<VmmChunk> chunks;
    uintptr_t p = addr;
    const uintptr_t end = addr + len;
    while (p < end) {
        CUdeviceptr base = 0;
        size_t size = 0;
        if (d.getAddressRange(&base, &size, static_cast<CUdeviceptr>(p)) != CUDA_SUCCESS || size == 0) {
            vmmCloseChunks(chunks);
            return false;
        }
        CUmemGenericAllocationHandle h = 0;
        if (d.retainHandle(&h, reinterpret_cast<void *>(base)) != CUDA_SUCCESS) { // not VMM memory
            vmmCloseChunks(chunks);
            return false;
        }
        int fd = -1;
        const CUresult e = d.exportHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
        d.release(h);
        if (e != CUDA_SUCCESS || fd < 0) { // created without the POSIX handle type
            vmmCloseChunks(chunks);
            return false;
        }
        chunks.push_back({static_cast<uint64_t>(base), static_cast<uint64_t>(size), fd});
        p = static_cast<uintptr_t>(base) + size;
        if (chunks.size() > 65536) { // a registration of that many allocations is not one we want to mirror
            vmmCloseChunks(chunks);
            return false;
        }
    }
    out = std::move(chunks);
    return true;
}

void vmmCloseChunks(std::vector<VmmChunk> &chunks) {
    for (auto &c : chunks)
        if (c.fd >= 0) ::close(c.fd);
    chunks.clear();
}

// ================================================================ import

bool vmmMap(const std::vector<VmmChunk> &chunks, const std::vector<int> &fds, int device_count, int owner_local_device, VmmMapping &out) {
    const Driver &d = driver();
    auto close_all = [&] {
        for (int fd : fds)
            if (fd >= 0) ::close(fd);
    };
    if (!d.ok || chunks.empty() || chunks.size() != fds.size()) {
        close_all();
        return false;
    }
    const uint64_t first = chunks.front().base;
    const uint64_t span = chunks.back().base + chunks.back().size - first;
    CUdeviceptr va = 0;
    if (d.reserve(&va, span, 2u << 20, 0, 0) != CUDA_SUCCESS) {
        close_all();
        return false;
    }
    VmmMapping m;
    m.va = va;
    m.span = span;
    std::vector<CUmemAccessDesc> access;
    for (int dev = 0; dev < device_count; ++dev) {
        int can = dev == owner_local_device;
        if (!can && owner_local_device >= 0 && cudaDeviceCanAccessPeer(&can, dev, owner_local_device) != cudaSuccess) {
            cudaGetLastError();
            can = 0;
        }
        if (owner_local_device < 0) can = 1; // owner not visible here by ordinal: let the driver decide per device
        if (!can) continue;
        CUmemAccessDesc a{};
        a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        a.location.id = dev;
        a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        access.push_back(a);
    }
    bool ok = !access.empty();
    for (size_t i = 0; ok && i < chunks.size(); ++i) {
        CUmemGenericAllocationHandle h = 0;
        if (d.importHandle(&h, reinterpret_cast<void *>(static_cast<uintptr_t>(fds[i])), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS) {
            ok = false;
            break;
        }
        const uint64_t off = chunks[i].base - first;
        if (d.map(va + off, chunks[i].size, 0, h, 0) != CUDA_SUCCESS) {
            d.release(h);
            ok = false;
            break;
        }
        d.release(h); // the mapping keeps the allocation alive
        m.mapped.emplace_back(off, chunks[i].size);
        // Access per device: a GPU that cannot be granted access is simply not granted it.
        bool any = false;
        for (const auto &a : access) any |= d.setAccess(va + off, chunks[i].size, &a, 1) == CUDA_SUCCESS;
        ok = any;
    }
    close_all();
    if (!ok) {
        vmmUnmap(m);
        return false;
    }
    out = std::move(m);
    return true;
}

void vmmUnmap(VmmMapping &m) {
    const Driver &d = driver();
    if (!d.ok || m.va == 0) return;
    for (auto &piece : m.mapped) d.unmap(m.va + piece.first, piece.second);
    d.addressFree(m.va, m.span);
    m = VmmMapping{};
}

// ================================================================ descriptor server

VmmFdServer::~VmmFdServer() {
    if (th_.joinable()) {
        const char c = 1;
        if (::write(wake_[1], &c, 1) < 0) {
        }
        th_.join();
    }
    if (sock_ >= 0) ::close(sock_);
    for (int fd : wake_)
        if (fd >= 0) ::close(fd);
}

bool VmmFdServer::start(const std::string &name) {
    std::lock_guard<std::mutex> g(mu_);
    if (sock_ >= 0) return true;
    const int s = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
    if (s < 0) return false;
    socklen_t alen = 0;
    sockaddr_un addr = abstractAddr(name, alen);
    if (::bind(s, reinterpret_cast<sockaddr *>(&addr), alen) != 0 || ::pipe(wake_) != 0) {
        ::close(s);
        return false;
    }
    sock_ = s;
    name_ = name;
    th_ = std::thread([this] { loop(); });
    return true;
}

void VmmFdServer::allow(int fd) {
    std::lock_guard<std::mutex> g(mu_);
    allowed_.push_back(fd);
}

void VmmFdServer::revoke(int fd) {
    std::lock_guard<std::mutex> g(mu_);
    allowed_.erase(std::remove(allowed_.begin(), allowed_.end(), fd), allowed_.end());
}

void VmmFdServer::loop() {
    for (;;) {
        pollfd fds[2] = {{sock_, POLLIN, 0}, {wake_[0], POLLIN, 0}};
        if (::poll(fds, 2, -1) < 0) {
            if (errno == EINTR) continue;
            return;
        }
        if (fds[1].revents) return;
        Wire req{};
        sockaddr_un from{};
        socklen_t flen = sizeof(from);
        const ssize_t n = ::recvfrom(sock_, &req, sizeof(req), MSG_DONTWAIT, reinterpret_cast<sockaddr *>(&from), &flen);
        if (n < static_cast<ssize_t>(offsetof(Wire, numbers)) || std::memcmp(req.magic, kMagic, 6) != 0 || req.count > kMaxPerMessage ||
            n < static_cast<ssize_t>(offsetof(Wire, numbers) + req.count * sizeof(int32_t)) || flen <= sizeof(sa_family_t))
            continue; // not a request, or the sender has no address to answer to
        bool known = true;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (uint32_t i = 0; i < req.count; ++i) known &= std::find(allowed_.begin(), allowed_.end(), req.numbers[i]) != allowed_.end();
        }
        Wire rep = req;
        if (!known) rep.count = 0;
        iovec iov{&rep, offsetof(Wire, numbers) + rep.count * sizeof(int32_t)};
        alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int) * kMaxPerMessage)];
        msghdr msg{};
        msg.msg_name = &from;
        msg.msg_namelen = flen;
        msg.msg_iov = &iov;
        msg.msg_iovlen = 1;
        if (rep.count > 0) {
            msg.msg_control = control;
            msg.msg_controllen = CMSG_SPACE(sizeof(int) * rep.count);
            cmsghdr *c = CMSG_FIRSTHDR(&msg);
            if (c == nullptr) continue; // cannot happen with the control length above; keeps the header access provably safe
            c->cmsg_level = SOL_SOCKET;
            c->cmsg_type = SCM_RIGHTS;
            c->cmsg_len = CMSG_LEN(sizeof(int) * rep.count);
            std::memcpy(CMSG_DATA(c), req.numbers, sizeof(int) * rep.count);
        }
        if (::sendmsg(sock_, &msg, MSG_NOSIGNAL) < 0) NIXL_WARN << "NVLINK backend: could not answer a memory-handle request: " << std::strerror(errno);
    }
}

std::vector<int> vmmFetchFds(const std::string &server_name, const std::vector<int> &numbers, int timeout_ms) {
    std::vector<int> out;
    const int s = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
    if (s < 0) return out;
    // Bind (autobind gives an abstract address): the server answers to the sender's address.
    sockaddr_un self{};
    self.sun_family = AF_UNIX;
    if (::bind(s, reinterpret_cast<sockaddr *>(&self), sizeof(sa_family_t)) != 0) {
        ::close(s);
        return out;
    }
    socklen_t alen = 0;
    sockaddr_un addr = abstractAddr(server_name, alen);
    bool ok = true;
    for (size_t done = 0; ok && done < numbers.size();) {
        const size_t n = std::min(kMaxPerMessage, numbers.size() - done);
        Wire req{};
        std::memcpy(req.magic, kMagic, 6);
        req.count = static_cast<uint32_t>(n);
        for (size_t i = 0; i < n; ++i) req.numbers[i] = numbers[done + i];
        if (::sendto(s, &req, offsetof(Wire, numbers) + n * sizeof(int32_t), MSG_NOSIGNAL, reinterpret_cast<sockaddr *>(&addr), alen) < 0) {
            ok = false;
            break;
        }
        pollfd pfd{s, POLLIN, 0};
        if (::poll(&pfd, 1, timeout_ms) <= 0) {
            ok = false;
            break;
        }
        Wire rep{};
        iovec iov{&rep, sizeof(rep)};
        alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int) * kMaxPerMessage)];
        msghdr msg{};
        msg.msg_iov = &iov;
        msg.msg_iovlen = 1;
        msg.msg_control = control;
        msg.msg_controllen = sizeof(control);
        const ssize_t got = ::recvmsg(s, &msg, MSG_CMSG_CLOEXEC);
        if (got < static_cast<ssize_t>(offsetof(Wire, numbers)) || std::memcmp(rep.magic, kMagic, 6) != 0 || rep.count != n) {
            ok = false;
        }
        size_t received = 0;
        for (cmsghdr *c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
            if (c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) continue;
            const size_t k = (c->cmsg_len - CMSG_LEN(0)) / sizeof(int);
            for (size_t i = 0; i < k; ++i) {
                int fd;
                std::memcpy(&fd, CMSG_DATA(c) + i * sizeof(int), sizeof(int));
                out.push_back(fd);
                ++received;
            }
        }
        if (received != n) ok = false;
        done += n;
    }
    ::close(s);
    if (!ok) {
        for (int fd : out) ::close(fd);
        out.clear();
    }
    return out;
}

} // namespace nixl_nvlink

// TCP backend: one-sided WRITE / READ and notifications between agents on DIFFERENT hosts (or on one host), over plain
// TCP sockets.  It is the backend for the part of a deployment that NVLink does not reach: the NVLINK backend refuses a
// peer on another host, the agent then picks whichever backend both sides have, and this one only needs an IP route.
//
// Role parity: the reference reaches other nodes through UCX (src/plugins/ucx/ucx_backend.cpp; over TCP when there is
// no RDMA NIC).  This engine gives the same contract with sockets only: registrations are published as (address,
// length, key), a transfer names remote ranges inside such registrations, the target checks every range against what
// it registered before touching memory, a notification follows its data.
//
// Shape
//   * Every engine listens on one port ("port" parameter, default: any).  The connection info it publishes holds the
//     host name, the port and the addresses to try (the "address" parameter or NIXL_TCP_ADDRESS; otherwise every IPv4 and
//     global IPv6 address of the host, loopback last; a peer on the same host tries loopback first).  `device_id` names the GPU
//     this engine serves: the interfaces nearest to it in the PCI tree (utils/topology.h) come first.  With several
//     addresses published, and `local_addresses` (a list, or "auto") on the initiator, connection k of a peer runs from
//     local address k to the peer's address k: the rails spread over the interfaces of both hosts.
//   * The initiator opens `rails` connections to a peer on first use.  A request is cut into messages of at most
//     `chunk_bytes` of payload (many small descriptors share one message, a large one is split) which are dealt over
//     the rails; each rail has a sender thread (queue) and a receiver thread (acknowledgements, READ replies), so a post
//     returns at once and `checkXfer` reads one atomic word.
//   * Payload goes from and to user memory directly (scatter / gather I/O); device memory is staged through a pinned
//     buffer of the connection with plain runtime copies.
//   * The target serves each accepted connection from a thread of its own: it reads a message, checks every range
//     against the registrations (key, bounds), moves the bytes, answers.  A range outside a registration is answered with
//     an error and its payload is discarded; the connection stays usable.
//   * A request's notification is sent when the last acknowledgement has arrived, on the peer's first rail.
//   * A read or a write that makes no progress for `stall_timeout_ms` (30 s) inside a message, or while answers are
//     outstanding, counts as a broken connection; silence between messages does not.
//   * A connection that breaks fails what was in flight on it with NIXL_ERR_REMOTE_DISCONNECT; the next post tries to
//     connect again, and reports the same status when the peer cannot be reached.
//
// Both ends are assumed little-endian (the wire structs are sent as they lie in memory).
#include <arpa/inet.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <thread>
#include <unordered_map>

#include <cuda_runtime.h>

#include "backend/backend_plugin.h"
#include "utils/log.h"
#include "utils/misc.h"
#include "utils/topology.h"

#ifndef NIXL_TCP_PLUGIN_NAME
#define NIXL_TCP_PLUGIN_NAME "TCP"
#endif

// ThreadSanitizer does not see an order that runs through a socket: the initiator waits for the answer to one message
// before it sends the next one that touches the same bytes, and the two may be served by different threads of the
// target.  The serving threads state that order themselves (release after a message, acquire before the next).
#if defined(__SANITIZE_THREAD__)
extern "C" void __tsan_acquire(void *addr);
extern "C" void __tsan_release(void *addr);
#define NIXL_TCP_ORDER_ACQUIRE(p) __tsan_acquire(p)
#define NIXL_TCP_ORDER_RELEASE(p) __tsan_release(p)
#else
#define NIXL_TCP_ORDER_ACQUIRE(p) ((void)0)
#define NIXL_TCP_ORDER_RELEASE(p) ((void)0)
#endif

namespace {

constexpr uint32_t kMagic = 0x4e585443u; // "CTXN"
constexpr uint32_t kMaxDescsPerMsg = 256;
constexpr size_t kBounceBytes = 4u << 20;
constexpr size_t kInlineBytes = 256u << 10; // a WRITE message up to this size may be sent by the posting thread itself (the last message of a request, when its connection is idle)
constexpr unsigned kSpinUs = 100;           // how long a thread polls its socket for the next message before it sleeps

enum Op : uint16_t { OP_HELLO = 1, OP_WRITE = 2, OP_READ = 3, OP_ACK = 4, OP_READ_REPLY = 5, OP_NOTIF = 6 };

struct Hdr {
    uint32_t magic = kMagic;
    uint16_t op = 0;
    uint16_t reserved = 0;
    uint64_t id = 0;
    uint32_t nDescs = 0;
    int32_t status = 0;
    uint64_t payloadLen = 0;
    uint32_t metaLen = 0;
    uint32_t reserved2 = 0;
};
static_assert(sizeof(Hdr) == 40, "wire header");

struct WireDesc {
    uint64_t addr, len, key;
};

// ------------------------------------------------------------------ socket helpers

// Sends or receives all of `iov` (modified in place).  false: the connection is gone (or timed out).
bool ioAll(int fd, iovec *iov, int cnt, bool send) {
    while (cnt > 0) {
        msghdr m{};
        m.msg_iov = iov;
        m.msg_iovlen = static_cast<size_t>(std::min(cnt, 512));
        const ssize_t n = send ? ::sendmsg(fd, &m, MSG_NOSIGNAL) : ::recvmsg(fd, &m, 0);
        if (n < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        if (n == 0 && !send) return false;
        size_t left = static_cast<size_t>(n);
        while (cnt > 0 && left >= iov->iov_len) {
            left -= iov->iov_len;
            ++iov;
            --cnt;
        }
        if (cnt > 0 && left) {
            iov->iov_base = static_cast<char *>(iov->iov_base) + left;
            iov->iov_len -= left;
        }
        while (cnt > 0 && iov->iov_len == 0) {
            ++iov;
            --cnt;
        }
    }
    return true;
}
bool sendBuf(int fd, const void *p, size_t n) {
    iovec v{const_cast<void *>(p), n};
    return n == 0 || ioAll(fd, &v, 1, true);
}
bool recvBuf(int fd, void *p, size_t n) {
    iovec v{p, n};
    return n == 0 || ioAll(fd, &v, 1, false);
}

// Reads `n` bytes, polling the socket for up to `spin_us` first: the answer to a small message is back sooner than a
// sleeping thread is woken.  The socket's receive time-out ends a read that has stalled; with `idle_ok` it does not end
// the wait for the first byte (a connection with nothing to say is not a stalled one).
bool recvSpin(int fd, void *p, size_t n, unsigned spin_us, bool idle_ok = false) {
    if (spin_us) {
        const uint64_t end = nixl_util::nowNs() + uint64_t(spin_us) * 1000;
        do {
            const ssize_t k = ::recv(fd, p, n, MSG_DONTWAIT);
            if (k > 0) return recvBuf(fd, static_cast<char *>(p) + k, n - static_cast<size_t>(k));
            if (k == 0 || (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) return false;
#if defined(__x86_64__)
            __builtin_ia32_pause();
#endif
        } while (nixl_util::nowNs() < end);
    }
    for (;;) {
        const ssize_t k = ::recv(fd, p, n, 0);
        if (k > 0) return recvBuf(fd, static_cast<char *>(p) + k, n - static_cast<size_t>(k));
        if (k == 0) return false;
        if (errno == EINTR || (idle_ok && (errno == EAGAIN || errno == EWOULDBLOCK))) continue;
        return false;
    }
}

// A read or write that makes no progress for this long ends the connection (0: never).
void setStallTimeout(int fd, int ms) {
    const timeval tv{ms / 1000, (ms % 1000) * 1000};
    ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
}

void tuneSocket(int fd, int buf_bytes) {
    const int one = 1;
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    ::setsockopt(fd, SOL_SOCKET, SO_KEEPALIVE, &one, sizeof(one));
    if (buf_bytes > 0) {
        ::setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf_bytes, sizeof(buf_bytes));
        ::setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf_bytes, sizeof(buf_bytes));
    }
}

// A numeric IPv4 or IPv6 address (the latter with or without brackets) as a socket address.
bool toSockaddr(std::string ip, uint16_t port, sockaddr_storage &out, socklen_t &len) {
    if (ip.size() > 2 && ip.front() == '[' && ip.back() == ']') ip = ip.substr(1, ip.size() - 2);
    std::memset(&out, 0, sizeof(out));
    auto *a4 = reinterpret_cast<sockaddr_in *>(&out);
    auto *a6 = reinterpret_cast<sockaddr_in6 *>(&out);
    if (::inet_pton(AF_INET, ip.c_str(), &a4->sin_addr) == 1) {
        a4->sin_family = AF_INET;
        a4->sin_port = htons(port);
        len = sizeof(sockaddr_in);
        return true;
    }
    if (::inet_pton(AF_INET6, ip.c_str(), &a6->sin6_addr) == 1) {
        a6->sin6_family = AF_INET6;
        a6->sin6_port = htons(port);
        len = sizeof(sockaddr_in6);
        return true;
    }
    return false;
}

bool isLoopback(const std::string &a) { return a.compare(0, 4, "127.") == 0 || a == "::1" || a == "[::1]"; }

// `from`: the local address to leave from (empty: the kernel's choice by route).
int connectTo(const std::string &ip, uint16_t port, int timeout_ms, const std::string &from = "") {
    sockaddr_storage a;
    socklen_t alen = 0;
    if (!toSockaddr(ip, port, a, alen)) return -1;
    const int fd = ::socket(a.ss_family, SOCK_STREAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
    if (fd < 0) return -1;
    if (!from.empty()) {
        sockaddr_storage l;
        socklen_t llen = 0;
        if (!toSockaddr(from, 0, l, llen) || l.ss_family != a.ss_family || ::bind(fd, reinterpret_cast<sockaddr *>(&l), llen) != 0) {
            ::close(fd);
            return -1;
        }
    }
    int rc = ::connect(fd, reinterpret_cast<sockaddr *>(&a), alen);
    if (rc != 0 && errno == EINPROGRESS) {
        pollfd p{fd, POLLOUT, 0};
        int err = 0;
        socklen_t len = sizeof(err);
        if (::poll(&p, 1, timeout_ms) == 1 && ::getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &len) == 0 && err == 0) rc = 0;
    }
    if (rc != 0) {
        ::close(fd);
        return -1;
    }
    const int flags = ::fcntl(fd, F_GETFL);
    ::fcntl(fd, F_SETFL, flags & ~O_NONBLOCK);
    return fd;
}

// Orders (interface, address) pairs so that the interfaces named in `near_first` come first, in that order.
std::vector<std::string> orderByInterface(std::vector<std::pair<std::string, std::string>> found, const std::vector<std::string> &near_first) {
    std::vector<std::string> out;
    for (const auto &want : near_first)
        for (auto &f : found)
            if (f.first == want && !f.second.empty()) {
                out.push_back(f.second);
                f.second.clear();
            }
    for (const auto &f : found)
        if (!f.second.empty()) out.push_back(f.second);
    return out;
}

// The host's addresses (IPv4, then global IPv6): interfaces near GPU `gpu` first when that is known (< 0: as the kernel lists them),
// loopback last.
std::vector<std::string> hostAddresses(int gpu) {
    std::vector<std::pair<std::string, std::string>> found;
    std::vector<std::string> loop;
    ifaddrs *ifs = nullptr;
    if (::getifaddrs(&ifs) == 0) {
        std::vector<std::pair<std::string, std::string>> found6;
        for (ifaddrs *i = ifs; i; i = i->ifa_next) {
            if (!i->ifa_addr || !(i->ifa_flags & IFF_UP)) continue;
            char buf[INET6_ADDRSTRLEN];
            if (i->ifa_addr->sa_family == AF_INET) {
                if (!::inet_ntop(AF_INET, &reinterpret_cast<sockaddr_in *>(i->ifa_addr)->sin_addr, buf, sizeof(buf))) continue;
                if (i->ifa_flags & IFF_LOOPBACK) loop.push_back(buf);
                else found.emplace_back(i->ifa_name, buf);
            } else if (i->ifa_addr->sa_family == AF_INET6) {
                const in6_addr &a6 = reinterpret_cast<sockaddr_in6 *>(i->ifa_addr)->sin6_addr;
                if (IN6_IS_ADDR_LINKLOCAL(&a6) || (i->ifa_flags & IFF_LOOPBACK)) continue; // link-local needs a scope; loopback: the IPv4 one does
                if (::inet_ntop(AF_INET6, &a6, buf, sizeof(buf))) found6.emplace_back(i->ifa_name, buf);
            }
        }
        ::freeifaddrs(ifs);
        found.insert(found.end(), found6.begin(), found6.end()); // IPv4 first: what most clusters route
    }
    std::vector<std::string> near;
    if (gpu >= 0) near = nixl::pciTopology::scan().interfacesNearGpu(static_cast<size_t>(gpu));
    std::vector<std::string> out = orderByInterface(std::move(found), near);
    if (loop.empty()) loop.push_back("127.0.0.1");
    out.insert(out.end(), loop.begin(), loop.end());
    return out;
}

// ------------------------------------------------------------------ registrations

struct Region {
    uintptr_t addr = 0;
    size_t len = 0;
    uint64_t key = 0;
    int device = -1; // >= 0: device memory of that GPU
};

class LocalMD final : public nixlBackendMD {
public:
    LocalMD() : nixlBackendMD(true) {}
    Region r;
};

class RemoteMD final : public nixlBackendMD {
public:
    RemoteMD() : nixlBackendMD(false) {}
    Region r;
    bool self = false; // a registration of this very engine (loadLocalMD)
};

// One piece of local memory of a message.
struct Seg {
    uintptr_t addr;
    size_t len;
    int device;
};

// Pinned staging buffer for device memory, allocated on first use.
struct Bounce {
    void *p = nullptr;
    ~Bounce() {
        if (p) cudaFreeHost(p);
    }
    void *get() {
        if (!p && cudaHostAlloc(&p, kBounceBytes, cudaHostAllocPortable) != cudaSuccess) {
            cudaGetLastError();
            p = nullptr;
        }
        return p;
    }
};

// Sends `segs` as one payload: host memory straight from where it lies, device memory through the staging buffer.
bool sendSegs(int fd, const std::vector<Seg> &segs, Bounce &bounce) {
    std::vector<iovec> iov;
    auto flush = [&] {
        const bool ok = iov.empty() || ioAll(fd, iov.data(), static_cast<int>(iov.size()), true);
        iov.clear();
        return ok;
    };
    for (const Seg &s : segs) {
        if (s.device < 0) {
            iov.push_back({reinterpret_cast<void *>(s.addr), s.len});
            continue;
        }
        if (!flush()) return false;
        void *b = bounce.get();
        if (!b || cudaSetDevice(s.device) != cudaSuccess) return false;
        for (size_t off = 0; off < s.len; off += kBounceBytes) {
            const size_t n = std::min(kBounceBytes, s.len - off);
            if (cudaMemcpy(b, reinterpret_cast<const void *>(s.addr + off), n, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
            if (!sendBuf(fd, b, n)) return false;
        }
    }
    return flush();
}

// Receives one payload into `segs`.  `io_ok` false: the connection is gone; return false with io_ok true: a device copy
// failed (the payload has still been taken off the socket).
bool recvSegs(int fd, const std::vector<Seg> &segs, Bounce &bounce, bool &io_ok) {
    io_ok = true;
    bool copy_ok = true;
    std::vector<iovec> iov;
    auto flush = [&] {
        const bool ok = iov.empty() || ioAll(fd, iov.data(), static_cast<int>(iov.size()), false);
        iov.clear();
        return ok;
    };
    for (const Seg &s : segs) {
        if (s.device < 0) {
            iov.push_back({reinterpret_cast<void *>(s.addr), s.len});
            continue;
        }
        if (!flush()) return io_ok = false;
        void *b = bounce.get();
        if (!b) return io_ok = false; // nowhere to put the bytes: give the connection up
        if (cudaSetDevice(s.device) != cudaSuccess) copy_ok = false;
        for (size_t off = 0; off < s.len; off += kBounceBytes) {
            const size_t n = std::min(kBounceBytes, s.len - off);
            if (!recvBuf(fd, b, n)) return io_ok = false;
            if (copy_ok && cudaMemcpy(reinterpret_cast<void *>(s.addr + off), b, n, cudaMemcpyHostToDevice) != cudaSuccess) copy_ok = false;
        }
    }
    if (!flush()) return io_ok = false;
    if (!copy_ok) cudaGetLastError();
    return copy_ok;
}

bool discard(int fd, uint64_t n) {
    char scratch[65536];
    while (n) {
        const size_t k = static_cast<size_t>(std::min<uint64_t>(n, sizeof(scratch)));
        if (!recvBuf(fd, scratch, k)) return false;
        n -= k;
    }
    return true;
}

// ------------------------------------------------------------------ one post of a request

class Engine;

struct Post {
    std::atomic<int> pending{0};
    std::atomic<int> error{0};              // first failure
    std::atomic<int> status{NIXL_IN_PROG};  // what checkXfer reports
    bool hasNotif = false;
    std::string notif, peer;
    const Engine *engine = nullptr;
    uint64_t bytes = 0, startNs = 0; // for the engine's running figures of what the path delivers
    void finishOne(int st);
};

struct Msg {
    Hdr h;
    std::vector<WireDesc> descs;
    std::vector<Seg> local;
    std::string meta;
    std::shared_ptr<Post> post;
};

class ReqH final : public nixlBackendReqH {
public:
    std::shared_ptr<Post> cur;
};

// ------------------------------------------------------------------ initiator side of one connection

class ClientConn {
public:
    explicit ClientConn(int fd) : fd_(fd) {
        sender_ = std::thread([this] { senderLoop(); });
        receiver_ = std::thread([this] { receiverLoop(); });
    }
    ~ClientConn() {
        die();
        {
            std::lock_guard<std::mutex> g(qmu_);
            stop_ = true;
        }
        qcv_.notify_all();
        if (sender_.joinable()) sender_.join();
        if (receiver_.joinable()) receiver_.join();
        ::close(fd_);
    }
    bool dead() const { return dead_.load(std::memory_order_acquire); }
    // false: the connection is gone, the message was not taken.  A small message is sent by the caller itself when the
    // connection is idle, which saves waking the sender thread; everything else queues behind what is being sent.
    bool submit(const std::shared_ptr<Msg> &m, bool may_send_here = true) {
        std::unique_lock<std::mutex> g(qmu_);
        if (dead()) return false;
        const bool small = m->h.op != OP_WRITE || m->h.payloadLen <= kInlineBytes;
        if (may_send_here && small && q_.empty() && !sending_) {
            sending_ = true;
            g.unlock();
            transmit(m);
            g.lock();
            sending_ = false;
            const bool more = !q_.empty();
            g.unlock();
            if (more) qcv_.notify_one();
            return true;
        }
        q_.push_back(m);
        g.unlock();
        qcv_.notify_one();
        return true;
    }

private:
    void die() {
        std::unordered_map<uint64_t, std::shared_ptr<Msg>> lost;
        {
            std::lock_guard<std::mutex> g(imu_);
            if (dead_.exchange(true, std::memory_order_acq_rel)) return;
            lost.swap(inflight_);
        }
        ::shutdown(fd_, SHUT_RDWR);
        std::deque<std::shared_ptr<Msg>> queued;
        {
            std::lock_guard<std::mutex> g(qmu_);
            queued.swap(q_);
        }
        qcv_.notify_all();
        for (auto &kv : lost)
            if (kv.second->post) kv.second->post->finishOne(NIXL_ERR_REMOTE_DISCONNECT);
        for (auto &m : queued)
            if (m->post) m->post->finishOne(NIXL_ERR_REMOTE_DISCONNECT);
    }

    void senderLoop() {
        std::unique_lock<std::mutex> g(qmu_);
        for (;;) {
            qcv_.wait(g, [&] { return (stop_ && q_.empty()) || (!q_.empty() && !sending_); });
            if (q_.empty()) return;
            std::shared_ptr<Msg> m = std::move(q_.front());
            q_.pop_front();
            sending_ = true;
            g.unlock();
            transmit(m);
            g.lock();
            sending_ = false;
        }
    }

    // One message onto the socket; the caller holds the right to send (sending_).
    void transmit(const std::shared_ptr<Msg> &m) {
        const bool wants_reply = m->h.op == OP_WRITE || m->h.op == OP_READ;
        if (wants_reply) {
            std::lock_guard<std::mutex> g(imu_);
            if (dead()) {
                if (m->post) m->post->finishOne(NIXL_ERR_REMOTE_DISCONNECT);
                return;
            }
            inflight_[m->h.id] = m;
            waiting_.fetch_add(1, std::memory_order_relaxed);
        }
        iovec iov[3 + 64];
        int n = 0;
        iov[n++] = {&m->h, sizeof(Hdr)};
        if (!m->descs.empty()) iov[n++] = {m->descs.data(), m->descs.size() * sizeof(WireDesc)};
        if (!m->meta.empty()) iov[n++] = {m->meta.data(), m->meta.size()};
        bool ok;
        bool host_only = m->h.op == OP_WRITE && m->local.size() <= 64;
        for (size_t i = 0; host_only && i < m->local.size(); ++i) host_only = m->local[i].device < 0;
        if (host_only) { // header, ranges and payload in one call
            for (const Seg &sg : m->local) iov[n++] = {reinterpret_cast<void *>(sg.addr), sg.len};
            ok = ioAll(fd_, iov, n, true);
        } else {
            ok = ioAll(fd_, iov, n, true);
            if (ok && m->h.op == OP_WRITE) ok = sendSegs(fd_, m->local, bounce_);
        }
        if (!ok) die(); // fails what is in flight, this message included
    }

    // The next header.  While nothing is awaited the receive time-out only ends one round of waiting.
    bool recvHeader(Hdr &h, bool awaiting) {
        if (awaiting) return recvSpin(fd_, &h, sizeof(h), kSpinUs);
        for (;;) {
            const ssize_t k = ::recv(fd_, &h, sizeof(h), 0);
            if (k > 0) return recvBuf(fd_, reinterpret_cast<char *>(&h) + k, sizeof(h) - static_cast<size_t>(k));
            if (k == 0) return false;
            if (errno == EINTR) continue;
            if (errno != EAGAIN && errno != EWOULDBLOCK) return false;
            if (waiting_.load(std::memory_order_relaxed) > 0) return recvSpin(fd_, &h, sizeof(h), 0); // something was sent meanwhile: from now on silence counts
        }
    }

    void receiverLoop() {
        Bounce bounce;
        for (;;) {
            Hdr h;
            // With answers outstanding a silent peer is a stalled one; with none it is merely idle.  (A request that is
            // submitted while this thread sits in an idle wait is covered by the wait's next round.)
            const bool awaiting = waiting_.load(std::memory_order_relaxed) > 0;
            if (!recvHeader(h, awaiting) || h.magic != kMagic) break;
            std::shared_ptr<Msg> m;
            {
                std::lock_guard<std::mutex> g(imu_);
                auto it = inflight_.find(h.id);
                if (it != inflight_.end()) {
                    m = std::move(it->second);
                    inflight_.erase(it);
                    waiting_.fetch_sub(1, std::memory_order_relaxed);
                }
            }
            if (h.op == OP_ACK) {
                if (m && m->post) m->post->finishOne(h.status);
            } else if (h.op == OP_READ_REPLY) {
                int st = h.status;
                if (!m) {
                    if (!discard(fd_, h.payloadLen)) break;
                    continue;
                }
                if (st == NIXL_SUCCESS) {
                    if (h.payloadLen != m->h.payloadLen) { // not what was asked for: the stream cannot be trusted any more
                        m->post->finishOne(NIXL_ERR_BACKEND);
                        break;
                    }
                    bool io_ok = true;
                    const bool copied = recvSegs(fd_, m->local, bounce, io_ok);
                    if (!io_ok) {
                        m->post->finishOne(NIXL_ERR_REMOTE_DISCONNECT);
                        break;
                    }
                    if (!copied) st = NIXL_ERR_BACKEND;
                }
                m->post->finishOne(st);
            } else {
                if (m && m->post) m->post->finishOne(NIXL_ERR_BACKEND);
                break;
            }
        }
        die();
    }

    const int fd_;
    std::atomic<bool> dead_{false};
    std::atomic<int> waiting_{0}; // messages whose answer has not come
    bool stop_ = false, sending_ = false;
    std::mutex qmu_;
    std::condition_variable qcv_;
    std::deque<std::shared_ptr<Msg>> q_;
    std::mutex imu_;
    std::unordered_map<uint64_t, std::shared_ptr<Msg>> inflight_;
    Bounce bounce_;
    std::thread sender_, receiver_;
};

struct Peer {
    std::string agent, host;
    std::vector<std::string> addrs;
    uint16_t port = 0;
    uint64_t tag = 0;
    std::mutex connectMu; // one (re)connect at a time; never held by a connection's own threads
    std::mutex railsMu;   // the vector below, held for moments only
    std::vector<std::shared_ptr<ClientConn>> rails;
    std::atomic<uint32_t> next{0};
};

struct ServerConn {
    int fd = -1;
    std::thread th;
    std::atomic<bool> done{false};
};

void putStr(std::string &out, const std::string &s) {
    const uint32_t n = static_cast<uint32_t>(s.size());
    out.append(reinterpret_cast<const char *>(&n), sizeof(n));
    out.append(s);
}
bool getStr(const std::string &in, size_t &pos, std::string &s) {
    uint32_t n = 0;
    if (in.size() - pos < sizeof(n)) return false;
    std::memcpy(&n, in.data() + pos, sizeof(n));
    pos += sizeof(n);
    if (in.size() - pos < n) return false;
    s.assign(in, pos, n);
    pos += n;
    return true;
}

long paramLong(const nixl_b_params_t &p, const char *key, long def) {
    auto it = p.find(key);
    if (it == p.end() || it->second.empty()) return def;
    char *end = nullptr;
    const long v = std::strtol(it->second.c_str(), &end, 10);
    return end && *end == 0 ? v : def;
}

// ------------------------------------------------------------------ the engine

class Engine final : public nixlBackendEngine {
public:
    explicit Engine(const nixlBackendInitParams *p) : nixlBackendEngine(p) {
        const nixl_b_params_t &cp = getCustomParams();
        rails_ = static_cast<int>(std::clamp(paramLong(cp, "rails", 4), 1L, 64L));
        chunk_ = static_cast<size_t>(std::clamp(paramLong(cp, "chunk_bytes", 4L << 20), 4096L, 1L << 30));
        bufBytes_ = static_cast<int>(std::clamp(paramLong(cp, "socket_buffer_bytes", 4L << 20), 0L, 1L << 30));
        connectTimeoutMs_ = static_cast<int>(std::clamp(paramLong(cp, "connect_timeout_ms", 3000), 1L, 600000L));
        stallTimeoutMs_ = static_cast<int>(std::clamp(paramLong(cp, "stall_timeout_ms", 30000), 0L, 3600000L));
        const long port = std::clamp(paramLong(cp, "port", 0), 0L, 65535L);
        tag_ = nixl_util::random64();
        host_ = nixl_util::hostName();
        int n = 0;
        cuda_ = cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
        if (!cuda_) cudaGetLastError();

        const int gpu = static_cast<int>(std::clamp(paramLong(cp, "device_id", -1), -1L, 1023L));
        std::string addr;
        auto it = cp.find("address");
        if (it != cp.end()) addr = it->second;
        if (addr.empty())
            if (const char *e = std::getenv("NIXL_TCP_ADDRESS")) addr = e;
        if (!addr.empty()) addrs_ = nixl_util::split(addr, ',');
        else addrs_ = hostAddresses(gpu);
        it = cp.find("local_addresses");
        if (it != cp.end() && it->second == "auto") {
            for (const auto &a2 : hostAddresses(gpu))
                if (!isLoopback(a2)) localAddrs_.push_back(a2);
        } else if (it != cp.end() && !it->second.empty()) {
            localAddrs_ = nixl_util::split(it->second, ',');
        }

        // One socket for both families where the host has IPv6 (an IPv6 socket that also takes IPv4), else IPv4 alone.
        const int one = 1, zero = 0;
        sockaddr_storage a{};
        auto listen_on = [&](int family) {
            const int fd = ::socket(family, SOCK_STREAM | SOCK_CLOEXEC, 0);
            if (fd < 0) return -1;
            std::memset(&a, 0, sizeof(a));
            socklen_t len;
            if (family == AF_INET6) {
                auto *a6 = reinterpret_cast<sockaddr_in6 *>(&a);
                a6->sin6_family = AF_INET6;
                a6->sin6_addr = in6addr_any;
                a6->sin6_port = htons(static_cast<uint16_t>(port));
                len = sizeof(sockaddr_in6);
                if (::setsockopt(fd, IPPROTO_IPV6, IPV6_V6ONLY, &zero, sizeof(zero)) != 0) return ::close(fd), -1;
            } else {
                auto *a4 = reinterpret_cast<sockaddr_in *>(&a);
                a4->sin_family = AF_INET;
                a4->sin_addr.s_addr = htonl(INADDR_ANY);
                a4->sin_port = htons(static_cast<uint16_t>(port));
                len = sizeof(sockaddr_in);
            }
            ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
            socklen_t got = sizeof(a);
            if (::bind(fd, reinterpret_cast<sockaddr *>(&a), len) != 0 || ::listen(fd, 128) != 0 ||
                ::getsockname(fd, reinterpret_cast<sockaddr *>(&a), &got) != 0)
                return ::close(fd), -1;
            return fd;
        };
        listenFd_ = listen_on(AF_INET6);
        if (listenFd_ < 0) listenFd_ = listen_on(AF_INET);
        if (listenFd_ < 0) {
            NIXL_ERROR << "TCP backend: cannot listen on port " << port << ": " << std::strerror(errno);
            initErr = true;
            return;
        }
        port_ = ntohs(a.ss_family == AF_INET6 ? reinterpret_cast<sockaddr_in6 *>(&a)->sin6_port : reinterpret_cast<sockaddr_in *>(&a)->sin_port);
        listener_ = std::thread([this] { acceptLoop(); });
    }

    ~Engine() override {
        stop_.store(true);
        if (listenFd_ >= 0) ::shutdown(listenFd_, SHUT_RDWR);
        if (listener_.joinable()) listener_.join();
        if (listenFd_ >= 0) ::close(listenFd_);
        // Outgoing connections first: their threads call back into this object (notifications after the last reply).
        std::map<std::string, std::shared_ptr<Peer>> peers;
        {
            std::lock_guard<std::mutex> g(peersMu_);
            peers.swap(peers_);
        }
        for (auto &kv : peers) dropRails(*kv.second);
        peers.clear();
        std::vector<std::unique_ptr<ServerConn>> served;
        {
            std::lock_guard<std::mutex> g(servedMu_);
            served.swap(served_);
        }
        for (auto &c : served) {
            ::shutdown(c->fd, SHUT_RDWR);
            if (c->th.joinable()) c->th.join();
            ::close(c->fd);
        }
    }

    bool supportsRemote() const override { return true; }
    bool supportsLocal() const override { return true; }
    bool supportsNotif() const override { return true; }
    nixl_mem_list_t getSupportedMems() const override { return cuda_ ? nixl_mem_list_t{DRAM_SEG, VRAM_SEG} : nixl_mem_list_t{DRAM_SEG}; }

    // ---- registration
    nixl_status_t registerMem(const nixlBlobDesc &mem, const nixl_mem_t &nixl_mem, nixlBackendMD *&out) override {
        if (mem.len == 0 || mem.addr + mem.len < mem.addr) return NIXL_ERR_INVALID_PARAM;
        auto md = std::make_unique<LocalMD>();
        md->r.addr = mem.addr;
        md->r.len = mem.len;
        if (nixl_mem == VRAM_SEG) {
            if (!cuda_) return NIXL_ERR_NOT_SUPPORTED;
            cudaPointerAttributes attr{};
            if (cudaPointerGetAttributes(&attr, reinterpret_cast<void *>(mem.addr)) != cudaSuccess ||
                (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)) {
                cudaGetLastError();
                NIXL_ERROR << "TCP backend: address " << reinterpret_cast<void *>(mem.addr) << " is not device memory";
                return NIXL_ERR_INVALID_PARAM;
            }
            if (attr.device != static_cast<int>(mem.devId)) {
                NIXL_ERROR << "TCP backend: descriptor says device " << mem.devId << " but the memory lives on " << attr.device;
                return NIXL_ERR_INVALID_PARAM;
            }
            md->r.device = attr.device;
        } else if (nixl_mem != DRAM_SEG) {
            return NIXL_ERR_NOT_SUPPORTED;
        }
        std::unique_lock<std::shared_mutex> g(regMu_);
        do md->r.key = nixl_util::random64();
        while (md->r.key == 0 || regions_.count(md->r.key));
        regions_[md->r.key] = md->r;
        out = md.release();
        return NIXL_SUCCESS;
    }
    nixl_status_t deregisterMem(nixlBackendMD *meta) override {
        auto *md = dynamic_cast<LocalMD *>(meta);
        if (!md) return NIXL_ERR_INVALID_PARAM;
        {
            // Exclusive: a message that is being moved into or out of this range finishes first.
            std::unique_lock<std::shared_mutex> g(regMu_);
            regions_.erase(md->r.key);
        }
        delete md;
        return NIXL_SUCCESS;
    }
    nixl_status_t getPublicData(const nixlBackendMD *meta, std::string &str) const override {
        auto *md = dynamic_cast<const LocalMD *>(meta);
        if (!md) return NIXL_ERR_INVALID_PARAM;
        const uint64_t w[4] = {md->r.addr, md->r.len, md->r.key, static_cast<uint64_t>(static_cast<int64_t>(md->r.device))};
        str.assign("TCPR").append(reinterpret_cast<const char *>(w), sizeof(w));
        return NIXL_SUCCESS;
    }
    nixl_status_t loadRemoteMD(const nixlBlobDesc &input, const nixl_mem_t &, const std::string &, nixlBackendMD *&output) override {
        uint64_t w[4];
        if (input.metaInfo.size() != 4 + sizeof(w) || input.metaInfo.compare(0, 4, "TCPR") != 0) return NIXL_ERR_MISMATCH;
        std::memcpy(w, input.metaInfo.data() + 4, sizeof(w));
        auto md = std::make_unique<RemoteMD>();
        md->r.addr = w[0];
        md->r.len = w[1];
        md->r.key = w[2];
        md->r.device = static_cast<int>(static_cast<int64_t>(w[3]));
        output = md.release();
        return NIXL_SUCCESS;
    }
    nixl_status_t loadLocalMD(nixlBackendMD *input, nixlBackendMD *&output) override {
        auto *l = dynamic_cast<LocalMD *>(input);
        if (!l) return NIXL_ERR_INVALID_PARAM;
        auto md = std::make_unique<RemoteMD>();
        md->r = l->r;
        md->self = true;
        output = md.release();
        return NIXL_SUCCESS;
    }
    nixl_status_t unloadMD(nixlBackendMD *input) override {
        delete input;
        return NIXL_SUCCESS;
    }

    // ---- connections
    nixl_status_t getConnInfo(std::string &str) const override {
        str.assign("TCP1");
        putStr(str, localAgent);
        putStr(str, host_);
        putStr(str, std::to_string(port_));
        putStr(str, std::to_string(tag_));
        putStr(str, std::to_string(addrs_.size()));
        for (const auto &a : addrs_) putStr(str, a);
        return NIXL_SUCCESS;
    }
    nixl_status_t loadRemoteConnInfo(const std::string &remote_agent, const std::string &info) override {
        if (info.compare(0, 4, "TCP1") != 0) return NIXL_ERR_MISMATCH;
        size_t pos = 4;
        auto peer = std::make_shared<Peer>();
        std::string port, tag, count;
        if (!getStr(info, pos, peer->agent) || !getStr(info, pos, peer->host) || !getStr(info, pos, port) || !getStr(info, pos, tag) ||
            !getStr(info, pos, count) || peer->agent != remote_agent)
            return NIXL_ERR_MISMATCH;
        peer->port = static_cast<uint16_t>(std::strtoul(port.c_str(), nullptr, 10));
        peer->tag = std::strtoull(tag.c_str(), nullptr, 10);
        const size_t n = std::strtoul(count.c_str(), nullptr, 10);
        for (size_t i = 0; i < n; ++i) {
            std::string a;
            if (!getStr(info, pos, a)) return NIXL_ERR_MISMATCH;
            peer->addrs.push_back(a);
        }
        if (peer->port == 0 || peer->addrs.empty()) return NIXL_ERR_MISMATCH;
        std::shared_ptr<Peer> old;
        {
            std::lock_guard<std::mutex> g(peersMu_);
            auto &slot = peers_[remote_agent];
            if (slot && slot->tag == peer->tag && slot->port == peer->port) return NIXL_SUCCESS; // the same engine again
            old = std::move(slot);
            slot = peer;
        }
        if (old) dropRails(*old); // the agent of that name was started again: its old connections are of no use
        return NIXL_SUCCESS;
    }
    nixl_status_t connect(const std::string &remote_agent) override {
        if (remote_agent == localAgent) return NIXL_SUCCESS;
        auto peer = findPeer(remote_agent);
        if (!peer) return NIXL_ERR_NOT_FOUND;
        std::vector<std::shared_ptr<ClientConn>> rails;
        return railsOf(*peer, rails);
    }
    nixl_status_t disconnect(const std::string &remote_agent) override {
        std::shared_ptr<Peer> peer;
        {
            std::lock_guard<std::mutex> g(peersMu_);
            auto it = peers_.find(remote_agent);
            if (it == peers_.end()) return NIXL_ERR_NOT_FOUND;
            peer = std::move(it->second);
            peers_.erase(it);
        }
        dropRails(*peer);
        return NIXL_SUCCESS;
    }

    // ---- transfers
    nixl_status_t prepXfer(const nixl_xfer_op_t &op, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote, const std::string &,
                           nixlBackendReqH *&handle, const nixl_opt_b_args_t *) const override {
        if (op != NIXL_WRITE && op != NIXL_READ) return NIXL_ERR_INVALID_PARAM;
        if (local.descCount() != remote.descCount()) return NIXL_ERR_INVALID_PARAM;
        for (int i = 0; i < local.descCount(); ++i)
            if (local[i].len != remote[i].len) return NIXL_ERR_INVALID_PARAM;
        handle = new ReqH();
        return NIXL_SUCCESS;
    }

    nixl_status_t postXfer(const nixl_xfer_op_t &op, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote,
                           const std::string &remote_agent, nixlBackendReqH *&handle, const nixl_opt_b_args_t *opt) const override {
        auto *req = dynamic_cast<ReqH *>(handle);
        if (!req || local.descCount() != remote.descCount()) return NIXL_ERR_INVALID_PARAM;
        if (req->cur && req->cur->status.load(std::memory_order_acquire) == NIXL_IN_PROG) return NIXL_ERR_REPOST_ACTIVE;
        const int n = local.descCount();
        auto post = std::make_shared<Post>();
        post->engine = this;
        post->peer = remote_agent;
        if (opt && opt->hasNotif) {
            post->hasNotif = true;
            post->notif = opt->notifMsg;
        }
        req->cur = post;

        bool self = n > 0;
        for (int i = 0; i < n && self; ++i) {
            auto *r = dynamic_cast<RemoteMD *>(remote[i].metadataP);
            self = r && r->self;
        }
        if (self || remote_agent == localAgent) return postLocal(op, local, remote, *post);

        auto peer = findPeer(remote_agent);
        if (!peer) return fail(*post, NIXL_ERR_NOT_FOUND);
        std::vector<std::shared_ptr<ClientConn>> rails;
        if (const nixl_status_t st = railsOf(*peer, rails); st != NIXL_SUCCESS) return fail(*post, st);

        // Cut the request into messages: at most chunk_bytes each, and small enough that a request of some size
        // keeps every connection busy.
        size_t total = 0;
        for (int i = 0; i < n; ++i) total += local[i].len;
        const size_t chunk = std::min(chunk_, std::max<size_t>(256u << 10, (total + rails.size() - 1) / rails.size()));
        std::vector<std::shared_ptr<Msg>> msgs;
        std::shared_ptr<Msg> cur;
        auto open = [&] {
            cur = std::make_shared<Msg>();
            cur->h.op = op == NIXL_WRITE ? OP_WRITE : OP_READ;
            cur->h.id = nextId_.fetch_add(1, std::memory_order_relaxed);
            cur->post = post;
        };
        auto close = [&] {
            if (!cur || cur->descs.empty()) return;
            cur->h.nDescs = static_cast<uint32_t>(cur->descs.size());
            cur->h.metaLen = static_cast<uint32_t>(cur->descs.size() * sizeof(WireDesc));
            msgs.push_back(std::move(cur));
            cur.reset();
        };
        for (int i = 0; i < n; ++i) {
            auto *l = dynamic_cast<LocalMD *>(local[i].metadataP);
            auto *r = dynamic_cast<RemoteMD *>(remote[i].metadataP);
            if (!l || !r || local[i].len != remote[i].len) return fail(*post, NIXL_ERR_INVALID_PARAM);
            size_t off = 0;
            while (off < local[i].len) {
                if (!cur) open();
                const size_t room = chunk - static_cast<size_t>(cur->h.payloadLen);
                const size_t take = std::min(room, local[i].len - off);
                cur->descs.push_back({remote[i].addr + off, take, r->r.key});
                cur->local.push_back({local[i].addr + off, take, l->r.device});
                cur->h.payloadLen += take;
                off += take;
                if (cur->h.payloadLen >= chunk || cur->descs.size() >= kMaxDescsPerMsg) close();
            }
        }
        close();
        if (msgs.empty()) { // nothing but empty descriptors
            post->pending.store(1);
            post->finishOne(NIXL_SUCCESS);
            return static_cast<nixl_status_t>(post->status.load());
        }
        post->bytes = total;
        post->startNs = nixl_util::nowNs();
        post->pending.store(static_cast<int>(msgs.size()), std::memory_order_release);
        // All messages but the last are handed to the connections' sender threads; the last one the posting thread may
        // send itself, while the others are already on their way: a request of one message costs no thread wake-up at
        // all, and a larger one keeps every connection busy at once.
        for (size_t i = 0; i < msgs.size(); ++i) {
            const uint32_t at = peer->next.fetch_add(1, std::memory_order_relaxed);
            const bool last = i + 1 == msgs.size();
            bool taken = false;
            for (size_t k = 0; k < rails.size() && !taken; ++k) taken = rails[(at + k) % rails.size()]->submit(msgs[i], last);
            if (!taken) post->finishOne(NIXL_ERR_REMOTE_DISCONNECT);
        }
        return static_cast<nixl_status_t>(post->status.load(std::memory_order_acquire));
    }

    nixl_status_t checkXfer(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<ReqH *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        if (!req->cur) return NIXL_ERR_NOT_POSTED;
        return static_cast<nixl_status_t>(req->cur->status.load(std::memory_order_acquire));
    }
    nixl_status_t releaseReqH(nixlBackendReqH *handle) const override {
        // Messages in flight keep their own reference to the post; user memory must stay valid until they have
        // completed, as with every backend (the agent only releases a request that is running when told to).
        delete handle;
        return NIXL_SUCCESS;
    }

    // ---- notifications
    nixl_status_t getNotifs(notif_list_t &list) override {
        std::lock_guard<std::mutex> g(notifMu_);
        for (auto &n : notifs_) list.push_back(std::move(n));
        notifs_.clear();
        return NIXL_SUCCESS;
    }
    nixl_status_t genNotif(const std::string &remote_agent, const std::string &msg) const override {
        if (remote_agent == localAgent) {
            pushNotif(localAgent, msg);
            return NIXL_SUCCESS;
        }
        auto peer = findPeer(remote_agent);
        if (!peer) return NIXL_ERR_NOT_FOUND;
        std::vector<std::shared_ptr<ClientConn>> rails;
        if (const nixl_status_t st = railsOf(*peer, rails); st != NIXL_SUCCESS) return st;
        return sendNotif(remote_agent, msg) ? NIXL_SUCCESS : NIXL_ERR_REMOTE_DISCONNECT;
    }

    // What finished requests have shown: small ones give the round trip, large ones the rate (running averages).
    void observe(uint64_t bytes, uint64_t ns) const {
        auto blend = [](std::atomic<double> &avg, double sample) {
            const double old = avg.load(std::memory_order_relaxed);
            avg.store(old == 0 ? sample : old * 0.875 + sample * 0.125, std::memory_order_relaxed);
        };
        if (bytes <= (16u << 10)) blend(seenLatencyUs_, static_cast<double>(ns) / 1e3);
        else if (bytes >= (1u << 20) && ns) blend(seenBytesPerUs_, static_cast<double>(bytes) / (static_cast<double>(ns) / 1e3));
    }
    // Round trip plus bytes over the rate: measured on this engine's own finished requests when there are any, else a
    // guess for a 25 Gb/s link.  The margin is wide: a shared network does not promise anything.
    nixl_status_t estimateXferCost(const nixl_xfer_op_t &, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &, const std::string &,
                                   nixlBackendReqH *const &, std::chrono::microseconds &duration, std::chrono::microseconds &err_margin,
                                   nixl_cost_t &method, const nixl_opt_args_t *) const override {
        double bytes = 0;
        for (const auto &d : local) bytes += static_cast<double>(d.len);
        const double lat = seenLatencyUs_.load(std::memory_order_relaxed), rate = seenBytesPerUs_.load(std::memory_order_relaxed);
        const double us = (lat > 0 ? lat : 100.0) + bytes / (rate > 0 ? rate : 3000.0);
        duration = std::chrono::microseconds(static_cast<int64_t>(us + 0.5));
        err_margin = std::chrono::microseconds(static_cast<int64_t>(us * 0.5 + 1.0));
        method = nixl_cost_t::ANALYTICAL_BACKEND;
        return NIXL_SUCCESS;
    }

    // Queues a notification on the first live connection to `agent` (never opens one: connections' own threads call this).
    bool sendNotif(const std::string &agent, const std::string &msg) const {
        if (agent == localAgent) {
            pushNotif(localAgent, msg);
            return true;
        }
        auto peer = findPeer(agent);
        if (!peer) return false;
        auto m = std::make_shared<Msg>();
        m->h.op = OP_NOTIF;
        m->h.id = nextId_.fetch_add(1, std::memory_order_relaxed);
        m->meta = msg;
        m->h.metaLen = static_cast<uint32_t>(msg.size());
        std::lock_guard<std::mutex> g(peer->railsMu);
        for (auto &r : peer->rails)
            if (r->submit(m)) return true;
        return false;
    }

private:
    nixl_status_t fail(Post &post, nixl_status_t st) const {
        post.error.store(st);
        post.status.store(st, std::memory_order_release);
        return st;
    }

    void pushNotif(const std::string &from, const std::string &msg) const {
        std::lock_guard<std::mutex> g(notifMu_);
        notifs_.emplace_back(from, msg);
    }

    std::shared_ptr<Peer> findPeer(const std::string &agent) const {
        std::lock_guard<std::mutex> g(peersMu_);
        auto it = peers_.find(agent);
        return it == peers_.end() ? nullptr : it->second;
    }

    void dropRails(Peer &peer) const {
        std::lock_guard<std::mutex> c(peer.connectMu);
        std::vector<std::shared_ptr<ClientConn>> old;
        {
            std::lock_guard<std::mutex> g(peer.railsMu);
            old.swap(peer.rails);
        }
        old.clear(); // joins their threads; railsMu is free, so a thread on its way through sendNotif gets out
    }

    // One connection to the peer's listener, introduced and accepted; nullptr if no address answers as that engine.
    // Connection number `rail` starts with the peer's address number `rail` (of those that apply) and leaves from local
    // address number `rail` when local addresses are configured: with several interfaces on either side the
    // connections spread over them.
    std::shared_ptr<ClientConn> dial(const Peer &peer, size_t rail) const {
        std::vector<std::string> order;
        const bool same_host = peer.host == host_;
        auto is_loop = [](const std::string &a) { return isLoopback(a); };
        if (same_host)
            for (const auto &a : peer.addrs)
                if (is_loop(a)) order.push_back(a);
        for (const auto &a : peer.addrs)
            if (!is_loop(a)) order.push_back(a);
        if (order.empty()) order = peer.addrs; // only a loopback address was published (tests, an explicit "address")
        // (loopback addresses come first for a peer on this host; they take turns among themselves, the rest follows)
        size_t group = 0;
        while (group < order.size() && is_loop(order[group]) == is_loop(order.front())) ++group;
        std::rotate(order.begin(), order.begin() + static_cast<long>(rail % group), order.begin() + static_cast<long>(group));
        const std::string from = localAddrs_.empty() ? std::string() : localAddrs_[rail % localAddrs_.size()];
        for (const auto &a : order) {
            int fd = connectTo(a, peer.port, connectTimeoutMs_, from);
            if (fd < 0 && !from.empty()) fd = connectTo(a, peer.port, connectTimeoutMs_); // no route from there: any way will do

            if (fd < 0) continue;
            tuneSocket(fd, bufBytes_);
            // Say who we are and whom we expect: the same port number on another machine is somebody else.
            std::string meta;
            putStr(meta, localAgent);
            putStr(meta, peer.agent);
            putStr(meta, std::to_string(peer.tag));
            Hdr h;
            h.op = OP_HELLO;
            h.metaLen = static_cast<uint32_t>(meta.size());
            timeval tv{connectTimeoutMs_ / 1000, (connectTimeoutMs_ % 1000) * 1000};
            ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
            Hdr reply;
            if (sendBuf(fd, &h, sizeof(h)) && sendBuf(fd, meta.data(), meta.size()) && recvBuf(fd, &reply, sizeof(reply)) &&
                reply.magic == kMagic && reply.op == OP_ACK && reply.status == NIXL_SUCCESS) {
                setStallTimeout(fd, stallTimeoutMs_);
                return std::make_shared<ClientConn>(fd);
            }
            ::close(fd);
        }
        return nullptr;
    }

    // The peer's live connections, opened or replaced as needed.
    nixl_status_t railsOf(Peer &peer, std::vector<std::shared_ptr<ClientConn>> &out) const {
        {
            std::lock_guard<std::mutex> g(peer.railsMu);
            bool all = !peer.rails.empty();
            for (auto &r : peer.rails) all = all && !r->dead();
            if (all) {
                out = peer.rails;
                return NIXL_SUCCESS;
            }
        }
        std::lock_guard<std::mutex> c(peer.connectMu);
        std::vector<std::shared_ptr<ClientConn>> keep, old;
        {
            std::lock_guard<std::mutex> g(peer.railsMu);
            old = peer.rails;
        }
        for (auto &r : old)
            if (!r->dead()) keep.push_back(r);
        while (static_cast<int>(keep.size()) < rails_) {
            auto c2 = dial(peer, keep.size());
            if (!c2) break;
            keep.push_back(std::move(c2));
        }
        {
            std::lock_guard<std::mutex> g(peer.railsMu);
            peer.rails = keep;
        }
        old.clear(); // the dead ones go here, outside railsMu
        if (keep.empty()) {
            NIXL_WARN << "TCP backend: agent " << peer.agent << " does not answer on port " << peer.port;
            return NIXL_ERR_REMOTE_DISCONNECT;
        }
        out = std::move(keep);
        return NIXL_SUCCESS;
    }

    nixl_status_t postLocal(const nixl_xfer_op_t &op, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote, Post &post) const {
        for (int i = 0; i < local.descCount(); ++i) {
            auto *l = dynamic_cast<LocalMD *>(local[i].metadataP);
            auto *r = dynamic_cast<RemoteMD *>(remote[i].metadataP);
            if (!l || !r || local[i].len != remote[i].len) return fail(post, NIXL_ERR_INVALID_PARAM);
            void *dst = reinterpret_cast<void *>(op == NIXL_WRITE ? remote[i].addr : local[i].addr);
            const void *src = reinterpret_cast<const void *>(op == NIXL_WRITE ? local[i].addr : remote[i].addr);
            if (l->r.device < 0 && r->r.device < 0) {
                std::memmove(dst, src, local[i].len);
            } else if (cudaMemcpy(dst, src, local[i].len, cudaMemcpyDefault) != cudaSuccess) {
                cudaGetLastError();
                return fail(post, NIXL_ERR_BACKEND);
            }
        }
        if (post.hasNotif) pushNotif(localAgent, post.notif);
        post.status.store(NIXL_SUCCESS, std::memory_order_release);
        return NIXL_SUCCESS;
    }

    // ---- target side
    bool resolve(const WireDesc &d, Seg &out) const { // regMu_ held (shared)
        auto it = regions_.find(d.key);
        if (it == regions_.end()) return false;
        const Region &r = it->second;
        if (d.addr < r.addr || d.len > r.len || d.addr - r.addr > r.len - d.len) return false;
        out = {static_cast<uintptr_t>(d.addr), static_cast<size_t>(d.len), r.device};
        return true;
    }

    void acceptLoop() {
        while (!stop_.load()) {
            const int fd = ::accept4(listenFd_, nullptr, nullptr, SOCK_CLOEXEC);
            if (fd < 0) {
                if (errno == EINTR || errno == ECONNABORTED) continue;
                if (stop_.load()) break;
                std::this_thread::sleep_for(std::chrono::milliseconds(10)); // out of descriptors and the like
                continue;
            }
            if (stop_.load()) {
                ::close(fd);
                break;
            }
            tuneSocket(fd, bufBytes_);
            // until it has introduced itself a connection may not keep a thread waiting
            const timeval intro{connectTimeoutMs_ / 1000, (connectTimeoutMs_ % 1000) * 1000};
            ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &intro, sizeof(intro));
            auto c = std::make_unique<ServerConn>();
            c->fd = fd;
            ServerConn *raw = c.get();
            std::lock_guard<std::mutex> g(servedMu_);
            for (auto it = served_.begin(); it != served_.end();) { // connections that have ended since
                if ((*it)->done.load()) {
                    (*it)->th.join();
                    ::close((*it)->fd);
                    it = served_.erase(it);
                } else ++it;
            }
            raw->th = std::thread([this, raw] {
                serve(raw->fd);
                ::shutdown(raw->fd, SHUT_RDWR); // the other side sees the end now; the descriptor itself is closed when the thread is reaped
                raw->done.store(true);
            });
            served_.push_back(std::move(c));
        }
    }

    void serve(int fd) {
        Bounce bounce;
        std::string from;
        std::vector<WireDesc> descs;
        std::vector<Seg> segs;
        for (bool first = true;; first = false) {
            Hdr h;
            if (!recvSpin(fd, &h, sizeof(h), first ? 0 : kSpinUs, !from.empty()) || h.magic != kMagic || h.metaLen > (64u << 20) || h.nDescs > kMaxDescsPerMsg) return;
            Hdr reply;
            reply.id = h.id;
            if (from.empty() && (h.op != OP_HELLO || h.metaLen > 4096)) return; // a stranger gets to say who it is, briefly, and nothing else
            if (h.op == OP_HELLO || h.op == OP_NOTIF) {
                std::string meta(h.metaLen, '\0');
                if (!recvBuf(fd, meta.data(), meta.size())) return;
                if (h.op == OP_NOTIF) {
                    if (from.empty()) return; // not introduced
                    pushNotif(from, meta);
                    continue;
                }
                size_t pos = 0;
                std::string who, to, tag;
                const bool ok = getStr(meta, pos, who) && getStr(meta, pos, to) && getStr(meta, pos, tag) && to == localAgent &&
                    std::strtoull(tag.c_str(), nullptr, 10) == tag_;
                reply.op = OP_ACK;
                reply.status = ok ? NIXL_SUCCESS : NIXL_ERR_MISMATCH;
                if (!sendBuf(fd, &reply, sizeof(reply)) || !ok) return;
                from = who;
                setStallTimeout(fd, stallTimeoutMs_); // a known peer may stay silent between messages for as long as it likes, not inside one
                continue;
            }
            if ((h.op != OP_WRITE && h.op != OP_READ) || from.empty() || h.metaLen != h.nDescs * sizeof(WireDesc)) return;
            descs.resize(h.nDescs);
            if (!recvBuf(fd, descs.data(), h.metaLen)) return;
            {
                std::shared_lock<std::shared_mutex> g(regMu_); // the ranges stay registered while the bytes move
                segs.resize(descs.size());
                uint64_t sum = 0;
                bool ok = true;
                for (size_t i = 0; i < descs.size() && ok; ++i) {
                    ok = resolve(descs[i], segs[i]);
                    sum += descs[i].len;
                }
                ok = ok && sum == h.payloadLen;
                NIXL_TCP_ORDER_ACQUIRE(&served_);
                if (h.op == OP_WRITE) {
                    reply.op = OP_ACK;
                    if (ok) {
                        bool io_ok = true;
                        const bool copied = recvSegs(fd, segs, bounce, io_ok);
                        if (!io_ok) return;
                        reply.status = copied ? NIXL_SUCCESS : NIXL_ERR_BACKEND;
                        NIXL_TCP_ORDER_RELEASE(&served_);
                    } else {
                        g.unlock();
                        if (!discard(fd, h.payloadLen)) return;
                        reply.status = NIXL_ERR_INVALID_PARAM;
                    }
                    if (!sendBuf(fd, &reply, sizeof(reply))) return;
                } else {
                    reply.op = OP_READ_REPLY;
                    reply.status = ok ? NIXL_SUCCESS : NIXL_ERR_INVALID_PARAM;
                    reply.payloadLen = ok ? sum : 0;
                    if (!sendBuf(fd, &reply, sizeof(reply))) return;
                    if (ok && !sendSegs(fd, segs, bounce)) return;
                    NIXL_TCP_ORDER_RELEASE(&served_);
                }
            }
        }
    }

    int rails_ = 4, bufBytes_ = 0, connectTimeoutMs_ = 3000, stallTimeoutMs_ = 30000;
    size_t chunk_ = 4u << 20;
    bool cuda_ = false;
    uint64_t tag_ = 0;
    uint16_t port_ = 0;
    std::string host_;
    std::vector<std::string> addrs_;      // published: where the listener can be reached
    std::vector<std::string> localAddrs_; // where outgoing connections leave from, in turn (empty: the kernel's choice)
    int listenFd_ = -1;
    std::atomic<bool> stop_{false};
    std::thread listener_;
    mutable std::shared_mutex regMu_;
    std::unordered_map<uint64_t, Region> regions_;
    mutable std::mutex peersMu_;
    mutable std::map<std::string, std::shared_ptr<Peer>> peers_;
    mutable std::mutex notifMu_;
    mutable notif_list_t notifs_;
    std::mutex servedMu_;
    std::vector<std::unique_ptr<ServerConn>> served_;
    mutable std::atomic<uint64_t> nextId_{1};
    mutable std::atomic<double> seenLatencyUs_{0}, seenBytesPerUs_{0};
};

void Post::finishOne(int st) {
    if (st != NIXL_SUCCESS) {
        int expected = 0;
        error.compare_exchange_strong(expected, st);
    }
    if (pending.fetch_sub(1, std::memory_order_acq_rel) != 1) return;
    int e = error.load();
    // The notification goes out before the request reads as complete: whoever sees SUCCESS may tear the agent down.
    if (e == NIXL_SUCCESS && hasNotif && !engine->sendNotif(peer, notif)) e = NIXL_ERR_REMOTE_DISCONNECT;
    if (e == NIXL_SUCCESS && startNs) engine->observe(bytes, nixl_util::nowNs() - startNs);
    status.store(e, std::memory_order_release);
}

} // namespace

extern "C" NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init() {
    return nixlBackendPluginCreator<Engine>::create(NIXL_PLUGIN_API_VERSION, NIXL_TCP_PLUGIN_NAME, "0.1.0",
                                                    {{"rails", "4"},
                                                     {"chunk_bytes", "4194304"},
                                                     {"port", "0"},
                                                     {"address", ""},
                                                     {"local_addresses", ""},
                                                     {"device_id", ""},
                                                     {"socket_buffer_bytes", "4194304"},
                                                     {"connect_timeout_ms", "3000"},
                                                     {"stall_timeout_ms", "30000"}},
                                                    {DRAM_SEG, VRAM_SEG});
}
extern "C" NIXL_PLUGIN_EXPORT void nixl_plugin_fini() {}

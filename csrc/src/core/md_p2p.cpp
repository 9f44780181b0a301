#include "core/md_p2p.h"

#include <arpa/inet.h>
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>

#include "utils/log.h"
#include "utils/misc.h"

namespace nixl_p2p {
namespace {
constexpr char kLoad[] = "NIXLCOMM:LOAD";
constexpr char kSend[] = "NIXLCOMM:SEND";
constexpr char kInvl[] = "NIXLCOMM:INVL";

using nixl_util::nowMs;

bool writeAll(int fd, const char *p, size_t n) {
    while (n) {
        const ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
        if (w < 0) {
            if (errno == EINTR) continue;
            if (errno == EAGAIN || errno == EWOULDBLOCK) {
                pollfd pf{fd, POLLOUT, 0};
                if (::poll(&pf, 1, kBodyTimeoutMs) <= 0) return false;
                continue;
            }
            return false;
        }
        p += w;
        n -= static_cast<size_t>(w);
    }
    return true;
}

bool readAll(int fd, char *p, size_t n, int timeout_ms) {
    const int64_t deadline = nowMs() + timeout_ms;
    while (n) {
        const int64_t left = deadline - nowMs();
        if (left <= 0) return false;
        pollfd pf{fd, POLLIN, 0};
        const int pr = ::poll(&pf, 1, static_cast<int>(left));
        if (pr < 0 && errno == EINTR) continue;
        if (pr <= 0) return false;
        const ssize_t r = ::recv(fd, p, n, 0);
        if (r == 0) return false;
        if (r < 0) {
            if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
            return false;
        }
        p += r;
        n -= static_cast<size_t>(r);
    }
    return true;
}
} // namespace

bool sendFrame(int fd, const std::string &body) {
    const uint64_t n = body.size();
    return writeAll(fd, reinterpret_cast<const char *>(&n), sizeof(n)) && writeAll(fd, body.data(), body.size());
}

bool recvFrame(int fd, std::string &body, int timeout_ms) {
    uint64_t n = 0;
    if (!readAll(fd, reinterpret_cast<char *>(&n), sizeof(n), timeout_ms)) return false;
    if (n > kMaxFrame) {
        NIXL_ERROR << "p2p metadata: frame of " << n << " bytes exceeds the limit";
        return false;
    }
    // Memory follows the bytes that have arrived, not the length a stranger announced.
    body.clear();
    const int64_t deadline = nowMs() + kBodyTimeoutMs;
    for (uint64_t got = 0; got < n;) {
        const size_t piece = static_cast<size_t>(std::min<uint64_t>(n - got, 1u << 20));
        const int64_t left = deadline - nowMs();
        if (left <= 0) return false;
        body.resize(static_cast<size_t>(got) + piece);
        if (!readAll(fd, body.data() + got, piece, static_cast<int>(left))) return false;
        got += piece;
    }
    return true;
}

int dial(const std::string &ip, int port, int timeout_ms) {
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_UNSPEC;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(ip.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || !res) return -1;
    int fd = -1;
    for (addrinfo *a = res; a; a = a->ai_next) {
        fd = ::socket(a->ai_family, a->ai_socktype | SOCK_NONBLOCK, a->ai_protocol);
        if (fd < 0) continue;
        int rc = ::connect(fd, a->ai_addr, a->ai_addrlen);
        if (rc != 0 && errno == EINPROGRESS) {
            pollfd pf{fd, POLLOUT, 0};
            if (::poll(&pf, 1, timeout_ms) == 1) {
                int err = 0;
                socklen_t len = sizeof(err);
                getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &len);
                rc = err ? -1 : 0;
            } else rc = -1;
        }
        if (rc == 0) break;
        ::close(fd);
        fd = -1;
    }
    freeaddrinfo(res);
    if (fd >= 0) {
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    }
    return fd;
}
} // namespace nixl_p2p

using namespace nixl_p2p;

nixlP2PListener::nixlP2PListener(nixlMetadataContext &ctx, uint16_t port, uint64_t poll_delay_us)
    : ctx_(ctx), delayUs_(poll_delay_us ? poll_delay_us : 100000) {
    listenFd_ = ::socket(AF_INET, SOCK_STREAM | SOCK_NONBLOCK, 0);
    if (listenFd_ < 0) return;
    int one = 1;
    setsockopt(listenFd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
    addr.sin_port = htons(port);
    if (::bind(listenFd_, reinterpret_cast<sockaddr *>(&addr), sizeof(addr)) != 0 || ::listen(listenFd_, 64) != 0) {
        NIXL_ERROR << "p2p metadata listener: cannot bind port " << port << ": " << std::strerror(errno);
        ::close(listenFd_);
        listenFd_ = -1;
        return;
    }
    socklen_t len = sizeof(addr);
    getsockname(listenFd_, reinterpret_cast<sockaddr *>(&addr), &len);
    port_ = ntohs(addr.sin_port);
}

nixlP2PListener::~nixlP2PListener() {
    stop();
    if (listenFd_ >= 0) ::close(listenFd_);
    for (const Client &c : clients_) ::close(c.fd);
}

void nixlP2PListener::start() {
    if (listenFd_ < 0 || th_.joinable()) return;
    stop_ = false;
    th_ = std::thread([this] { loop(); });
}

void nixlP2PListener::stop() {
    stop_ = true;
    if (th_.joinable()) th_.join();
}

void nixlP2PListener::loop() {
    const int wait_ms = static_cast<int>(std::max<uint64_t>(1, std::min<uint64_t>(delayUs_ / 1000, 200)));
    constexpr size_t kMaxClients = 256;
    while (!stop_) {
        std::vector<pollfd> fds;
        fds.push_back({listenFd_, POLLIN, 0});
        for (const Client &c : clients_) fds.push_back({c.fd, POLLIN, 0});
        const int pr = ::poll(fds.data(), fds.size(), wait_ms);
        const size_t polled = clients_.size();
        if (pr > 0 && (fds[0].revents & POLLIN)) {
            const int fd = ::accept4(listenFd_, nullptr, nullptr, SOCK_NONBLOCK | SOCK_CLOEXEC);
            if (fd >= 0 && clients_.size() >= kMaxClients) {
                ::close(fd); // full house: better to refuse than to let strangers push the peers out
            } else if (fd >= 0) {
                int one = 1;
                setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
                Client c;
                c.fd = fd;
                clients_.push_back(std::move(c));
            }
        }
        const int64_t now = nowMs();
        for (size_t i = 0; i < polled; ++i) {
            Client &c = clients_[i];
            bool keep = true;
            if (pr > 0 && (fds[i + 1].revents & (POLLIN | POLLHUP | POLLERR))) keep = advance(c);
            if (keep && c.startedMs && now - c.startedMs > kBodyTimeoutMs) keep = false; // a frame must not take for ever
            if (!keep) {
                ::close(c.fd);
                c.fd = -1;
            }
        }
        clients_.erase(std::remove_if(clients_.begin(), clients_.end(), [](const Client &c) { return c.fd < 0; }), clients_.end());
    }
}

bool nixlP2PListener::advance(Client &c) {
    for (;;) {
        const bool have_len = c.buf.size() >= sizeof(uint64_t);
        if (have_len && c.buf.size() == sizeof(uint64_t)) {
            std::memcpy(&c.frameLen, c.buf.data(), sizeof(uint64_t));
            if (c.frameLen > kMaxFrame) {
                NIXL_ERROR << "p2p metadata: frame of " << c.frameLen << " bytes exceeds the limit";
                return false;
            }
        }
        const uint64_t want = have_len ? sizeof(uint64_t) + c.frameLen : sizeof(uint64_t);
        if (have_len && c.buf.size() == want) { // a whole frame
            const std::string frame = c.buf.substr(sizeof(uint64_t));
            c.buf.clear();
            c.startedMs = 0;
            if (!handle(c, frame)) return false;
            continue;
        }
        char tmp[65536];
        const size_t room = static_cast<size_t>(std::min<uint64_t>(want - c.buf.size(), sizeof(tmp)));
        const ssize_t r = ::recv(c.fd, tmp, room, 0);
        if (r == 0) return false;
        if (r < 0) return errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK; // nothing more for now
        if (c.buf.empty()) c.startedMs = nowMs();
        c.buf.append(tmp, static_cast<size_t>(r));
    }
}

// One frame from a client; false drops the connection (protocol error, or the answer could not be sent).
bool nixlP2PListener::handle(Client &c, const std::string &body) {
    const int fd = c.fd;
    auto drop = [] { return false; };

    auto is = [&](const char *cmd) { return body.compare(0, std::strlen(cmd), cmd) == 0; };
    if (is(kLoad)) {
        std::string who;
        const nixl_status_t st = ctx_.mdLoadRemote(body.substr(std::strlen(kLoad)), who);
        if (st != NIXL_SUCCESS) NIXL_ERROR << "p2p metadata: received metadata was rejected: " << nixlEnumStrings::statusStr(st);
    } else if (is(kSend)) {
        nixl_blob_t mine;
        if (ctx_.mdGetLocal(mine) == NIXL_SUCCESS) {
            if (!sendFrame(fd, std::string(kLoad) + mine)) return drop();
        } else {
            sendFrame(fd, std::string(kInvl) + ctx_.mdAgentName()); // nothing to offer
        }
    } else if (is(kInvl)) {
        ctx_.mdInvalidateRemote(body.substr(std::strlen(kInvl)));
    } else {
        NIXL_ERROR << "p2p metadata: unknown command";
        return drop();
    }
    return true;
}

#include "core/md_tcpstore.h"

#include <chrono>
#include <cstring>
#include <sys/socket.h>
#include <thread>
#include <unistd.h>

#include "core/md_p2p.h"
#include "utils/config.h"
#include "utils/log.h"

namespace {
constexpr uint32_t kMagic = 0x3C85F7CE;
// c10d TCPStore query codes.
enum : uint8_t { Q_VALIDATE = 0, Q_SET = 1, Q_COMPARE_SET = 2, Q_GET = 3, Q_ADD = 4, Q_CHECK = 5, Q_WAIT = 6,
                 Q_GETNUMKEYS = 7, Q_DELETE_KEY = 8, Q_APPEND = 9, Q_MULTI_GET = 10, Q_MULTI_SET = 11,
                 Q_CANCEL_WAIT = 12, Q_PING = 13 };
enum : uint8_t { CHECK_READY = 0, CHECK_NOT_READY = 1 };
} // namespace

nixlTcpStoreClient::nixlTcpStoreClient(const std::string &host, int port, int connect_timeout_ms, int op_timeout_ms)
    : host_(host), port_(port), connectMs_(connect_timeout_ms), opMs_(op_timeout_ms) {
    fd_ = nixl_p2p::dial(host_, port_, connectMs_);
    if (fd_ >= 0 && !handshake()) reset();
}

nixlTcpStoreClient::~nixlTcpStoreClient() { reset(); }

void nixlTcpStoreClient::reset() {
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
}

void nixlTcpStoreClient::putStr(std::string &buf, const std::string &s) {
    const uint64_t n = s.size();
    buf.append(reinterpret_cast<const char *>(&n), sizeof(n));
    buf.append(s);
}

bool nixlTcpStoreClient::sendAll(const std::string &buf) {
    size_t off = 0;
    while (off < buf.size()) {
        const ssize_t w = ::send(fd_, buf.data() + off, buf.size() - off, MSG_NOSIGNAL);
        if (w <= 0) {
            if (w < 0 && (errno == EINTR || errno == EAGAIN)) {
                std::this_thread::sleep_for(std::chrono::microseconds(50));
                continue;
            }
            return false;
        }
        off += static_cast<size_t>(w);
    }
    return true;
}

bool nixlTcpStoreClient::recvAll(void *p, size_t n) {
    // Reuse the framed reader's timeout logic through a tiny shim: poll + recv.
    char *c = static_cast<char *>(p);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(opMs_);
    while (n) {
        if (std::chrono::steady_clock::now() > deadline) return false;
        const ssize_t r = ::recv(fd_, c, n, MSG_DONTWAIT);
        if (r == 0) return false;
        if (r < 0) {
            if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) {
                std::this_thread::sleep_for(std::chrono::microseconds(50));
                continue;
            }
            return false;
        }
        c += r;
        n -= static_cast<size_t>(r);
    }
    return true;
}

bool nixlTcpStoreClient::handshake() {
    std::string buf;
    buf.push_back(static_cast<char>(Q_VALIDATE));
    buf.append(reinterpret_cast<const char *>(&kMagic), sizeof(kMagic));
    const uint32_t nonce = static_cast<uint32_t>(::getpid());
    buf.push_back(static_cast<char>(Q_PING));
    buf.append(reinterpret_cast<const char *>(&nonce), sizeof(nonce));
    if (!sendAll(buf)) return false;
    uint32_t echo = 0;
    return recvAll(&echo, sizeof(echo)) && echo == nonce;
}

nixl_status_t nixlTcpStoreClient::set(const std::string &key, const std::string &value) {
    std::lock_guard<std::mutex> g(mu_);
    if (fd_ < 0) return NIXL_ERR_BACKEND;
    std::string buf;
    buf.push_back(static_cast<char>(Q_SET));
    putStr(buf, "/" + key);
    putStr(buf, value);
    if (!sendAll(buf)) {
        reset();
        return NIXL_ERR_BACKEND;
    }
    return NIXL_SUCCESS;
}

nixl_status_t nixlTcpStoreClient::check(const std::vector<std::string> &keys, bool &all_present) {
    std::lock_guard<std::mutex> g(mu_);
    if (fd_ < 0) return NIXL_ERR_BACKEND;
    std::string buf;
    buf.push_back(static_cast<char>(Q_CHECK));
    const uint64_t n = keys.size();
    buf.append(reinterpret_cast<const char *>(&n), sizeof(n));
    for (auto &k : keys) putStr(buf, "/" + k);
    uint8_t resp = CHECK_NOT_READY;
    if (!sendAll(buf) || !recvAll(&resp, 1)) {
        reset();
        return NIXL_ERR_BACKEND;
    }
    all_present = resp == CHECK_READY;
    return NIXL_SUCCESS;
}

nixl_status_t nixlTcpStoreClient::get(const std::string &key, std::string &value) {
    bool present = false;
    if (auto st = check({key}, present); st != NIXL_SUCCESS) return st;
    if (!present) return NIXL_ERR_NOT_FOUND; // GET on a missing key would block inside the server
    std::lock_guard<std::mutex> g(mu_);
    if (fd_ < 0) return NIXL_ERR_BACKEND;
    std::string buf;
    buf.push_back(static_cast<char>(Q_GET));
    putStr(buf, "/" + key);
    uint64_t n = 0;
    if (!sendAll(buf) || !recvAll(&n, sizeof(n)) || n > nixl_p2p::kMaxFrame) {
        reset();
        return NIXL_ERR_BACKEND;
    }
    value.resize(n);
    if (n && !recvAll(value.data(), n)) {
        reset();
        return NIXL_ERR_BACKEND;
    }
    return NIXL_SUCCESS;
}

nixl_status_t nixlTcpStoreClient::deleteKey(const std::string &key) {
    std::lock_guard<std::mutex> g(mu_);
    if (fd_ < 0) return NIXL_ERR_BACKEND;
    std::string buf;
    buf.push_back(static_cast<char>(Q_DELETE_KEY));
    putStr(buf, "/" + key);
    int64_t deleted = 0;
    if (!sendAll(buf) || !recvAll(&deleted, sizeof(deleted))) {
        reset();
        return NIXL_ERR_BACKEND;
    }
    return deleted > 0 ? NIXL_SUCCESS : NIXL_ERR_NOT_FOUND;
}

// ---------------------------------------------------------------- backend

nixlTcpStoreMetadataBackend::nixlTcpStoreMetadataBackend(const std::string &endpoint) {
    const size_t colon = endpoint.rfind(':');
    const std::string host = colon == std::string::npos ? endpoint : endpoint.substr(0, colon);
    const int port = colon == std::string::npos ? 29500 : std::atoi(endpoint.c_str() + colon + 1);
    const int connect_ms = nixl::config::getValueDefaulted<int>("NIXL_TCPSTORE_TIMEOUT_MS", 30000);
    const int op_ms = nixl::config::getValueDefaulted<int>("NIXL_TCPSTORE_OP_TIMEOUT_MS", 5000);
    fetchTimeoutMs_ = connect_ms;
    client_ = std::make_unique<nixlTcpStoreClient>(host, port, std::min(connect_ms, 5000), op_ms);
    if (!client_->connected()) NIXL_ERROR << "cannot reach TCPStore at " << endpoint;
}

std::string nixlTcpStoreMetadataBackend::makeKey(const std::string &agent, const std::string &label) {
    return "nixl/agents/" + label + "/" + agent + "/" + nixl_null_agent;
}

nixl_status_t nixlTcpStoreMetadataBackend::publish(const std::string &agent, const std::string &label, const nixl_blob_t &blob) {
    if (!ok()) return NIXL_ERR_BACKEND;
    const std::string key = makeKey(agent, label);
    const nixl_status_t st = client_->set(key, blob);
    if (st == NIXL_SUCCESS) {
        std::lock_guard<std::mutex> g(mu_);
        if (std::find(published_.begin(), published_.end(), key) == published_.end()) published_.push_back(key);
    }
    return st;
}

nixl_status_t nixlTcpStoreMetadataBackend::fetch(const std::string &agent, const std::string &label, nixl_blob_t &blob) {
    if (!ok()) return NIXL_ERR_BACKEND;
    const std::string key = makeKey(agent, label);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(fetchTimeoutMs_);
    for (;;) {
        const nixl_status_t st = client_->get(key, blob);
        if (st != NIXL_ERR_NOT_FOUND) return st;
        if (std::chrono::steady_clock::now() > deadline) return NIXL_ERR_NOT_FOUND;
        std::this_thread::sleep_for(std::chrono::milliseconds(10));
    }
}

nixl_status_t nixlTcpStoreMetadataBackend::remove(const std::string &) {
    if (!ok()) return NIXL_ERR_BACKEND;
    std::vector<std::string> keys;
    {
        std::lock_guard<std::mutex> g(mu_);
        keys.swap(published_);
    }
    for (auto &k : keys) client_->deleteKey(k);
    return NIXL_SUCCESS;
}

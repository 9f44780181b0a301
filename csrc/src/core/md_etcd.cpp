#include "core/md_etcd.h"

#include <arpa/inet.h>
#include <netdb.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>

#include "utils/config.h"
#include "utils/log.h"

// ---------------------------------------------------------------- tiny HTTP + base64

namespace nixl_http {

static const char kB64[] = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";

std::string base64Encode(const std::string &raw) {
    std::string out;
    out.reserve((raw.size() + 2) / 3 * 4);
    size_t i = 0;
    for (; i + 2 < raw.size(); i += 3) {
        const unsigned v = (static_cast<unsigned char>(raw[i]) << 16) | (static_cast<unsigned char>(raw[i + 1]) << 8) | static_cast<unsigned char>(raw[i + 2]);
        out += kB64[v >> 18];
        out += kB64[(v >> 12) & 63];
        out += kB64[(v >> 6) & 63];
        out += kB64[v & 63];
    }
    if (i + 1 == raw.size()) {
        const unsigned v = static_cast<unsigned char>(raw[i]) << 16;
        out += kB64[v >> 18];
        out += kB64[(v >> 12) & 63];
        out += "==";
    } else if (i + 2 == raw.size()) {
        const unsigned v = (static_cast<unsigned char>(raw[i]) << 16) | (static_cast<unsigned char>(raw[i + 1]) << 8);
        out += kB64[v >> 18];
        out += kB64[(v >> 12) & 63];
        out += kB64[(v >> 6) & 63];
        out += '=';
    }
    return out;
}

bool base64Decode(const std::string &text, std::string &raw) {
    raw.clear();
    unsigned acc = 0;
    int bits = 0;
    for (char c : text) {
        if (c == '=' || c == '\n' || c == '\r') continue;
        const char *p = std::strchr(kB64, c);
        if (!p || !c) return false;
        acc = (acc << 6) | static_cast<unsigned>(p - kB64);
        bits += 6;
        if (bits >= 8) {
            bits -= 8;
            raw += static_cast<char>((acc >> bits) & 0xff);
        }
    }
    return true;
}

static bool waitFd(int fd, short events, int timeout_ms) {
    pollfd p{fd, events, 0};
    return ::poll(&p, 1, timeout_ms) > 0;
}

// Connected TCP socket with send / receive timeouts, or -1.
static int connectTo(const std::string &host, int port, int timeout_ms) {
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_UNSPEC;
    hints.ai_socktype = SOCK_STREAM;
    if (::getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || !res) return -1;
    int fd = -1;
    for (addrinfo *a = res; a; a = a->ai_next) {
        fd = ::socket(a->ai_family, a->ai_socktype | SOCK_CLOEXEC, a->ai_protocol);
        if (fd < 0) continue;
        timeval tv{timeout_ms / 1000, (timeout_ms % 1000) * 1000};
        ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
        ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        if (::connect(fd, a->ai_addr, a->ai_addrlen) == 0) break;
        ::close(fd);
        fd = -1;
    }
    ::freeaddrinfo(res);
    return fd;
}

static bool sendAll(int fd, const std::string &req) {
    size_t off = 0;
    while (off < req.size()) {
        const ssize_t n = ::send(fd, req.data() + off, req.size() - off, MSG_NOSIGNAL);
        if (n <= 0) return false;
        off += static_cast<size_t>(n);
    }
    return true;
}

int postJson(const std::string &host, int port, const std::string &path, const std::string &body, std::string &reply, int timeout_ms) {
    reply.clear();
    const int fd = connectTo(host, port, timeout_ms);
    if (fd < 0) return 0;
    std::string req = "POST " + path + " HTTP/1.1\r\nHost: " + host + ":" + std::to_string(port) +
        "\r\nContent-Type: application/json\r\nConnection: close\r\nContent-Length: " + std::to_string(body.size()) + "\r\n\r\n" + body;
    if (!sendAll(fd, req)) {
        ::close(fd);
        return 0;
    }
    std::string raw;
    char buf[8192];
    while (waitFd(fd, POLLIN, timeout_ms)) {
        const ssize_t n = ::recv(fd, buf, sizeof(buf), 0);
        if (n <= 0) break;
        raw.append(buf, static_cast<size_t>(n));
        if (raw.size() > (size_t(1) << 30)) break;
    }
    ::close(fd);
    const size_t hdr_end = raw.find("\r\n\r\n");
    if (raw.compare(0, 5, "HTTP/") != 0 || hdr_end == std::string::npos) return 0;
    const int status = std::atoi(raw.c_str() + raw.find(' ') + 1);
    std::string headers = raw.substr(0, hdr_end);
    std::transform(headers.begin(), headers.end(), headers.begin(), [](unsigned char c) { return std::tolower(c); });
    std::string payload = raw.substr(hdr_end + 4);
    if (headers.find("transfer-encoding: chunked") != std::string::npos) {
        std::string joined;
        size_t pos = 0;
        while (pos < payload.size()) {
            const size_t eol = payload.find("\r\n", pos);
            if (eol == std::string::npos) break;
            const size_t len = std::strtoul(payload.c_str() + pos, nullptr, 16);
            if (len == 0) break;
            joined.append(payload, eol + 2, len);
            pos = eol + 2 + len + 2;
        }
        payload.swap(joined);
    }
    reply.swap(payload);
    return status;
}

// A streaming POST: the reply body (chunked or not) is handed to `on_data` piece by piece as it
// arrives, until the peer closes, `keep_going` turns false or `on_data` returns false.  Returns the
// HTTP status (0: transport failure before a status line).
int postStream(const std::string &host, int port, const std::string &path, const std::string &body, int timeout_ms,
               const std::function<bool()> &keep_going, const std::function<bool(const std::string &)> &on_data) {
    const int fd = connectTo(host, port, timeout_ms);
    if (fd < 0) return 0;
    const std::string req = "POST " + path + " HTTP/1.1\r\nHost: " + host + ":" + std::to_string(port) +
        "\r\nContent-Type: application/json\r\nContent-Length: " + std::to_string(body.size()) + "\r\n\r\n" + body;
    if (!sendAll(fd, req)) {
        ::close(fd);
        return 0;
    }
    std::string raw;   // bytes not yet consumed
    int status = 0;
    bool chunked = false, headers_done = false;
    size_t chunk_left = 0; // bytes of the current chunk still to come
    char buf[8192];
    bool open = true;
    while (open && keep_going()) {
        if (!waitFd(fd, POLLIN, 200)) continue;
        const ssize_t n = ::recv(fd, buf, sizeof(buf), 0);
        if (n <= 0) break;
        raw.append(buf, static_cast<size_t>(n));
        if (!headers_done) {
            const size_t hdr_end = raw.find("\r\n\r\n");
            if (hdr_end == std::string::npos) continue;
            if (raw.compare(0, 5, "HTTP/") != 0) break;
            status = std::atoi(raw.c_str() + raw.find(' ') + 1);
            std::string headers = raw.substr(0, hdr_end);
            std::transform(headers.begin(), headers.end(), headers.begin(), [](unsigned char c) { return std::tolower(c); });
            chunked = headers.find("transfer-encoding: chunked") != std::string::npos;
            raw.erase(0, hdr_end + 4);
            headers_done = true;
            if (status != 200) break;
        }
        if (!chunked) {
            if (!raw.empty() && !on_data(raw)) open = false;
            raw.clear();
            continue;
        }
        for (;;) { // as many whole pieces as the buffer holds
            if (chunk_left == 0) {
                const size_t eol = raw.find("\r\n");
                if (eol == std::string::npos) break;
                if (eol == 0) { // the CRLF that closes the previous chunk
                    raw.erase(0, 2);
                    continue;
                }
                chunk_left = std::strtoul(raw.c_str(), nullptr, 16);
                raw.erase(0, eol + 2);
                if (chunk_left == 0) { // last chunk
                    open = false;
                    break;
                }
            }
            if (raw.empty()) break;
            const size_t take = std::min(chunk_left, raw.size());
            if (!on_data(raw.substr(0, take))) {
                open = false;
                break;
            }
            raw.erase(0, take);
            chunk_left -= take;
        }
    }
    ::close(fd);
    return status;
}

} // namespace nixl_http

// ---------------------------------------------------------------- backend

namespace {

// Value of the first "name":"..." string member in a JSON text (the gateway's replies are flat enough).
bool jsonString(const std::string &json, const std::string &name, std::string &out, size_t from = 0) {
    const std::string needle = "\"" + name + "\"";
    size_t p = json.find(needle, from);
    if (p == std::string::npos) return false;
    p = json.find(':', p + needle.size());
    if (p == std::string::npos) return false;
    p = json.find('"', p);
    if (p == std::string::npos) return false;
    const size_t e = json.find('"', p + 1);
    if (e == std::string::npos) return false;
    out = json.substr(p + 1, e - p - 1);
    return true;
}

} // namespace

nixlEtcdMetadataBackend::nixlEtcdMetadataBackend(const std::string &endpoints, std::chrono::microseconds watch_timeout) : watchTimeout_(watch_timeout) {
    namespace_ = nixl::config::getValueDefaulted<std::string>("NIXL_ETCD_NAMESPACE", "/nixl/agents");
    while (namespace_.size() > 1 && namespace_.back() == '/') namespace_.pop_back();
    opTimeoutMs_ = nixl::config::getValueDefaulted<int>("NIXL_ETCD_OP_TIMEOUT_MS", 5000);
    pollMs_ = std::max(10, nixl::config::getValueDefaulted<int>("NIXL_ETCD_POLL_MS", 500));
    size_t pos = 0;
    while (pos <= endpoints.size() && port_ == 0) {
        size_t comma = endpoints.find(',', pos);
        if (comma == std::string::npos) comma = endpoints.size();
        std::string ep = endpoints.substr(pos, comma - pos);
        pos = comma + 1;
        const size_t scheme = ep.find("://");
        if (scheme != std::string::npos) ep = ep.substr(scheme + 3);
        while (!ep.empty() && ep.back() == '/') ep.pop_back();
        if (ep.empty()) continue;
        const size_t colon = ep.rfind(':');
        const std::string host = colon == std::string::npos ? ep : ep.substr(0, colon);
        const int port = colon == std::string::npos ? 2379 : std::atoi(ep.c_str() + colon + 1);
        std::string reply;
        // Any HTTP answer to a range request means a gateway is listening there.
        if (nixl_http::postJson(host, port, "/v3/kv/range", "{\"key\":\"" + nixl_http::base64Encode(namespace_) + "\"}", reply, std::min(opTimeoutMs_, 3000)) == 200) {
            host_ = host;
            port_ = port;
        }
    }
    if (!ok()) {
        NIXL_ERROR << "no etcd gateway answered at " << endpoints;
        return;
    }
    watcher_ = std::thread([this] { watchLoop(); });
}

nixlEtcdMetadataBackend::~nixlEtcdMetadataBackend() {
    stop_ = true;
    if (watcher_.joinable()) watcher_.join();
}

void nixlEtcdMetadataBackend::setInvalidateCallback(std::function<void(const std::string &)> cb) {
    std::lock_guard<std::mutex> g(mu_);
    onGone_ = std::move(cb);
}

std::string nixlEtcdMetadataBackend::makeKey(const std::string &agent, const std::string &label) const {
    return namespace_ + "/" + agent + "/" + label;
}

nixl_status_t nixlEtcdMetadataBackend::get(const std::string &key, std::string &value) {
    std::string reply;
    const int st = nixl_http::postJson(host_, port_, "/v3/kv/range", "{\"key\":\"" + nixl_http::base64Encode(key) + "\"}", reply, opTimeoutMs_);
    if (st != 200) return NIXL_ERR_BACKEND;
    const size_t kvs = reply.find("\"kvs\"");
    std::string b64;
    if (kvs == std::string::npos || !jsonString(reply, "value", b64, kvs)) return NIXL_ERR_NOT_FOUND;
    if (!nixl_http::base64Decode(b64, value)) return NIXL_ERR_MISMATCH;
    return value.empty() ? NIXL_ERR_NOT_FOUND : NIXL_SUCCESS;
}

nixl_status_t nixlEtcdMetadataBackend::publish(const std::string &agent, const std::string &label, const nixl_blob_t &blob) {
    if (!ok()) return NIXL_ERR_BACKEND;
    const std::string key = makeKey(agent, label);
    std::string reply;
    const std::string body = "{\"key\":\"" + nixl_http::base64Encode(key) + "\",\"value\":\"" + nixl_http::base64Encode(blob) + "\"}";
    if (nixl_http::postJson(host_, port_, "/v3/kv/put", body, reply, opTimeoutMs_) != 200) return NIXL_ERR_BACKEND;
    std::lock_guard<std::mutex> g(mu_);
    if (std::find(published_.begin(), published_.end(), key) == published_.end()) published_.push_back(key);
    return NIXL_SUCCESS;
}

nixl_status_t nixlEtcdMetadataBackend::fetch(const std::string &agent, const std::string &label, nixl_blob_t &blob) {
    if (!ok()) return NIXL_ERR_BACKEND;
    const std::string key = makeKey(agent, label);
    const auto deadline = std::chrono::steady_clock::now() + watchTimeout_;
    for (;;) {
        const nixl_status_t st = get(key, blob);
        if (st == NIXL_SUCCESS) {
            std::lock_guard<std::mutex> g(mu_);
            watched_[key] = agent;
            return st;
        }
        if (st != NIXL_ERR_NOT_FOUND) return st;
        if (std::chrono::steady_clock::now() > deadline || stop_) return NIXL_ERR_NOT_FOUND;
        std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
}

nixl_status_t nixlEtcdMetadataBackend::remove(const std::string &) {
    if (!ok()) return NIXL_ERR_BACKEND;
    std::vector<std::string> keys;
    {
        std::lock_guard<std::mutex> g(mu_);
        keys.swap(published_);
    }
    nixl_status_t ret = NIXL_SUCCESS;
    for (const auto &k : keys) {
        std::string reply;
        if (nixl_http::postJson(host_, port_, "/v3/kv/deleterange", "{\"key\":\"" + nixl_http::base64Encode(k) + "\"}", reply, opTimeoutMs_) != 200)
            ret = NIXL_ERR_BACKEND;
    }
    return ret;
}

// Called with the key of a peer's record that is gone.
void nixlEtcdMetadataBackend::keyGone(const std::string &key) {
    std::string agent;
    std::function<void(const std::string &)> cb;
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = watched_.find(key);
        if (it == watched_.end()) return;
        agent = it->second;
        watched_.erase(it);
        cb = onGone_;
    }
    NIXL_INFO << "etcd: key " << key << " is gone, invalidating the metadata of " << agent;
    if (cb) cb(agent);
}

// One watch stream over the whole namespace (POST /v3/watch, the gateway's form of the reference's
// DELETE watchers, nixl_etcd_metadata_backend.cpp:262-318): every DELETE event of a key this agent
// fetched invalidates that peer at once.  Returns false when the gateway has no watch endpoint.
bool nixlEtcdMetadataBackend::watchStream() {
    // prefix range: [namespace + "/", namespace + "0")   ('0' is the byte after '/')
    const std::string body = "{\"create_request\":{\"key\":\"" + nixl_http::base64Encode(namespace_ + "/") + "\",\"range_end\":\"" +
        nixl_http::base64Encode(namespace_ + "0") + "\"}}";
    std::string pending; // text of the stream up to the last complete line
    bool created = false;
    const int status = nixl_http::postStream(
        host_, port_, "/v3/watch", body, opTimeoutMs_, [this] { return !stop_.load(); },
        [&](const std::string &piece) {
            pending += piece;
            size_t nl;
            while ((nl = pending.find('\n')) != std::string::npos) { // one JSON object per line
                const std::string line = pending.substr(0, nl);
                pending.erase(0, nl + 1);
                if (line.find("\"created\"") != std::string::npos) created = true;
                size_t at = 0;
                while ((at = line.find("\"DELETE\"", at)) != std::string::npos) {
                    std::string b64, key;
                    if (jsonString(line, "key", b64, at) && nixl_http::base64Decode(b64, key)) keyGone(key);
                    at += 8;
                }
            }
            return true;
        });
    watchActive_ = false;
    return status == 200 && created;
}

void nixlEtcdMetadataBackend::watchLoop() {
    // The stream when the gateway offers one; whenever it is not up (old gateway, connection lost),
    // the keys fetched so far are polled instead, so a deletion is never missed for long.
    bool stream_ok = true;
    while (!stop_) {
        if (stream_ok) {
            watchActive_ = true;
            const auto t0 = std::chrono::steady_clock::now();
            stream_ok = watchStream();
            if (stop_) return;
            // what was deleted while no stream was up shows in one poll round below
            if (!stream_ok) NIXL_INFO << "etcd: no watch stream at " << host_ << ":" << port_ << "; polling every " << pollMs_ << " ms";
            else if (std::chrono::steady_clock::now() - t0 < std::chrono::seconds(1)) std::this_thread::sleep_for(std::chrono::milliseconds(200));
        } else {
            for (int waited = 0; waited < pollMs_ && !stop_; waited += 10) std::this_thread::sleep_for(std::chrono::milliseconds(10));
        }
        std::map<std::string, std::string> snapshot;
        {
            std::lock_guard<std::mutex> g(mu_);
            snapshot = watched_;
        }
        for (const auto &[key, agent] : snapshot) {
            if (stop_) return;
            std::string value;
            if (get(key, value) != NIXL_ERR_NOT_FOUND) continue; // still there, or the store is unreachable: no verdict
            keyGone(key);
        }
    }
}

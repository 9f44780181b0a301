// A small S3 client over the service's REST interface, for the OBJ backend: PutObject, ranged GetObject, HeadObject and
// multipart upload, signed with AWS Signature Version 4, over HTTP/1.1 keep-alive connections (plain, or TLS through the
// system's OpenSSL loaded at run time).  Role parity: the reference's OBJ plug-in uses aws-sdk-cpp for the same calls
// (src/plugins/obj/s3/client.cpp: put :64, ranged get :96, head :124); this build has no SDK, so the protocol is
// written out: SHA-256 / HMAC, canonical request, string to sign, signing key, and a minimal HTTP exchange.
//
// Header-only so that the one-file plug-in build picks it up.
#ifndef NIXL_B200_S3_REST_H
#define NIXL_B200_S3_REST_H

#include <arpa/inet.h>
#include <dlfcn.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <unistd.h>

#include <algorithm>
#include <array>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <ctime>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

namespace nixl_s3 {

// ------------------------------------------------------------------ SHA-256, HMAC

class Sha256 {
public:
    Sha256() { reset(); }
    void reset() {
        static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
        std::memcpy(h_, init, sizeof(h_));
        len_ = 0;
        fill_ = 0;
    }
    void update(const void *data, size_t n) {
        const uint8_t *p = static_cast<const uint8_t *>(data);
        len_ += n;
        if (fill_) {
            const size_t take = std::min(n, sizeof(buf_) - fill_);
            std::memcpy(buf_ + fill_, p, take);
            fill_ += take;
            p += take;
            n -= take;
            if (fill_ < sizeof(buf_)) return;
            block(buf_);
            fill_ = 0;
        }
        for (; n >= 64; p += 64, n -= 64) block(p);
        if (n) {
            std::memcpy(buf_, p, n);
            fill_ = n;
        }
    }
    std::array<uint8_t, 32> finish() {
        const uint64_t bits = len_ * 8;
        const uint8_t one = 0x80, zero = 0;
        update(&one, 1);
        while (fill_ != 56) update(&zero, 1);
        uint8_t tail[8];
        for (int i = 0; i < 8; ++i) tail[i] = static_cast<uint8_t>(bits >> (56 - 8 * i));
        update(tail, 8);
        std::array<uint8_t, 32> out;
        for (int i = 0; i < 8; ++i)
            for (int j = 0; j < 4; ++j) out[static_cast<size_t>(i * 4 + j)] = static_cast<uint8_t>(h_[i] >> (24 - 8 * j));
        return out;
    }

private:
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void block(const uint8_t *p) {
        static const uint32_t k[64] = {
            0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be,
            0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa,
            0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85,
            0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3,
            0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f,
            0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
        uint32_t w[64];
        for (int i = 0; i < 16; ++i)
            w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) | (uint32_t(p[4 * i + 2]) << 8) | uint32_t(p[4 * i + 3]);
        for (int i = 16; i < 64; ++i) {
            const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h_[0], b = h_[1], c = h_[2], d = h_[3], e = h_[4], f = h_[5], g = h_[6], h = h_[7];
        for (int i = 0; i < 64; ++i) {
            const uint32_t t1 = h + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + k[i] + w[i];
            const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
            h = g;
            g = f;
            f = e;
            e = d + t1;
            d = c;
            c = b;
            b = a;
            a = t1 + t2;
        }
        h_[0] += a;
        h_[1] += b;
        h_[2] += c;
        h_[3] += d;
        h_[4] += e;
        h_[5] += f;
        h_[6] += g;
        h_[7] += h;
    }
    uint32_t h_[8];
    uint8_t buf_[64];
    size_t fill_ = 0;
    uint64_t len_ = 0;
};

using Digest = std::array<uint8_t, 32>;

inline Digest sha256(const void *data, size_t n) {
    Sha256 s;
    s.update(data, n);
    return s.finish();
}

inline std::string hex(const uint8_t *p, size_t n) {
    static const char *digits = "0123456789abcdef";
    std::string out(n * 2, '0');
    for (size_t i = 0; i < n; ++i) {
        out[2 * i] = digits[p[i] >> 4];
        out[2 * i + 1] = digits[p[i] & 15];
    }
    return out;
}
inline std::string hex(const Digest &d) { return hex(d.data(), d.size()); }

// CRC-32 (IEEE 802.3, the one S3 calls CRC32), eight bytes per step.
inline uint32_t crc32(const void *data, size_t n, uint32_t crc = 0) {
    static const auto table = [] {
        std::array<std::array<uint32_t, 256>, 8> t{};
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k) c = (c >> 1) ^ (0xedb88320u & (0u - (c & 1)));
            t[0][i] = c;
        }
        for (uint32_t i = 0; i < 256; ++i)
            for (int k = 1; k < 8; ++k) t[static_cast<size_t>(k)][i] = (t[static_cast<size_t>(k - 1)][i] >> 8) ^ t[0][t[static_cast<size_t>(k - 1)][i] & 0xff];
        return t;
    }();
    const uint8_t *p = static_cast<const uint8_t *>(data);
    crc = ~crc;
    while (n >= 8) {
        uint32_t lo, hi;
        std::memcpy(&lo, p, 4);
        std::memcpy(&hi, p + 4, 4);
        lo ^= crc;
        crc = table[7][lo & 0xff] ^ table[6][(lo >> 8) & 0xff] ^ table[5][(lo >> 16) & 0xff] ^ table[4][lo >> 24] ^ table[3][hi & 0xff] ^
            table[2][(hi >> 8) & 0xff] ^ table[1][(hi >> 16) & 0xff] ^ table[0][hi >> 24];
        p += 8;
        n -= 8;
    }
    while (n--) crc = (crc >> 8) ^ table[0][(crc ^ *p++) & 0xff];
    return ~crc;
}

// The checksum as S3 wants it in a header: base64 of the four bytes, most significant first.
inline std::string crc32Header(uint32_t crc) {
    static const char *t = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
    const uint8_t b[4] = {static_cast<uint8_t>(crc >> 24), static_cast<uint8_t>(crc >> 16), static_cast<uint8_t>(crc >> 8), static_cast<uint8_t>(crc)};
    const uint32_t v0 = (uint32_t(b[0]) << 16) | (uint32_t(b[1]) << 8) | b[2], v1 = uint32_t(b[3]) << 16;
    std::string out;
    out += t[(v0 >> 18) & 63];
    out += t[(v0 >> 12) & 63];
    out += t[(v0 >> 6) & 63];
    out += t[v0 & 63];
    out += t[(v1 >> 18) & 63];
    out += t[(v1 >> 12) & 63];
    out += "==";
    return out;
}

inline Digest hmacSha256(const void *key, size_t key_len, const void *msg, size_t msg_len) {
    uint8_t k[64] = {0};
    if (key_len > 64) {
        const Digest d = sha256(key, key_len);
        std::memcpy(k, d.data(), d.size());
    } else {
        std::memcpy(k, key, key_len);
    }
    uint8_t ipad[64], opad[64];
    for (int i = 0; i < 64; ++i) {
        ipad[i] = k[i] ^ 0x36;
        opad[i] = k[i] ^ 0x5c;
    }
    Sha256 inner;
    inner.update(ipad, 64);
    inner.update(msg, msg_len);
    const Digest in = inner.finish();
    Sha256 outer;
    outer.update(opad, 64);
    outer.update(in.data(), in.size());
    return outer.finish();
}
inline Digest hmacSha256(const Digest &key, const std::string &msg) { return hmacSha256(key.data(), key.size(), msg.data(), msg.size()); }

// ------------------------------------------------------------------ Signature Version 4

// RFC 3986 unreserved characters stay; everything else becomes %XX (upper-case hex).  `keep_slash` for object paths.
inline std::string uriEncode(const std::string &s, bool keep_slash) {
    static const char *digits = "0123456789ABCDEF";
    std::string out;
    for (unsigned char c : s) {
        if ((c >= 'A' && c <= 'Z') || (c >= 'a' && c <= 'z') || (c >= '0' && c <= '9') || c == '-' || c == '_' || c == '.' || c == '~' ||
            (c == '/' && keep_slash)) {
            out.push_back(static_cast<char>(c));
        } else {
            out.push_back('%');
            out.push_back(digits[c >> 4]);
            out.push_back(digits[c & 15]);
        }
    }
    return out;
}

struct Credentials {
    std::string accessKey, secretKey, sessionToken;
    bool empty() const { return accessKey.empty() || secretKey.empty(); }
};

struct Request {
    std::string method;                                      // "GET", "PUT", ...
    std::string path;                                        // "/bucket/key", not yet encoded
    std::vector<std::pair<std::string, std::string>> query;  // not yet encoded
    std::map<std::string, std::string> headers;              // lower-case names; "host" and the x-amz-* ones are signed
    std::string payloadHash;                                 // hex SHA-256 of the body, or "UNSIGNED-PAYLOAD"
};

inline std::string canonicalQuery(const Request &r) {
    std::vector<std::pair<std::string, std::string>> q;
    for (const auto &kv : r.query) q.emplace_back(uriEncode(kv.first, false), uriEncode(kv.second, false));
    std::sort(q.begin(), q.end());
    std::string out;
    for (const auto &kv : q) {
        if (!out.empty()) out.push_back('&');
        out += kv.first + "=" + kv.second;
    }
    return out;
}

inline std::string trimmed(const std::string &v) {
    size_t a = 0, b = v.size();
    while (a < b && (v[a] == ' ' || v[a] == '\t')) ++a;
    while (b > a && (v[b - 1] == ' ' || v[b - 1] == '\t')) --b;
    return v.substr(a, b - a);
}

// The value of the Authorization header for `r`.  `amz_date` is "YYYYMMDDTHHMMSSZ" and must equal r.headers["x-amz-date"].
inline std::string authorizationV4(const Request &r, const Credentials &cred, const std::string &region, const std::string &service,
                                   const std::string &amz_date) {
    std::string canonical_headers, signed_headers;
    for (const auto &kv : r.headers) { // std::map: already sorted by (lower-case) name
        canonical_headers += kv.first + ":" + trimmed(kv.second) + "\n";
        if (!signed_headers.empty()) signed_headers.push_back(';');
        signed_headers += kv.first;
    }
    const std::string canonical = r.method + "\n" + uriEncode(r.path, true) + "\n" + canonicalQuery(r) + "\n" + canonical_headers + "\n" +
        signed_headers + "\n" + r.payloadHash;
    const std::string date = amz_date.substr(0, 8);
    const std::string scope = date + "/" + region + "/" + service + "/aws4_request";
    const std::string to_sign = "AWS4-HMAC-SHA256\n" + amz_date + "\n" + scope + "\n" + hex(sha256(canonical.data(), canonical.size()));
    const std::string k0 = "AWS4" + cred.secretKey;
    Digest k = hmacSha256(k0.data(), k0.size(), date.data(), date.size());
    k = hmacSha256(k, region);
    k = hmacSha256(k, service);
    k = hmacSha256(k, "aws4_request");
    const Digest sig = hmacSha256(k, to_sign);
    return "AWS4-HMAC-SHA256 Credential=" + cred.accessKey + "/" + scope + ", SignedHeaders=" + signed_headers + ", Signature=" + hex(sig);
}

inline std::string amzDateNow() {
    const std::time_t t = std::time(nullptr);
    std::tm tm{};
    ::gmtime_r(&t, &tm);
    char buf[32];
    std::strftime(buf, sizeof(buf), "%Y%m%dT%H%M%SZ", &tm);
    return buf;
}

// ------------------------------------------------------------------ TLS through the system's OpenSSL, loaded on first use

class Tls {
public:
    void *(*TLS_client_method)() = nullptr;
    void *(*SSL_CTX_new)(void *) = nullptr;
    void (*SSL_CTX_free)(void *) = nullptr;
    int (*SSL_CTX_set_default_verify_paths)(void *) = nullptr;
    int (*SSL_CTX_load_verify_locations)(void *, const char *, const char *) = nullptr;
    void (*SSL_CTX_set_verify)(void *, int, void *) = nullptr;
    void *(*SSL_new)(void *) = nullptr;
    void (*SSL_free)(void *) = nullptr;
    int (*SSL_set_fd)(void *, int) = nullptr;
    int (*SSL_connect)(void *) = nullptr;
    int (*SSL_read)(void *, void *, int) = nullptr;
    int (*SSL_write)(void *, const void *, int) = nullptr;
    long (*SSL_ctrl)(void *, int, long, void *) = nullptr;
    int (*SSL_set1_host)(void *, const char *) = nullptr;
    int (*SSL_shutdown)(void *) = nullptr;
    bool ok = false;

    static const Tls &get() {
        static const Tls t = [] {
            Tls x;
            void *lib = nullptr;
            for (const char *name : {"libssl.so.3", "libssl.so.1.1", "libssl.so"})
                if ((lib = ::dlopen(name, RTLD_NOW | RTLD_GLOBAL))) break;
            if (!lib) return x;
            bool all = true;
            auto sym = [&](auto &fn, const char *name) {
                fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(::dlsym(lib, name));
                all = all && fn;
            };
            sym(x.TLS_client_method, "TLS_client_method");
            sym(x.SSL_CTX_new, "SSL_CTX_new");
            sym(x.SSL_CTX_free, "SSL_CTX_free");
            sym(x.SSL_CTX_set_default_verify_paths, "SSL_CTX_set_default_verify_paths");
            sym(x.SSL_CTX_load_verify_locations, "SSL_CTX_load_verify_locations");
            sym(x.SSL_CTX_set_verify, "SSL_CTX_set_verify");
            sym(x.SSL_new, "SSL_new");
            sym(x.SSL_free, "SSL_free");
            sym(x.SSL_set_fd, "SSL_set_fd");
            sym(x.SSL_connect, "SSL_connect");
            sym(x.SSL_read, "SSL_read");
            sym(x.SSL_write, "SSL_write");
            sym(x.SSL_ctrl, "SSL_ctrl");
            sym(x.SSL_set1_host, "SSL_set1_host");
            sym(x.SSL_shutdown, "SSL_shutdown");
            x.ok = all;
            return x;
        }();
        return t;
    }
};

// ------------------------------------------------------------------ one HTTP/1.1 connection

class Conn {
public:
    Conn() = default;
    Conn(const Conn &) = delete;
    Conn &operator=(const Conn &) = delete;
    ~Conn() { close(); }
    bool reused = false; // has carried a request before: a failure on it may only mean that the server closed it meanwhile

    bool open(const std::string &host, uint16_t port, void *tls_ctx, int timeout_ms) {
        close();
        addrinfo hints{}, *res = nullptr;
        hints.ai_family = AF_UNSPEC;
        hints.ai_socktype = SOCK_STREAM;
        if (::getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0) return false;
        for (addrinfo *a = res; a && fd_ < 0; a = a->ai_next) {
            const int fd = ::socket(a->ai_family, a->ai_socktype | SOCK_CLOEXEC, a->ai_protocol);
            if (fd < 0) continue;
            timeval tv{timeout_ms / 1000, (timeout_ms % 1000) * 1000};
            ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
            ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
            if (::connect(fd, a->ai_addr, a->ai_addrlen) != 0) {
                ::close(fd);
                continue;
            }
            const int one = 1;
            ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            fd_ = fd;
        }
        ::freeaddrinfo(res);
        if (fd_ < 0) return false;
        if (tls_ctx) {
            const Tls &t = Tls::get();
            ssl_ = t.SSL_new(tls_ctx);
            if (!ssl_) return close(), false;
            t.SSL_ctrl(ssl_, 55 /* set TLS extension: host name */, 0, const_cast<char *>(host.c_str()));
            t.SSL_set1_host(ssl_, host.c_str());
            if (t.SSL_set_fd(ssl_, fd_) != 1 || t.SSL_connect(ssl_) != 1) return close(), false;
        }
        reused = false;
        return true;
    }
    void close() {
        if (ssl_) {
            Tls::get().SSL_shutdown(ssl_);
            Tls::get().SSL_free(ssl_);
            ssl_ = nullptr;
        }
        if (fd_ >= 0) ::close(fd_);
        fd_ = -1;
    }
    bool isOpen() const { return fd_ >= 0; }
    bool writeAll(const void *data, size_t n) {
        const char *p = static_cast<const char *>(data);
        while (n) {
            ssize_t k;
            if (ssl_) k = Tls::get().SSL_write(ssl_, p, static_cast<int>(std::min<size_t>(n, 1u << 30)));
            else k = ::send(fd_, p, n, MSG_NOSIGNAL);
            if (k <= 0) {
                if (!ssl_ && errno == EINTR) continue;
                return false;
            }
            p += k;
            n -= static_cast<size_t>(k);
        }
        return true;
    }
    ssize_t readSome(void *data, size_t n) {
        for (;;) {
            ssize_t k;
            if (ssl_) k = Tls::get().SSL_read(ssl_, data, static_cast<int>(std::min<size_t>(n, 1u << 30)));
            else k = ::recv(fd_, data, n, 0);
            if (k < 0 && !ssl_ && errno == EINTR) continue;
            return k;
        }
    }

private:
    int fd_ = -1;
    void *ssl_ = nullptr;
};

struct Response {
    int status = 0; // HTTP status; <= 0: no answer (the connection failed)
    std::map<std::string, std::string> headers; // lower-case names
    std::string body;                           // what was not delivered into the caller's buffer
};

struct HttpConfig {
    std::string scheme = "https", host, caBundle;
    std::string connectHost; // where to connect when it is not `host` (tried first; `host` is the fall-back)
    uint16_t port = 0;
    bool verifyTls = true;
    int timeoutMs = 30000;
    int maxAttempts = 3; // a request that got no answer, or 500 / 502 / 503 / 504, is sent again (after 100 ms, 400 ms, ...)
};

// Runs `once` until it gives an answer worth keeping or the attempts are used up.  Object stores ask for this: "slow
// down" and internal errors are part of their contract, and the SDKs retry them by default.
template<class Once> inline Response withRetries(int max_attempts, Once &&once) {
    Response resp;
    int wait_ms = 100;
    for (int attempt = 1;; ++attempt) {
        resp = once();
        const bool again = resp.status <= 0 || resp.status == 500 || resp.status == 502 || resp.status == 503 || resp.status == 504;
        if (!again || attempt >= max_attempts) return resp;
        timespec ts{wait_ms / 1000, (wait_ms % 1000) * 1000000L};
        ::nanosleep(&ts, nullptr);
        wait_ms *= 4;
    }
}

struct Config : HttpConfig {
    std::string bucket, region = "us-east-1";
    bool virtualAddressing = false;
    bool signPayload = true; // hash the body of a PUT into the signature (off: "UNSIGNED-PAYLOAD")
    bool sendChecksum = false;  // a CRC32 of every uploaded body goes with it and the service checks it
    bool checkChecksum = false; // ask for the stored checksum with every download and compare (whole objects only: a range has none)
    Credentials cred;
};

// What the OBJ engine asks of an object service.  Every call returns the HTTP status (200, 206, 404, 403, ...) or 0 when
// the service could not be reached.  A large object goes up in parts: create -> parts (any order, side by side) ->
// complete (or abort).
class ObjectService {
public:
    virtual ~ObjectService() = default;
    virtual bool usable() const = 0;
    virtual int putObject(const std::string &key, const void *data, size_t len, std::string *etag = nullptr) = 0;
    virtual int getObject(const std::string &key, uint64_t offset, void *dst, size_t len) = 0;
    virtual int headObject(const std::string &key, uint64_t *size) = 0;
    virtual int deleteObject(const std::string &key) = 0;
    virtual int createMultipart(const std::string &key, std::string &upload_id) = 0;
    virtual int uploadPart(const std::string &key, const std::string &upload_id, int number, const void *data, size_t len, std::string &etag) = 0;
    virtual int completeMultipart(const std::string &key, const std::string &upload_id, const std::vector<std::string> &etags) = 0;
    virtual int abortMultipart(const std::string &key, const std::string &upload_id) = 0;
    virtual size_t minPartBytes() const = 0; // no part but the last may be smaller
    virtual std::string lastError() const = 0;
};

// "scheme://host[:port]" -> parts.  false: not an endpoint this client understands.
inline bool parseEndpoint(const std::string &url, std::string &scheme, std::string &host, uint16_t &port) {
    std::string rest = url;
    const size_t sep = rest.find("://");
    if (sep != std::string::npos) {
        scheme = rest.substr(0, sep);
        rest = rest.substr(sep + 3);
    }
    while (!rest.empty() && rest.back() == '/') rest.pop_back();
    if (rest.empty() || (scheme != "http" && scheme != "https")) return false;
    port = scheme == "https" ? 443 : 80;
    const size_t colon = rest.rfind(':');
    if (colon != std::string::npos && rest.find(']') == std::string::npos) {
        const long p = std::strtol(rest.c_str() + colon + 1, nullptr, 10);
        if (p <= 0 || p > 65535) return false;
        port = static_cast<uint16_t>(p);
        rest = rest.substr(0, colon);
    }
    host = rest;
    return !host.empty();
}

// ------------------------------------------------------------------ HTTP/1.1 requests over a pool of connections

class Http {
public:
    explicit Http(HttpConfig cfg) : cfg_(std::move(cfg)) {
        if (cfg_.scheme == "https") {
            const Tls &t = Tls::get();
            if (t.ok && (tlsCtx_ = t.SSL_CTX_new(t.TLS_client_method()))) {
                if (!cfg_.caBundle.empty()) t.SSL_CTX_load_verify_locations(tlsCtx_, cfg_.caBundle.c_str(), nullptr);
                else t.SSL_CTX_set_default_verify_paths(tlsCtx_);
                t.SSL_CTX_set_verify(tlsCtx_, cfg_.verifyTls ? 1 : 0, nullptr);
            }
        }
    }
    ~Http() {
        idle_.clear();
        if (tlsCtx_) Tls::get().SSL_CTX_free(tlsCtx_);
    }
    Http(const Http &) = delete;
    Http &operator=(const Http &) = delete;
    // false: https was asked for and no TLS library could be loaded
    bool usable() const { return cfg_.scheme != "https" || tlsCtx_; }
    const HttpConfig &config() const { return cfg_; }
    // "host" or "host:port" as it belongs into the Host header
    std::string hostHeader() const {
        const bool default_port = cfg_.port == (cfg_.scheme == "https" ? 443 : 80);
        return cfg_.host + (default_port ? "" : ":" + std::to_string(cfg_.port));
    }

    // Sends `head` (request line and headers, ending in an empty line) and `body`, reads the answer.  A successful
    // answer's body goes into `sink` (up to sink_len bytes, `*got` says how many came), anything else into
    // Response::body.  A connection that had been idle and fails before a single byte of the answer is tried once more
    // on a fresh one.
    Response roundTrip(const std::string &head, const void *body, size_t body_len, bool is_head, void *sink, size_t sink_len, size_t *got = nullptr) {
        for (int attempt = 0; attempt < 2; ++attempt) {
            std::unique_ptr<Conn> c = acquire();
            if (!c) return Response{};
            const bool was_reused = c->reused;
            bool fresh_failure = false;
            Response resp = onConnection(*c, head, body, body_len, is_head, sink, sink_len, got, fresh_failure);
            if (resp.status > 0) {
                auto it = resp.headers.find("connection");
                if (c->isOpen() && (it == resp.headers.end() || it->second != "close")) release(std::move(c));
                return resp;
            }
            if (!(was_reused && fresh_failure)) return resp;
        }
        return Response{};
    }

private:
    std::unique_ptr<Conn> acquire() {
        {
            std::lock_guard<std::mutex> g(mu_);
            if (!idle_.empty()) {
                auto c = std::move(idle_.back());
                idle_.pop_back();
                return c;
            }
        }
        auto c = std::make_unique<Conn>();
        if (!(!cfg_.connectHost.empty() && c->open(cfg_.connectHost, cfg_.port, tlsCtx_, cfg_.timeoutMs)) &&
            !c->open(cfg_.host, cfg_.port, tlsCtx_, cfg_.timeoutMs))
            return nullptr;
        return c;
    }
    void release(std::unique_ptr<Conn> c) {
        c->reused = true;
        std::lock_guard<std::mutex> g(mu_);
        if (idle_.size() < 64) idle_.push_back(std::move(c));
    }

    Response onConnection(Conn &c, const std::string &head, const void *body, size_t body_len, bool is_head, void *sink, size_t sink_len,
                          size_t *got, bool &before_answer) {
        Response resp;
        before_answer = true;
        if (body_len && body_len <= (16u << 10)) { // a small body rides in the packet of its headers
            std::string both = head;
            both.append(static_cast<const char *>(body), body_len);
            if (!c.writeAll(both.data(), both.size())) return c.close(), resp;
        } else if (!c.writeAll(head.data(), head.size()) || (body_len && !c.writeAll(body, body_len))) {
            return c.close(), resp;
        }
        // status line and headers
        std::string buf;
        size_t end = std::string::npos;
        char tmp[4096];
        while (end == std::string::npos) {
            const ssize_t k = c.readSome(tmp, sizeof(tmp));
            if (k <= 0) return c.close(), resp;
            before_answer = false;
            buf.append(tmp, static_cast<size_t>(k));
            end = buf.find("\r\n\r\n");
            if (buf.size() > (1u << 20)) return c.close(), resp;
        }
        std::string rest = buf.substr(end + 4);
        buf.resize(end);
        size_t line_end = buf.find("\r\n");
        const std::string status_line = buf.substr(0, line_end);
        int status = 0;
        if (status_line.size() > 12 && status_line.compare(0, 5, "HTTP/") == 0) status = std::atoi(status_line.c_str() + status_line.find(' ') + 1);
        if (status <= 0) return c.close(), resp;
        while (line_end != std::string::npos) {
            const size_t start = line_end + 2;
            line_end = buf.find("\r\n", start);
            const std::string line = buf.substr(start, line_end == std::string::npos ? std::string::npos : line_end - start);
            const size_t colon = line.find(':');
            if (colon == std::string::npos) continue;
            std::string name = line.substr(0, colon);
            std::transform(name.begin(), name.end(), name.begin(), [](unsigned char ch) { return static_cast<char>(std::tolower(ch)); });
            resp.headers[name] = trimmed(line.substr(colon + 1));
        }
        // body
        const bool no_body = is_head || status == 204 || status == 304 || (status >= 100 && status < 200);
        const bool to_sink = sink && (status == 200 || status == 206);
        size_t delivered = 0;
        auto take = [&](const char *p, size_t n) {
            if (to_sink) {
                const size_t k = std::min(n, sink_len - std::min(sink_len, delivered));
                std::memcpy(static_cast<char *>(sink) + delivered, p, k);
                delivered += n; // counts what came, so that an answer longer than the range shows
            } else if (resp.body.size() < (1u << 20)) {
                resp.body.append(p, n);
            }
        };
        bool ok = true;
        if (!no_body) {
            auto te = resp.headers.find("transfer-encoding");
            if (te != resp.headers.end() && te->second.find("chunked") != std::string::npos) {
                ok = readChunked(c, rest, take);
            } else {
                auto cl = resp.headers.find("content-length");
                uint64_t left = cl == resp.headers.end() ? 0 : std::strtoull(cl->second.c_str(), nullptr, 10);
                const size_t have = static_cast<size_t>(std::min<uint64_t>(left, rest.size()));
                take(rest.data(), have);
                left -= have;
                while (left && ok) {
                    // straight into the caller's buffer when that is where it belongs
                    if (to_sink && delivered < sink_len) {
                        const ssize_t k = c.readSome(static_cast<char *>(sink) + delivered, static_cast<size_t>(std::min<uint64_t>(left, sink_len - delivered)));
                        if (k <= 0) ok = false;
                        else {
                            delivered += static_cast<size_t>(k);
                            left -= static_cast<uint64_t>(k);
                        }
                    } else {
                        const ssize_t k = c.readSome(tmp, static_cast<size_t>(std::min<uint64_t>(left, sizeof(tmp))));
                        if (k <= 0) ok = false;
                        else {
                            take(tmp, static_cast<size_t>(k));
                            left -= static_cast<uint64_t>(k);
                        }
                    }
                }
                if (cl == resp.headers.end() && !no_body) c.close(); // length unknown: the body ends with the connection; not used by S3
            }
        }
        if (!ok) return c.close(), Response{};
        if (got) *got = delivered;
        resp.status = status;
        return resp;
    }

    template<class Take> static bool readChunked(Conn &c, std::string pending, Take &&take) {
        char tmp[4096];
        auto need = [&](size_t n) {
            while (pending.size() < n) {
                const ssize_t k = c.readSome(tmp, sizeof(tmp));
                if (k <= 0) return false;
                pending.append(tmp, static_cast<size_t>(k));
            }
            return true;
        };
        for (;;) {
            size_t eol;
            while ((eol = pending.find("\r\n")) == std::string::npos)
                if (!need(pending.size() + 1)) return false;
            const size_t n = std::strtoul(pending.c_str(), nullptr, 16);
            if (n > (64u << 20)) return false; // no answer this client reads in chunks is anywhere near that: do not trust the stream
            pending.erase(0, eol + 2);
            if (!need(n + 2)) return false;
            if (n == 0) return true; // (trailers are not used by S3)
            take(pending.data(), n);
            pending.erase(0, n + 2);
        }
    }

    HttpConfig cfg_;
    void *tlsCtx_ = nullptr;
    std::mutex mu_;
    std::vector<std::unique_ptr<Conn>> idle_;
};

// ------------------------------------------------------------------ the client

class Client final : public ObjectService {
public:
    explicit Client(Config cfg) : cfg_(std::move(cfg)), http_(withConnectHost(cfg_)) {}
    bool usable() const override { return http_.usable(); }
    const Config &config() const { return cfg_; }
    size_t minPartBytes() const override { return 5u << 20; }

    // Each returns the HTTP status (200, 206, 404, 403, ...) or 0 when the service could not be reached.
    int putObject(const std::string &key, const void *data, size_t len, std::string *etag = nullptr) override {
        Request r = base("PUT", key);
        if (cfg_.sendChecksum) r.headers["x-amz-checksum-crc32"] = crc32Header(crc32(data, len));
        Response resp = exchange(r, data, len, nullptr, 0);
        if (etag) *etag = resp.headers["etag"];
        return note(resp, "PutObject", key);
    }
    int getObject(const std::string &key, uint64_t offset, void *dst, size_t len) override {
        if (len == 0) return headObject(key, nullptr);
        Request r = base("GET", key);
        r.headers["range"] = "bytes=" + std::to_string(offset) + "-" + std::to_string(offset + len - 1);
        if (cfg_.checkChecksum) r.headers["x-amz-checksum-mode"] = "ENABLED";
        size_t got = 0;
        Response resp = exchange(r, nullptr, 0, dst, len, &got);
        if ((resp.status == 200 || resp.status == 206) && got != len) { // an object that ends before the range does
            std::lock_guard<std::mutex> g(mu_);
            lastError_ = "GetObject " + key + ": the object ends inside the requested range";
            return 416;
        }
        // The service sends the object's checksum only when the answer is the whole object.
        auto sum = resp.headers.find("x-amz-checksum-crc32");
        if (cfg_.checkChecksum && (resp.status == 200 || resp.status == 206) && sum != resp.headers.end() && sum->second.size() == 8 &&
            sum->second != crc32Header(crc32(dst, len))) {
            std::lock_guard<std::mutex> g(mu_);
            lastError_ = "GetObject " + key + ": the bytes received do not match the object's stored CRC32";
            return 500;
        }
        return note(resp, "GetObject", key);
    }
    int headObject(const std::string &key, uint64_t *size) override {
        Request r = base("HEAD", key);
        Response resp = exchange(r, nullptr, 0, nullptr, 0);
        if (size && resp.status == 200) *size = std::strtoull(resp.headers["content-length"].c_str(), nullptr, 10);
        return note(resp, "HeadObject", key);
    }
    int deleteObject(const std::string &key) override {
        Request r = base("DELETE", key);
        return note(exchange(r, nullptr, 0, nullptr, 0), "DeleteObject", key);
    }
    // Multipart upload: create -> parts (any order, in parallel) -> complete (or abort).
    int createMultipart(const std::string &key, std::string &upload_id) override {
        Request r = base("POST", key);
        r.query.emplace_back("uploads", "");
        Response resp = exchange(r, nullptr, 0, nullptr, 0);
        upload_id = between(resp.body, "<UploadId>", "</UploadId>");
        if (resp.status == 200 && upload_id.empty()) resp.status = 500;
        return note(resp, "CreateMultipartUpload", key);
    }
    int uploadPart(const std::string &key, const std::string &upload_id, int number, const void *data, size_t len, std::string &etag) override {
        Request r = base("PUT", key);
        r.query.emplace_back("partNumber", std::to_string(number));
        r.query.emplace_back("uploadId", upload_id);
        if (cfg_.sendChecksum) r.headers["x-amz-checksum-crc32"] = crc32Header(crc32(data, len));
        Response resp = exchange(r, data, len, nullptr, 0);
        etag = resp.headers["etag"];
        return note(resp, "UploadPart", key);
    }
    int completeMultipart(const std::string &key, const std::string &upload_id, const std::vector<std::string> &etags) override {
        std::string xml = "<CompleteMultipartUpload>";
        for (size_t i = 0; i < etags.size(); ++i)
            xml += "<Part><PartNumber>" + std::to_string(i + 1) + "</PartNumber><ETag>" + etags[i] + "</ETag></Part>";
        xml += "</CompleteMultipartUpload>";
        Request r = base("POST", key);
        r.query.emplace_back("uploadId", upload_id);
        Response resp = exchange(r, xml.data(), xml.size(), nullptr, 0);
        if (resp.status == 200 && resp.body.find("<Error>") != std::string::npos) resp.status = 500; // S3 reports some failures inside a 200
        return note(resp, "CompleteMultipartUpload", key);
    }
    int abortMultipart(const std::string &key, const std::string &upload_id) override {
        Request r = base("DELETE", key);
        r.query.emplace_back("uploadId", upload_id);
        return note(exchange(r, nullptr, 0, nullptr, 0), "AbortMultipartUpload", key);
    }
    std::string lastError() const override {
        std::lock_guard<std::mutex> g(mu_);
        return lastError_;
    }

private:
    static std::string between(const std::string &s, const std::string &a, const std::string &b) {
        const size_t i = s.find(a);
        if (i == std::string::npos) return "";
        const size_t j = s.find(b, i + a.size());
        return j == std::string::npos ? "" : s.substr(i + a.size(), j - i - a.size());
    }

    Request base(const char *method, const std::string &key) const {
        Request r;
        r.method = method;
        std::string host = http_.hostHeader();
        if (cfg_.virtualAddressing) {
            host = cfg_.bucket + "." + host;
            r.path = "/" + key;
        } else {
            r.path = "/" + cfg_.bucket + "/" + key;
        }
        r.headers["host"] = host;
        return r;
    }

    int note(const Response &resp, const char *what, const std::string &key) {
        if (resp.status >= 200 && resp.status < 300) return resp.status;
        std::lock_guard<std::mutex> g(mu_);
        if (resp.status <= 0) lastError_ = std::string(what) + " " + key + ": no answer from " + cfg_.host + ":" + std::to_string(cfg_.port);
        else
            lastError_ = std::string(what) + " " + key + ": HTTP " + std::to_string(resp.status) + " " + between(resp.body, "<Code>", "</Code>") + " " +
                between(resp.body, "<Message>", "</Message>");
        return resp.status;
    }

    // Signs and sends `r` with `body`; the answer as Http::roundTrip gives it.  Every attempt is signed afresh (the date
    // is part of the signature).
    Response exchange(Request &r, const void *body, size_t body_len, void *sink, size_t sink_len, size_t *got = nullptr) {
        return withRetries(cfg_.maxAttempts, [&] { return exchangeOnce(r, body, body_len, sink, sink_len, got); });
    }
    Response exchangeOnce(Request &r, const void *body, size_t body_len, void *sink, size_t sink_len, size_t *got) {
        const std::string date = amzDateNow();
        r.headers["x-amz-date"] = date;
        if (body_len && cfg_.signPayload) r.payloadHash = hex(sha256(body, body_len));
        else if (body_len) r.payloadHash = "UNSIGNED-PAYLOAD";
        else r.payloadHash = hex(sha256("", 0));
        r.headers["x-amz-content-sha256"] = r.payloadHash;
        if (!cfg_.cred.sessionToken.empty()) r.headers["x-amz-security-token"] = cfg_.cred.sessionToken;
        std::string head = r.method + " " + uriEncode(r.path, true);
        const std::string q = canonicalQuery(r);
        if (!q.empty()) head += "?" + q;
        head += " HTTP/1.1\r\n";
        for (const auto &kv : r.headers) head += kv.first + ": " + kv.second + "\r\n";
        if (!cfg_.cred.empty()) head += "authorization: " + authorizationV4(r, cfg_.cred, cfg_.region, "s3", date) + "\r\n";
        if (body_len || r.method == "PUT" || r.method == "POST") head += "content-length: " + std::to_string(body_len) + "\r\n";
        head += "\r\n";

        return http_.roundTrip(head, body, body_len, r.method == "HEAD", sink, sink_len, got);
    }

    static HttpConfig withConnectHost(const Config &cfg) {
        HttpConfig h = cfg;
        if (cfg.virtualAddressing) h.connectHost = cfg.bucket + "." + cfg.host; // where it resolves; else the endpoint itself
        return h;
    }

    Config cfg_;
    Http http_;
    mutable std::mutex mu_;
    std::string lastError_;
};

} // namespace nixl_s3

#endif

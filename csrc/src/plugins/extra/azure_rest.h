// Azure Blob Storage over its REST interface, for the OBJ engine built under the name AZURE_BLOB: Put Blob, ranged Get
// Blob, Get Blob Properties, Delete Blob, and block upload (Put Block + Put Block List) for large blobs, authorised with
// the account's Shared Key (HMAC-SHA256 over the canonicalised request) or a shared access signature.  Role parity: the
// reference's plug-in uses the Azure SDK for C++ (src/plugins/azure_blob/azure_blob_client.cpp); this build has no SDK,
// so the protocol is written out on top of the HTTP client of s3_rest.h.  Signing in with Microsoft Entra ID (the SDK's
// default credential chain) is not built: it needs a token service.
#ifndef NIXL_B200_AZURE_REST_H
#define NIXL_B200_AZURE_REST_H

#include "plugins/extra/s3_rest.h"

namespace nixl_azure {

inline std::string base64Encode(const uint8_t *p, size_t n) {
    static const char *t = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
    std::string out;
    for (size_t i = 0; i < n; i += 3) {
        const uint32_t v = (uint32_t(p[i]) << 16) | (i + 1 < n ? uint32_t(p[i + 1]) << 8 : 0) | (i + 2 < n ? uint32_t(p[i + 2]) : 0);
        out.push_back(t[(v >> 18) & 63]);
        out.push_back(t[(v >> 12) & 63]);
        out.push_back(i + 1 < n ? t[(v >> 6) & 63] : '=');
        out.push_back(i + 2 < n ? t[v & 63] : '=');
    }
    return out;
}
inline bool base64Decode(const std::string &s, std::vector<uint8_t> &out) {
    out.clear();
    uint32_t v = 0;
    int bits = 0;
    for (unsigned char c : s) {
        int d;
        if (c >= 'A' && c <= 'Z') d = c - 'A';
        else if (c >= 'a' && c <= 'z') d = c - 'a' + 26;
        else if (c >= '0' && c <= '9') d = c - '0' + 52;
        else if (c == '+') d = 62;
        else if (c == '/') d = 63;
        else if (c == '=') break;
        else return false;
        v = (v << 6) | static_cast<uint32_t>(d);
        bits += 6;
        if (bits >= 8) {
            bits -= 8;
            out.push_back(static_cast<uint8_t>(v >> bits));
        }
    }
    return true;
}

struct Config : nixl_s3::HttpConfig {
    std::string account, container;
    std::string pathPrefix;   // "/devstoreaccount1" when the account is part of the path (Azurite, custom endpoints)
    std::vector<uint8_t> key; // Shared Key, decoded
    std::string sas;          // shared access signature ("sv=...&sig=..."), used when there is no key
};

// "Name=value;Name=value" as the portal and Azurite give it.  false: `err` says what is missing.
inline bool parseConnectionString(const std::string &text, Config &cfg, std::string &err) {
    std::map<std::string, std::string> kv;
    size_t start = 0;
    while (start < text.size()) {
        size_t end = text.find(';', start);
        if (end == std::string::npos) end = text.size();
        const std::string item = text.substr(start, end - start);
        const size_t eq = item.find('=');
        if (eq != std::string::npos) kv[item.substr(0, eq)] = item.substr(eq + 1);
        start = end + 1;
    }
    if (kv["UseDevelopmentStorage"] == "true") { // the storage emulator's published account
        kv.emplace("AccountName", "devstoreaccount1");
        kv.emplace("AccountKey", "Eby8vdM02xNOcqFlqUwJPLlmEtlCDXJ1OUzFT50uSRZ6IFsuFq2UVErCz4I6tq/K1SZFPTOtr/KBHBeksoGMGw==");
        kv.emplace("BlobEndpoint", "http://127.0.0.1:10000/devstoreaccount1");
    }
    cfg.account = kv["AccountName"];
    if (!kv["AccountKey"].empty() && !base64Decode(kv["AccountKey"], cfg.key)) return err = "AccountKey is not base64", false;
    cfg.sas = kv["SharedAccessSignature"];
    if (!cfg.sas.empty() && cfg.sas[0] == '?') cfg.sas.erase(0, 1);
    std::string endpoint = kv["BlobEndpoint"];
    if (endpoint.empty()) {
        if (cfg.account.empty()) return err = "neither BlobEndpoint nor AccountName", false;
        const std::string proto = kv["DefaultEndpointsProtocol"].empty() ? "https" : kv["DefaultEndpointsProtocol"];
        const std::string suffix = kv["EndpointSuffix"].empty() ? "core.windows.net" : kv["EndpointSuffix"];
        endpoint = proto + "://" + cfg.account + ".blob." + suffix;
    }
    // scheme://host[:port][/path]
    const size_t sep = endpoint.find("://");
    const size_t slash = endpoint.find('/', sep == std::string::npos ? 0 : sep + 3);
    if (slash != std::string::npos) {
        cfg.pathPrefix = endpoint.substr(slash);
        while (!cfg.pathPrefix.empty() && cfg.pathPrefix.back() == '/') cfg.pathPrefix.pop_back();
        endpoint.resize(slash);
    }
    if (!nixl_s3::parseEndpoint(endpoint, cfg.scheme, cfg.host, cfg.port)) return err = "cannot use endpoint '" + endpoint + "'", false;
    if (cfg.account.empty()) { // https://<account>.blob.<suffix>, or the first piece of the path
        if (!cfg.pathPrefix.empty()) cfg.account = cfg.pathPrefix.substr(1, cfg.pathPrefix.find('/', 1) - 1);
        else cfg.account = cfg.host.substr(0, cfg.host.find('.'));
    }
    if (cfg.key.empty() && cfg.sas.empty()) return err = "no AccountKey and no SharedAccessSignature (signing in with Entra ID is not built)", false;
    return true;
}

inline std::string httpDateNow() {
    const std::time_t t = std::time(nullptr);
    std::tm tm{};
    ::gmtime_r(&t, &tm);
    char buf[64];
    std::strftime(buf, sizeof(buf), "%a, %d %b %Y %H:%M:%S GMT", &tm);
    return buf;
}

struct Request {
    std::string method, path; // path as it goes on the wire, already escaped
    std::vector<std::pair<std::string, std::string>> query;
    std::map<std::string, std::string> headers; // lower-case names
    size_t contentLength = 0;
};

// The text the Shared Key signs (service version 2015-02-21 and later).
inline std::string stringToSign(const Request &r, const std::string &account) {
    auto h = [&](const char *name) {
        auto it = r.headers.find(name);
        return it == r.headers.end() ? std::string() : it->second;
    };
    std::string s = r.method + "\n" + h("content-encoding") + "\n" + h("content-language") + "\n" +
        (r.contentLength ? std::to_string(r.contentLength) : std::string()) + "\n" + h("content-md5") + "\n" + h("content-type") + "\n" + h("date") + "\n" +
        h("if-modified-since") + "\n" + h("if-match") + "\n" + h("if-none-match") + "\n" + h("if-unmodified-since") + "\n" + h("range") + "\n";
    for (const auto &kv : r.headers)
        if (kv.first.compare(0, 5, "x-ms-") == 0) s += kv.first + ":" + nixl_s3::trimmed(kv.second) + "\n";
    s += "/" + account + r.path;
    std::vector<std::pair<std::string, std::string>> q = r.query;
    for (auto &kv : q) std::transform(kv.first.begin(), kv.first.end(), kv.first.begin(), [](unsigned char c) { return static_cast<char>(std::tolower(c)); });
    std::sort(q.begin(), q.end());
    for (const auto &kv : q) s += "\n" + kv.first + ":" + kv.second;
    return s;
}

inline std::string sharedKeyAuthorization(const Request &r, const std::string &account, const std::vector<uint8_t> &key) {
    const std::string text = stringToSign(r, account);
    const nixl_s3::Digest mac = nixl_s3::hmacSha256(key.data(), key.size(), text.data(), text.size());
    return "SharedKey " + account + ":" + base64Encode(mac.data(), mac.size());
}

class Client final : public nixl_s3::ObjectService {
public:
    explicit Client(Config cfg) : cfg_(std::move(cfg)), http_(cfg_) {}
    bool usable() const override { return http_.usable(); }
    size_t minPartBytes() const override { return 1; } // blocks may have any size
    const Config &config() const { return cfg_; }

    int putObject(const std::string &key, const void *data, size_t len, std::string *etag = nullptr) override {
        Request r = base("PUT", key);
        r.headers["x-ms-blob-type"] = "BlockBlob";
        nixl_s3::Response resp = exchange(r, data, len, nullptr, 0);
        if (etag) *etag = resp.headers["etag"];
        return note(resp, "Put Blob", key);
    }
    int getObject(const std::string &key, uint64_t offset, void *dst, size_t len) override {
        if (len == 0) return headObject(key, nullptr);
        Request r = base("GET", key);
        r.headers["x-ms-range"] = "bytes=" + std::to_string(offset) + "-" + std::to_string(offset + len - 1);
        size_t got = 0;
        nixl_s3::Response resp = exchange(r, nullptr, 0, dst, len, &got);
        if ((resp.status == 200 || resp.status == 206) && got != len) {
            std::lock_guard<std::mutex> g(mu_);
            lastError_ = "Get Blob " + key + ": the blob ends inside the requested range";
            return 416;
        }
        return note(resp, "Get Blob", key);
    }
    int headObject(const std::string &key, uint64_t *size) override {
        Request r = base("HEAD", key);
        nixl_s3::Response resp = exchange(r, nullptr, 0, nullptr, 0);
        if (size && resp.status == 200) *size = std::strtoull(resp.headers["content-length"].c_str(), nullptr, 10);
        return note(resp, "Get Blob Properties", key);
    }
    int deleteObject(const std::string &key) override {
        Request r = base("DELETE", key);
        return note(exchange(r, nullptr, 0, nullptr, 0), "Delete Blob", key);
    }
    // Blocks need no announcement; the "upload id" is only there for the interface.
    int createMultipart(const std::string &, std::string &upload_id) override {
        upload_id = "blocks";
        return 200;
    }
    int uploadPart(const std::string &key, const std::string &, int number, const void *data, size_t len, std::string &etag) override {
        etag = blockId(number);
        Request r = base("PUT", key);
        r.query = {{"comp", "block"}, {"blockid", etag}};
        return note(exchange(r, data, len, nullptr, 0), "Put Block", key);
    }
    int completeMultipart(const std::string &key, const std::string &, const std::vector<std::string> &ids) override {
        std::string xml = "<?xml version=\"1.0\" encoding=\"utf-8\"?><BlockList>";
        for (const auto &id : ids) xml += "<Latest>" + id + "</Latest>";
        xml += "</BlockList>";
        Request r = base("PUT", key);
        r.query = {{"comp", "blocklist"}};
        r.headers["content-type"] = "application/xml";
        return note(exchange(r, xml.data(), xml.size(), nullptr, 0), "Put Block List", key);
    }
    int abortMultipart(const std::string &, const std::string &) override { return 204; } // blocks never committed expire by themselves
    std::string lastError() const override {
        std::lock_guard<std::mutex> g(mu_);
        return lastError_;
    }

private:
    static std::string blockId(int number) { // ids of one blob must have one length
        char buf[16];
        std::snprintf(buf, sizeof(buf), "block-%08d", number);
        return base64Encode(reinterpret_cast<const uint8_t *>(buf), std::strlen(buf));
    }
    Request base(const char *method, const std::string &key) const {
        Request r;
        r.method = method;
        r.path = cfg_.pathPrefix + "/" + nixl_s3::uriEncode(cfg_.container, false) + "/" + nixl_s3::uriEncode(key, true);
        r.headers["x-ms-date"] = httpDateNow();
        r.headers["x-ms-version"] = "2021-08-06";
        return r;
    }
    int note(const nixl_s3::Response &resp, const char *what, const std::string &key) {
        if (resp.status >= 200 && resp.status < 300) return resp.status;
        std::lock_guard<std::mutex> g(mu_);
        auto between = [&](const char *a, const char *b) {
            const size_t i = resp.body.find(a);
            if (i == std::string::npos) return std::string();
            const size_t j = resp.body.find(b, i);
            return j == std::string::npos ? std::string() : resp.body.substr(i + std::strlen(a), j - i - std::strlen(a));
        };
        if (resp.status <= 0) lastError_ = std::string(what) + " " + key + ": no answer from " + cfg_.host + ":" + std::to_string(cfg_.port);
        else lastError_ = std::string(what) + " " + key + ": HTTP " + std::to_string(resp.status) + " " + between("<Code>", "</Code>") + " " + between("<Message>", "</Message>");
        return resp.status;
    }
    nixl_s3::Response exchange(Request &r, const void *body, size_t body_len, void *sink, size_t sink_len, size_t *got = nullptr) {
        return nixl_s3::withRetries(cfg_.maxAttempts, [&] {
            r.headers["x-ms-date"] = httpDateNow();
            return exchangeOnce(r, body, body_len, sink, sink_len, got);
        });
    }
    nixl_s3::Response exchangeOnce(Request &r, const void *body, size_t body_len, void *sink, size_t sink_len, size_t *got) {
        r.contentLength = body_len;
        std::string target = r.path;
        char sep = '?';
        for (const auto &kv : r.query) {
            target += sep + nixl_s3::uriEncode(kv.first, false) + "=" + nixl_s3::uriEncode(kv.second, false);
            sep = '&';
        }
        if (cfg_.key.empty() && !cfg_.sas.empty()) target += sep + cfg_.sas;
        std::string head = r.method + " " + target + " HTTP/1.1\r\nhost: " + http_.hostHeader() + "\r\n";
        for (const auto &kv : r.headers) head += kv.first + ": " + kv.second + "\r\n";
        if (!cfg_.key.empty()) head += "authorization: " + sharedKeyAuthorization(r, cfg_.account, cfg_.key) + "\r\n";
        if (body_len || r.method == "PUT") head += "content-length: " + std::to_string(body_len) + "\r\n";
        head += "\r\n";
        return http_.roundTrip(head, body, body_len, r.method == "HEAD", sink, sink_len, got);
    }

    Config cfg_;
    nixl_s3::Http http_;
    mutable std::mutex mu_;
    std::string lastError_;
};

} // namespace nixl_azure

#endif

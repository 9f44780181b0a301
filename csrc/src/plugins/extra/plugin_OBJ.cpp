// OBJ backend: host memory <-> named objects.  The reference's OBJ plugin talks to S3
// (src/plugins/obj: local-only, DRAM + OBJ, object key in the registration's metaInfo, devId a
// caller-chosen id, asynchronous put/get).  Two stores:
//
//   * an S3 service, when an endpoint is named (`endpoint_override` parameter or $AWS_ENDPOINT_OVERRIDE, e.g.
//     "http://minio:9000" or "https://s3.us-west-2.amazonaws.com"): the REST client of s3_rest.h, with the reference's
//     parameters (`bucket` / $AWS_DEFAULT_BUCKET, `access_key`, `secret_key`, `session_token` or the AWS_* variables,
//     `region`, `scheme`, `use_virtual_addressing`, `ca_bundle`, `crtMinLimit`, `req_checksum`, `resp_checksum`).  WRITE puts the whole object (an
//     offset other than 0 is refused, as in the reference), READ gets a byte range, queryMem asks HeadObject.  Objects of
//     at least `crtMinLimit` bytes take the role of the reference's second client: a multipart upload whose parts, and a
//     download whose ranges, run side by side on the engine's threads.  `payload_signing` (default: on over http, off
//     over https, as the SDK does) says whether a PUT's body is hashed into its signature.
//   * a directory, otherwise: bucket = directory (`bucket` parameter, else $NIXL_OBJ_BUCKET_DIR, else
//     /tmp/nixl_obj), object = file named by its key; WRITE puts [offset, offset+len) of the object, READ gets it.
//
// The same engine is also built under the reference's other object-store names, with the
// parameter that names the bucket in each of them (NIXL_OBJ_PLUGIN_NAME / NIXL_OBJ_BUCKET_PARAM):
//   * AZURE_BLOB (`container_name`; src/plugins/azure_blob): Azure Blob Storage over REST (azure_rest.h) when a
//     `connection_string` (or $AZURE_STORAGE_CONNECTION_STRING) names the account: Shared Key or shared access
//     signature; blobs of at least `crtMinLimit` bytes go up as blocks side by side.  An `account_url` with
//     `account_key` (or $AZURE_STORAGE_KEY) or `sas_token` (or $AZURE_STORAGE_SAS_TOKEN) beside it does the same.  With
//     only an `account_url` (Entra ID sign-in, not built) the directory store answers, with a warning.
//   * INFINIA (`dataset`; src/plugins/infinia): there is no client for that appliance's own protocol; its cluster and
//     tenant parameters are accepted and ignored.  The directory store answers, or, when `endpoint_override` names an
//     S3-compatible endpoint, the S3 client with `dataset` as the bucket.
#ifndef NIXL_OBJ_PLUGIN_NAME
#define NIXL_OBJ_PLUGIN_NAME "OBJ"
#endif
#ifndef NIXL_OBJ_BUCKET_PARAM
#define NIXL_OBJ_BUCKET_PARAM "bucket"
#endif
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <memory>

#include "backend/backend_plugin.h"
#include "plugins/extra/azure_rest.h"
#include "plugins/extra/s3_rest.h"
#include "utils/file/file_utils.h"
#include "utils/log.h"
#include "utils/thread_pool.h"

namespace {

class ObjMD final : public nixlBackendMD {
public:
    explicit ObjMD(std::string k) : nixlBackendMD(true), key(std::move(k)) {}
    std::string key;
};

struct ObjIo {
    std::string path; // directory store: the file; S3: the key
    off_t offset;
    char *mem;
    size_t len;
    bool put;
};

class ObjReq final : public nixlBackendReqH {
public:
    std::vector<ObjIo> ios;
    std::atomic<size_t> remaining{0};
    std::atomic<int> error{0};
    bool posted = false;
};

int objectIo(const ObjIo &io) {
    const int fd = ::open(io.path.c_str(), io.put ? (O_WRONLY | O_CREAT) : O_RDONLY, 0644);
    if (fd < 0) return errno;
    char *p = io.mem;
    size_t n = io.len;
    off_t off = io.offset;
    int err = 0;
    while (n && !err) {
        const ssize_t r = io.put ? ::pwrite(fd, p, n, off) : ::pread(fd, p, n, off);
        if (r < 0) {
            if (errno != EINTR) err = errno;
        } else if (r == 0) err = EIO;
        else {
            p += r;
            off += r;
            n -= static_cast<size_t>(r);
        }
    }
    ::close(fd);
    return err;
}

class ObjEngine final : public nixlBackendEngine {
public:
    explicit ObjEngine(const nixlBackendInitParams *p) : nixlBackendEngine(p) {
        std::string v;
        // (INFINIA: no client for the appliance's own protocol here, but an S3-compatible endpoint, if the deployment
        // offers one, is served like any other: `endpoint_override`, with `dataset` naming the bucket.)
        const bool is_azure = std::strcmp(NIXL_OBJ_PLUGIN_NAME, "AZURE_BLOB") == 0, is_s3 = !is_azure;
        if ((is_s3 && !setupS3()) || (is_azure && !setupAzure())) {
            initErr = true;
            return;
        }
        if (!s3_ && std::strcmp(NIXL_OBJ_PLUGIN_NAME, "OBJ") != 0)
            NIXL_WARN << NIXL_OBJ_PLUGIN_NAME << " backend: " << (is_azure ? "no connection string was given" : "this build has no client for that service and no S3 endpoint was named")
                      << "; objects are files in a local directory";
        if (!s3_) {
            if (getInitParam(NIXL_OBJ_BUCKET_PARAM, v) == NIXL_SUCCESS && !v.empty()) dir_ = v;
            else if (const char *e = std::getenv("NIXL_OBJ_BUCKET_DIR")) dir_ = e;
            else dir_ = "/tmp/nixl_obj";
            ::mkdir(dir_.c_str(), 0755);
        }
        unsigned threads = s3_ ? 8 : 4;
        if (getInitParam("num_threads", v) == NIXL_SUCCESS && std::atoi(v.c_str()) > 0) threads = static_cast<unsigned>(std::atoi(v.c_str()));
        pool_ = std::make_unique<nixlThreadPool>(threads);
    }
    bool supportsRemote() const override { return false; }
    bool supportsLocal() const override { return true; }
    bool supportsNotif() const override { return false; }
    nixl_mem_list_t getSupportedMems() const override { return {DRAM_SEG, OBJ_SEG}; }

    nixl_status_t registerMem(const nixlBlobDesc &mem, const nixl_mem_t &nixl_mem, nixlBackendMD *&out) override {
        out = nullptr;
        if (nixl_mem == DRAM_SEG) return NIXL_SUCCESS;
        if (nixl_mem != OBJ_SEG) return NIXL_ERR_NOT_SUPPORTED;
        // Key: metaInfo, or the decimal devId when none is given.  No path separators: one flat bucket.
        std::string key = mem.metaInfo.empty() ? std::to_string(mem.devId) : mem.metaInfo;
        if (!s3_ && (key.find('/') != std::string::npos || key == "." || key == "..")) return NIXL_ERR_INVALID_PARAM;
        if (key.empty()) return NIXL_ERR_INVALID_PARAM;
        out = new ObjMD(key);
        return NIXL_SUCCESS;
    }
    nixl_status_t deregisterMem(nixlBackendMD *meta) override {
        delete meta;
        return NIXL_SUCCESS;
    }
    nixl_status_t connect(const std::string &) override { return NIXL_SUCCESS; }
    nixl_status_t disconnect(const std::string &) override { return NIXL_SUCCESS; }
    nixl_status_t unloadMD(nixlBackendMD *) override { return NIXL_SUCCESS; }
    nixl_status_t loadLocalMD(nixlBackendMD *input, nixlBackendMD *&output) override {
        output = input;
        return NIXL_SUCCESS;
    }
    nixl_status_t prepXfer(const nixl_xfer_op_t &op, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote,
                           const std::string &remote_agent, nixlBackendReqH *&handle, const nixl_opt_b_args_t *) const override {
        if (remote_agent != localAgent || local.getType() != DRAM_SEG || remote.getType() != OBJ_SEG || local.descCount() != remote.descCount())
            return NIXL_ERR_INVALID_PARAM;
        auto req = std::make_unique<ObjReq>();
        for (int i = 0; i < local.descCount(); ++i) {
            auto *o = dynamic_cast<ObjMD *>(remote[i].metadataP);
            if (!o || local[i].len != remote[i].len) return NIXL_ERR_INVALID_PARAM;
            if (s3_ && op == NIXL_WRITE && remote[i].addr != 0) {
                NIXL_ERROR << "OBJ backend: an object is written whole; offset " << remote[i].addr << " of " << o->key << " is not 0";
                return NIXL_ERR_NOT_SUPPORTED;
            }
            req->ios.push_back({s3_ ? o->key : dir_ + "/" + o->key, static_cast<off_t>(remote[i].addr), reinterpret_cast<char *>(local[i].addr),
                                local[i].len, op == NIXL_WRITE});
        }
        handle = req.release();
        return NIXL_SUCCESS;
    }
    nixl_status_t postXfer(const nixl_xfer_op_t &, const nixl_meta_dlist_t &, const nixl_meta_dlist_t &, const std::string &,
                           nixlBackendReqH *&handle, const nixl_opt_b_args_t *) const override {
        auto *req = dynamic_cast<ObjReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        req->error = 0;
        req->remaining = req->ios.size();
        req->posted = true;
        for (const ObjIo &io : req->ios) {
            if (s3_) {
                s3Start(req, io);
                continue;
            }
            pool_->submit([req, io] { finish(req, objectIo(io)); });
        }
        return checkXfer(handle);
    }
    nixl_status_t checkXfer(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<ObjReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        if (!req->posted) return NIXL_ERR_NOT_POSTED;
        if (req->remaining.load(std::memory_order_acquire)) return NIXL_IN_PROG;
        if (const int e = req->error.load()) return e == ENOENT ? NIXL_ERR_NOT_FOUND : e == EACCES ? NIXL_ERR_NOT_ALLOWED : NIXL_ERR_BACKEND;
        return NIXL_SUCCESS;
    }
    nixl_status_t releaseReqH(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<ObjReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        while (req->posted && req->remaining.load(std::memory_order_acquire)) std::this_thread::yield();
        delete req;
        return NIXL_SUCCESS;
    }
    nixl_status_t queryMem(const nixl_reg_dlist_t &descs, std::vector<nixl_query_resp_t> &resp) const override {
        if (s3_) {
            resp.clear();
            for (const auto &d : descs) {
                uint64_t size = 0;
                const int st = s3_->headObject(d.metaInfo.empty() ? std::to_string(d.devId) : d.metaInfo, &size);
                if (st == 200) resp.push_back(nixl_b_params_t{{"size", std::to_string(size)}});
                else if (st == 404) resp.push_back(std::nullopt);
                else {
                    NIXL_ERROR << "OBJ backend: " << s3_->lastError();
                    return NIXL_ERR_BACKEND;
                }
            }
            return NIXL_SUCCESS;
        }
        std::vector<std::string> names;
        for (const auto &d : descs) names.push_back(dir_ + "/" + (d.metaInfo.empty() ? std::to_string(d.devId) : d.metaInfo));
        return nixl::queryFileInfoList(names, resp);
    }

private:
    static void finish(ObjReq *req, int err) {
        if (err) {
            int zero = 0;
            req->error.compare_exchange_strong(zero, err);
        }
        req->remaining.fetch_sub(1, std::memory_order_acq_rel); // the request may be released from here on
    }
    static int errnoOf(int http_status) {
        if (http_status >= 200 && http_status < 300) return 0;
        return http_status == 404 ? ENOENT : http_status == 403 || http_status == 401 ? EACCES : http_status == 0 ? ECONNREFUSED : EIO;
    }
    std::string param(const char *key, const char *env = nullptr) const {
        std::string v;
        if (getInitParam(key, v) == NIXL_SUCCESS && !v.empty()) return v;
        if (env)
            if (const char *e = std::getenv(env)) return e;
        return "";
    }

    // S3 mode when an endpoint is named.  false: it was named and cannot be used.
    bool setupS3() {
        const std::string endpoint = param("endpoint_override", "AWS_ENDPOINT_OVERRIDE");
        if (endpoint.empty()) return true;
        nixl_s3::Config cfg;
        const std::string scheme = param("scheme");
        cfg.scheme = scheme.empty() ? "https" : scheme;
        if (!nixl_s3::parseEndpoint(endpoint, cfg.scheme, cfg.host, cfg.port)) {
            NIXL_ERROR << "OBJ backend: cannot use endpoint '" << endpoint << "' (http://host[:port] or https://host[:port])";
            return false;
        }
        cfg.bucket = param(NIXL_OBJ_BUCKET_PARAM, "AWS_DEFAULT_BUCKET");
        if (cfg.bucket.empty()) {
            NIXL_ERROR << "OBJ backend: no bucket (parameter 'bucket' or AWS_DEFAULT_BUCKET)";
            return false;
        }
        cfg.cred.accessKey = param("access_key", "AWS_ACCESS_KEY_ID");
        cfg.cred.secretKey = param("secret_key", "AWS_SECRET_ACCESS_KEY");
        cfg.cred.sessionToken = param("session_token", "AWS_SESSION_TOKEN");
        std::string region = param("region", "AWS_REGION");
        if (region.empty()) region = param("region", "AWS_DEFAULT_REGION");
        if (!region.empty()) cfg.region = region;
        cfg.virtualAddressing = param("use_virtual_addressing") == "true";
        cfg.caBundle = param("ca_bundle", "AWS_CA_BUNDLE");
        const std::string signing = param("payload_signing");
        cfg.signPayload = signing.empty() ? cfg.scheme == "http" : signing == "true";
        // "supported": use checksums where the service takes them; "required" (and nothing): only where the protocol
        // demands one, which none of the calls made here does.  The names are the reference's.
        if (const std::string tries = param("max_attempts"); !tries.empty()) cfg.maxAttempts = std::max(1, std::atoi(tries.c_str()));
        cfg.sendChecksum = param("req_checksum") == "supported";
        cfg.checkChecksum = param("resp_checksum") == "supported";
        const std::string limit = param("crtMinLimit");
        if (!limit.empty()) {
            const long long n = std::atoll(limit.c_str());
            if (n > 0) largeLimit_ = static_cast<size_t>(n);
        }
        if (cfg.cred.empty()) NIXL_WARN << "OBJ backend: no credentials (access_key / secret_key or AWS_ACCESS_KEY_ID / AWS_SECRET_ACCESS_KEY): requests go out unsigned";
        s3_ = std::make_unique<nixl_s3::Client>(cfg);
        if (!s3_->usable()) {
            NIXL_ERROR << "OBJ backend: https endpoint but no TLS library (libssl) could be loaded";
            return false;
        }
        return true;
    }

    // Azure Blob Storage when a connection string names an account (`connection_string` or
    // $AZURE_STORAGE_CONNECTION_STRING; `container_name` or $AZURE_STORAGE_CONTAINER_NAME).  An `account_url` alone means
    // signing in with Entra ID, which is not built: the directory store answers then, with a warning.
    bool setupAzure() {
        std::string conn = param("connection_string", "AZURE_STORAGE_CONNECTION_STRING");
        if (conn.empty()) {
            // An account URL with the account's key or a shared access signature beside it says the same as a
            // connection string; an account URL alone means Entra ID.
            const std::string url = param("account_url", "AZURE_STORAGE_ACCOUNT_URL");
            const std::string key = param("account_key", "AZURE_STORAGE_KEY"), sas = param("sas_token", "AZURE_STORAGE_SAS_TOKEN");
            if (url.empty() || (key.empty() && sas.empty())) return true;
            conn = "BlobEndpoint=" + url + ";" + (key.empty() ? "SharedAccessSignature=" + sas : "AccountKey=" + key);
            if (const std::string name = param("account_name", "AZURE_STORAGE_ACCOUNT"); !name.empty()) conn += ";AccountName=" + name;
        }
        nixl_azure::Config cfg;
        std::string err;
        if (!nixl_azure::parseConnectionString(conn, cfg, err)) {
            NIXL_ERROR << "AZURE_BLOB backend: connection string: " << err;
            return false;
        }
        cfg.container = param(NIXL_OBJ_BUCKET_PARAM, "AZURE_STORAGE_CONTAINER_NAME");
        if (cfg.container.empty()) {
            NIXL_ERROR << "AZURE_BLOB backend: no container (parameter 'container_name' or AZURE_STORAGE_CONTAINER_NAME)";
            return false;
        }
        cfg.caBundle = param("ca_bundle", "AZURE_CA_BUNDLE");
        if (const std::string tries = param("max_attempts"); !tries.empty()) cfg.maxAttempts = std::max(1, std::atoi(tries.c_str()));
        const std::string limit = param("crtMinLimit");
        if (!limit.empty() && std::atoll(limit.c_str()) > 0) largeLimit_ = static_cast<size_t>(std::atoll(limit.c_str()));
        s3_ = std::make_unique<nixl_azure::Client>(cfg);
        if (!s3_->usable()) {
            NIXL_ERROR << "AZURE_BLOB backend: https endpoint but no TLS library (libssl) could be loaded";
            return false;
        }
        return true;
    }

    // Progress of one object moved in pieces.
    struct Pieces {
        ObjReq *req;
        ObjIo io;
        std::string uploadId;
        std::vector<std::string> etags;
        std::atomic<size_t> left{0};
        std::atomic<int> err{0};
        size_t piece = 0;
    };

    void s3Start(ObjReq *req, const ObjIo &io) const {
        const bool large = largeLimit_ && io.len >= largeLimit_ && io.len > 0;
        if (!large) {
            pool_->submit([this, req, io] {
                const int st = io.put ? s3_->putObject(io.path, io.mem, io.len) : s3_->getObject(io.path, static_cast<uint64_t>(io.offset), io.mem, io.len);
                if (errnoOf(st)) NIXL_ERROR << "OBJ backend: " << s3_->lastError();
                finish(req, errnoOf(st));
            });
            return;
        }
        auto ps = std::make_shared<Pieces>();
        ps->req = req;
        ps->io = io;
        // S3 takes no part under 5 MiB except the last one; ranges of a download have no such rule.
        ps->piece = io.put ? std::max(largeLimit_, s3_->minPartBytes()) : largeLimit_;
        const size_t n = (io.len + ps->piece - 1) / ps->piece;
        ps->etags.resize(n);
        ps->left.store(n);
        auto piece_task = [this, ps](size_t i) {
            const size_t off = i * ps->piece, len = std::min(ps->piece, ps->io.len - off);
            int st = 0;
            if (ps->err.load() == 0) { // after a failure the other pieces are not worth the traffic
                st = ps->io.put ? s3_->uploadPart(ps->io.path, ps->uploadId, static_cast<int>(i + 1), ps->io.mem + off, len, ps->etags[i])
                                : s3_->getObject(ps->io.path, static_cast<uint64_t>(ps->io.offset) + off, ps->io.mem + off, len);
                if (const int e = errnoOf(st)) {
                    NIXL_ERROR << "OBJ backend: " << s3_->lastError();
                    int zero = 0;
                    ps->err.compare_exchange_strong(zero, e);
                }
            }
            if (ps->left.fetch_sub(1, std::memory_order_acq_rel) != 1) return;
            int err = ps->err.load();
            if (ps->io.put) { // the last piece closes the upload
                if (!err) {
                    err = errnoOf(s3_->completeMultipart(ps->io.path, ps->uploadId, ps->etags));
                    if (err) NIXL_ERROR << "OBJ backend: " << s3_->lastError();
                }
                if (err) s3_->abortMultipart(ps->io.path, ps->uploadId);
            }
            finish(ps->req, err);
        };
        pool_->submit([this, ps, n, piece_task] {
            if (ps->io.put) {
                const int st = s3_->createMultipart(ps->io.path, ps->uploadId);
                if (const int e = errnoOf(st)) {
                    NIXL_ERROR << "OBJ backend: " << s3_->lastError();
                    finish(ps->req, e);
                    return;
                }
            }
            for (size_t i = 1; i < n; ++i) pool_->submit([piece_task, i] { piece_task(i); });
            piece_task(0);
        });
    }

    std::string dir_;
    std::unique_ptr<nixl_s3::ObjectService> s3_; // the object service (S3 or Azure Blob); none: a directory
    size_t largeLimit_ = 0; // objects of at least this many bytes move in pieces (0: never)
    std::unique_ptr<nixlThreadPool> pool_;
};

} // namespace

extern "C" NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init() {
    return nixlBackendPluginCreator<ObjEngine>::create(NIXL_PLUGIN_API_VERSION, NIXL_OBJ_PLUGIN_NAME, "1.0.0",
                                                       {{NIXL_OBJ_BUCKET_PARAM, ""},
                                                        {"num_threads", ""},
                                                        {"endpoint_override", ""},
                                                        {"access_key", ""},
                                                        {"secret_key", ""},
                                                        {"session_token", ""},
                                                        {"scheme", "https"},
                                                        {"region", "us-east-1"},
                                                        {"use_virtual_addressing", "false"},
                                                        {"ca_bundle", ""},
                                                        {"crtMinLimit", ""},
                                                        {"payload_signing", ""},
                                                        {"max_attempts", "3"},
                                                        {"req_checksum", ""},
                                                        {"resp_checksum", ""},
                                                        {"connection_string", ""},
                                                        {"account_url", ""},
                                                        {"account_key", ""},
                                                        {"account_name", ""},
                                                        {"sas_token", ""}},
                                                       {DRAM_SEG, OBJ_SEG});
}
extern "C" NIXL_PLUGIN_EXPORT void nixl_plugin_fini() {}

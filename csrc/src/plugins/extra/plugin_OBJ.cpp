// OBJ backend: host memory <-> named objects.  The reference's OBJ plugin talks to S3
// (src/plugins/obj: local-only, DRAM + OBJ, object key in the registration's metaInfo, devId a
// caller-chosen id, asynchronous put/get).  This build has no S3 client: the object store is
// a directory: bucket = directory (`bucket` parameter, else $NIXL_OBJ_BUCKET_DIR, else
// /tmp/nixl_obj), object = file named by its key.  WRITE puts [offset, offset+len) of the
// object, READ gets it; queryMem tells whether a key exists.  The engine keeps the reference's
// contract so an S3 transport can replace the file calls without touching callers.
//
// The same engine is also built under the reference's other object-store names, with the
// parameter that names the bucket in each of them (NIXL_OBJ_PLUGIN_NAME / NIXL_OBJ_BUCKET_PARAM):
// AZURE_BLOB (`container_name`; src/plugins/azure_blob) and INFINIA (`dataset`;
// src/plugins/infinia).  Their remaining parameters (account URLs, cluster and tenant names) are
// accepted and ignored: there is no service to talk to.
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
    std::string path;
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
        if (std::strcmp(NIXL_OBJ_PLUGIN_NAME, "OBJ") != 0)
            NIXL_WARN << NIXL_OBJ_PLUGIN_NAME << " backend: this build has no client for that service; objects are files in a local directory";
        std::string v;
        if (getInitParam(NIXL_OBJ_BUCKET_PARAM, v) == NIXL_SUCCESS && !v.empty()) dir_ = v;
        else if (const char *e = std::getenv("NIXL_OBJ_BUCKET_DIR")) dir_ = e;
        else dir_ = "/tmp/nixl_obj";
        ::mkdir(dir_.c_str(), 0755);
        unsigned threads = 4;
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
        if (key.find('/') != std::string::npos || key == "." || key == "..") return NIXL_ERR_INVALID_PARAM;
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
            req->ios.push_back({dir_ + "/" + o->key, static_cast<off_t>(remote[i].addr), reinterpret_cast<char *>(local[i].addr), local[i].len,
                                op == NIXL_WRITE});
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
        for (const ObjIo &io : req->ios)
            pool_->submit([req, io] {
                if (const int e = objectIo(io)) {
                    int zero = 0;
                    req->error.compare_exchange_strong(zero, e);
                }
                req->remaining.fetch_sub(1, std::memory_order_acq_rel);
            });
        return checkXfer(handle);
    }
    nixl_status_t checkXfer(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<ObjReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        if (!req->posted) return NIXL_ERR_NOT_POSTED;
        if (req->remaining.load(std::memory_order_acquire)) return NIXL_IN_PROG;
        if (const int e = req->error.load()) return e == ENOENT ? NIXL_ERR_NOT_FOUND : NIXL_ERR_BACKEND;
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
        std::vector<std::string> names;
        for (const auto &d : descs) names.push_back(dir_ + "/" + (d.metaInfo.empty() ? std::to_string(d.devId) : d.metaInfo));
        return nixl::queryFileInfoList(names, resp);
    }

private:
    std::string dir_;
    std::unique_ptr<nixlThreadPool> pool_;
};

} // namespace

extern "C" NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init() {
    return nixlBackendPluginCreator<ObjEngine>::create(NIXL_PLUGIN_API_VERSION, NIXL_OBJ_PLUGIN_NAME, "1.0.0", {{NIXL_OBJ_BUCKET_PARAM, ""}, {"num_threads", "4"}},
                                                       {DRAM_SEG, OBJ_SEG});
}
extern "C" NIXL_PLUGIN_EXPORT void nixl_plugin_fini() {}

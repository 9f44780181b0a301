// POSIX backend: moves data between registered DRAM and files.
//
// Behavioural parity with the reference's src/plugins/posix/posix_backend.cpp: local-only
// (the "remote" agent of a transfer is the agent itself), initiator side DRAM, target side
// FILE (:37-66); FILE descriptors are {addr = file offset, len, devId = fd}, or path mode
// where metaInfo names the file and devId is a caller-chosen unique id (:228); one I/O per
// descriptor (:170-201); queue chosen by the use_aio / use_uring / use_posix_aio parameters
// (:82); queryMem stats files (:348).
//
// Also built as libplugin_HF3FS.so (NIXL_POSIX_PLUGIN_NAME): the reference's HF3FS plugin
// (src/plugins/hf3fs) has the same contract (local, DRAM + FILE, fd in devId) over the 3FS
// user-space I/O rings, for which this build has no client; under that name (an opt-in stand-in,
// outside the default plug-in path) the files are served with the queues of this engine.
#ifndef NIXL_POSIX_PLUGIN_NAME
#define NIXL_POSIX_PLUGIN_NAME "POSIX"
#endif
#include <atomic>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "backend/backend_plugin.h"
#include "plugins/posix/io_queue.h"
#include "utils/file/file_utils.h"
#include "utils/log.h"

namespace nixl_posix {
namespace {

class FileMD final : public nixlBackendMD {
public:
    FileMD(uint64_t dev_id, const std::string &meta) : nixlBackendMD(true), devId(dev_id), file(static_cast<int>(dev_id), meta) {}
    uint64_t devId;
    nixl::FileFd file;
};

class Req final : public nixlBackendReqH {
public:
    std::vector<IoOp> ops;
    IoBatchState state;
    bool posted = false;
};

bool flag(const nixl_b_params_t &p, const char *k) {
    auto it = p.find(k);
    return it != p.end() && (it->second == "true" || it->second == "1" || it->second == "yes");
}

unsigned num(const nixl_b_params_t &p, const char *k, unsigned dflt) {
    auto it = p.find(k);
    if (it == p.end() || it->second.empty()) return dflt;
    const long v = std::strtol(it->second.c_str(), nullptr, 10);
    return v > 0 ? static_cast<unsigned>(v) : dflt;
}

class Engine final : public nixlBackendEngine {
public:
    explicit Engine(const nixlBackendInitParams *init) : nixlBackendEngine(init) {
        if (std::strcmp(NIXL_POSIX_PLUGIN_NAME, "POSIX") != 0)
            NIXL_WARN << NIXL_POSIX_PLUGIN_NAME << " backend: this build has no client for that file system; files are served by the POSIX engine's queues";
        const nixl_b_params_t &p = getCustomParams();
        QueueKind kind = QueueKind::THREADS;
        if (flag(p, "use_aio")) kind = QueueKind::LINUX_AIO;
        else if (flag(p, "use_uring")) kind = QueueKind::IO_URING;
        else if (flag(p, "use_posix_aio")) kind = QueueKind::POSIX_AIO;
        // `iopool_size` is the name the reference's HF3FS plugin gives its pool (src/plugins/hf3fs).
        queue_ = makeQueue(kind, num(p, "ios_pool_size", num(p, "iopool_size", 8)), num(p, "kernel_queue_size", 256));
        NIXL_INFO << "POSIX backend: I/O queue " << queue_->name();
    }

    bool supportsRemote() const override { return false; }
    bool supportsLocal() const override { return true; }
    bool supportsNotif() const override { return false; }
    nixl_mem_list_t getSupportedMems() const override { return {DRAM_SEG, FILE_SEG}; }

    nixl_status_t registerMem(const nixlBlobDesc &mem, const nixl_mem_t &nixl_mem, nixlBackendMD *&out) override {
        out = nullptr;
        if (nixl_mem == DRAM_SEG) return NIXL_SUCCESS; // nothing to pin for buffered I/O
        if (nixl_mem != FILE_SEG) return NIXL_ERR_NOT_SUPPORTED;
        const bool path_mode = nixl::parsePathMeta(mem.metaInfo).has_value();
        std::lock_guard<std::mutex> g(mu_);
        if (path_mode && pathIds_.count(mem.devId)) {
            NIXL_ERROR << "POSIX backend: path mode needs a unique devId per file (" << mem.devId << " is taken)";
            return NIXL_ERR_INVALID_PARAM;
        }
        try {
            out = new FileMD(mem.devId, mem.metaInfo);
        } catch (const std::exception &e) {
            NIXL_ERROR << "POSIX backend: " << e.what();
            return NIXL_ERR_BACKEND;
        }
        if (path_mode) pathIds_[mem.devId] = 1;
        return NIXL_SUCCESS;
    }

    nixl_status_t deregisterMem(nixlBackendMD *meta) override {
        if (auto *f = dynamic_cast<FileMD *>(meta)) {
            if (f->file.owned()) {
                std::lock_guard<std::mutex> g(mu_);
                pathIds_.erase(f->devId);
            }
        }
        delete meta;
        return NIXL_SUCCESS;
    }

    nixl_status_t connect(const std::string &) override { return NIXL_SUCCESS; }
    nixl_status_t disconnect(const std::string &) override { return NIXL_SUCCESS; }
    nixl_status_t unloadMD(nixlBackendMD *) override { return NIXL_SUCCESS; }
    nixl_status_t loadLocalMD(nixlBackendMD *input, nixlBackendMD *&output) override {
        output = input; // same object: the agent's loopback view borrows the registration
        return NIXL_SUCCESS;
    }

    nixl_status_t prepXfer(const nixl_xfer_op_t &op, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote,
                           const std::string &remote_agent, nixlBackendReqH *&handle, const nixl_opt_b_args_t *) const override {
        if (remote_agent != localAgent) {
            NIXL_ERROR << "POSIX backend: transfers are local (remote agent must be '" << localAgent << "')";
            return NIXL_ERR_INVALID_PARAM;
        }
        if (local.getType() != DRAM_SEG || remote.getType() != FILE_SEG) {
            NIXL_ERROR << "POSIX backend: expected local DRAM and remote FILE descriptor lists";
            return NIXL_ERR_INVALID_PARAM;
        }
        if (local.descCount() != remote.descCount() || local.isEmpty()) return NIXL_ERR_INVALID_PARAM;
        auto req = std::make_unique<Req>();
        req->ops.reserve(local.descCount());
        for (int i = 0; i < local.descCount(); ++i) {
            if (local[i].len != remote[i].len) return NIXL_ERR_INVALID_PARAM;
            auto *f = dynamic_cast<FileMD *>(remote[i].metadataP);
            if (!f || f->file.fd() < 0) return NIXL_ERR_INVALID_PARAM;
            req->ops.push_back({f->file.fd(), reinterpret_cast<void *>(local[i].addr), local[i].len,
                                static_cast<off_t>(remote[i].addr), op == NIXL_READ});
        }
        handle = req.release();
        return NIXL_SUCCESS;
    }

    nixl_status_t postXfer(const nixl_xfer_op_t &, const nixl_meta_dlist_t &, const nixl_meta_dlist_t &, const std::string &,
                           nixlBackendReqH *&handle, const nixl_opt_b_args_t *) const override {
        auto *req = dynamic_cast<Req *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        std::lock_guard<std::mutex> g(qmu_);
        req->state.error = 0;
        req->state.remaining = req->ops.size();
        req->posted = true;
        for (const auto &op : req->ops) queue_->enqueue(op, &req->state);
        if (queue_->submit() != NIXL_SUCCESS) return NIXL_ERR_BACKEND;
        return status(req);
    }

    nixl_status_t checkXfer(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<Req *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        if (!req->posted) return NIXL_ERR_NOT_POSTED;
        std::lock_guard<std::mutex> g(qmu_);
        queue_->poll();
        return status(req);
    }

    nixl_status_t releaseReqH(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<Req *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        // Queued I/O refers to the request's state: let it drain first.
        while (req->posted && req->state.remaining.load(std::memory_order_acquire) != 0) {
            std::lock_guard<std::mutex> g(qmu_);
            queue_->poll();
        }
        delete req;
        return NIXL_SUCCESS;
    }

    nixl_status_t queryMem(const nixl_reg_dlist_t &descs, std::vector<nixl_query_resp_t> &resp) const override {
        std::vector<std::string> names;
        for (const auto &d : descs) names.push_back(d.metaInfo);
        return nixl::queryFileInfoList(names, resp);
    }

private:
    nixl_status_t status(Req *req) const {
        if (req->state.remaining.load(std::memory_order_acquire) != 0) return NIXL_IN_PROG;
        if (const int e = req->state.error.load()) {
            NIXL_ERROR << "POSIX backend: I/O failed: " << std::strerror(e);
            return NIXL_ERR_BACKEND;
        }
        return NIXL_SUCCESS;
    }

    std::mutex mu_;
    std::unordered_map<uint64_t, int> pathIds_;
    mutable std::mutex qmu_;
    std::unique_ptr<IoQueue> queue_;
};

nixl_b_params_t defaults() {
    return {{"use_aio", "false"}, {"use_uring", "false"}, {"use_posix_aio", "false"}, {"ios_pool_size", "8"}, {"kernel_queue_size", "256"}};
}

} // namespace
} // namespace nixl_posix

extern "C" NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init() {
    return nixlBackendPluginCreator<nixl_posix::Engine>::create(NIXL_PLUGIN_API_VERSION, NIXL_POSIX_PLUGIN_NAME, "1.0.0", nixl_posix::defaults(),
                                                                {DRAM_SEG, FILE_SEG});
}

extern "C" NIXL_PLUGIN_EXPORT void nixl_plugin_fini() {}

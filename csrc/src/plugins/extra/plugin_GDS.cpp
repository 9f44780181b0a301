// GDS backend: files <-> GPU memory (and host memory) under the backend name the reference uses
// for its cuFile plugins (src/plugins/cuda_gds, src/plugins/gds_mt: local-only, DRAM / VRAM /
// FILE, one I/O per descriptor, `thread_count` workers).
//
// GPUDirect Storage needs the nvidia-fs kernel driver and a supported file system; without
// them cuFile runs in its compatibility mode, i.e. a pinned bounce buffer plus cudaMemcpy.
// This engine is exactly that path, written out (it never calls cuFile): each worker
// streams a descriptor through two pinned staging buffers so the file I/O of chunk i+1
// overlaps the PCIe copy of chunk i.  Host memory goes through pread/pwrite directly.
#ifndef NIXL_GDS_PLUGIN_NAME
#define NIXL_GDS_PLUGIN_NAME "GDS"
#endif
#include <cerrno>
#include <cstring>
#include <unistd.h>

#include <atomic>
#include <memory>
#include <mutex>

#include <cuda_runtime.h>

#include "backend/backend_plugin.h"
#include "utils/file/file_utils.h"
#include "utils/log.h"
#include "utils/thread_pool.h"

namespace {

constexpr size_t kChunk = size_t(8) << 20;

class GdsFileMD final : public nixlBackendMD {
public:
    GdsFileMD(uint64_t dev, const std::string &meta) : nixlBackendMD(true), file(static_cast<int>(dev), meta) {}
    nixl::FileFd file;
};

class GdsMemMD final : public nixlBackendMD {
public:
    GdsMemMD() : nixlBackendMD(true) {}
    bool vram = false;
    int device = 0;
};

struct Io {
    int fd;
    off_t offset;
    char *mem;
    size_t len;
    bool vram;
    int device;
    bool to_file; // WRITE: memory -> file
};

class GdsReq final : public nixlBackendReqH {
public:
    std::vector<Io> ios;
    std::atomic<size_t> remaining{0};
    std::atomic<int> error{0};
    bool posted = false;
};

int fullIo(int fd, char *p, size_t n, off_t off, bool write) {
    while (n) {
        const ssize_t r = write ? ::pwrite(fd, p, n, off) : ::pread(fd, p, n, off);
        if (r < 0) {
            if (errno == EINTR) continue;
            return errno;
        }
        if (r == 0) return EIO;
        p += r;
        off += r;
        n -= static_cast<size_t>(r);
    }
    return 0;
}

// One descriptor between a file and GPU memory through two pinned staging buffers.
int stagedIo(const Io &io) {
    if (cudaSetDevice(io.device) != cudaSuccess) return EIO;
    char *stage[2] = {nullptr, nullptr};
    cudaStream_t s = nullptr;
    cudaEvent_t ev[2] = {nullptr, nullptr};
    int err = 0;
    if (cudaHostAlloc(reinterpret_cast<void **>(&stage[0]), kChunk, cudaHostAllocDefault) != cudaSuccess ||
        cudaHostAlloc(reinterpret_cast<void **>(&stage[1]), kChunk, cudaHostAllocDefault) != cudaSuccess ||
        cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess || cudaEventCreate(&ev[0]) != cudaSuccess ||
        cudaEventCreate(&ev[1]) != cudaSuccess)
        err = ENOMEM;
    size_t done = 0;
    int slot = 0;
    bool used[2] = {false, false};
    while (!err && done < io.len) {
        const size_t n = std::min(kChunk, io.len - done);
        if (used[slot] && cudaEventSynchronize(ev[slot]) != cudaSuccess) err = EIO; // staging buffer free again?
        if (err) break;
        if (io.to_file) {
            if (cudaMemcpyAsync(stage[slot], io.mem + done, n, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)
                err = EIO;
            else err = fullIo(io.fd, stage[slot], n, io.offset + static_cast<off_t>(done), true);
        } else {
            err = fullIo(io.fd, stage[slot], n, io.offset + static_cast<off_t>(done), false);
            if (!err && (cudaMemcpyAsync(io.mem + done, stage[slot], n, cudaMemcpyHostToDevice, s) != cudaSuccess ||
                         cudaEventRecord(ev[slot], s) != cudaSuccess))
                err = EIO;
            used[slot] = true;
        }
        done += n;
        slot ^= 1;
    }
    if (s && cudaStreamSynchronize(s) != cudaSuccess && !err) err = EIO;
    for (int i = 0; i < 2; ++i) {
        if (ev[i]) cudaEventDestroy(ev[i]);
        if (stage[i]) cudaFreeHost(stage[i]);
    }
    if (s) cudaStreamDestroy(s);
    cudaGetLastError();
    return err;
}

class GdsEngine final : public nixlBackendEngine {
public:
    explicit GdsEngine(const nixlBackendInitParams *p) : nixlBackendEngine(p) {
        if (std::strcmp(NIXL_GDS_PLUGIN_NAME, "GDS") != 0)
            NIXL_WARN << NIXL_GDS_PLUGIN_NAME << " backend: served by the staged-copy GDS engine of this build (same worker pool, no cuFile thread pool)";
        std::string v;
        unsigned threads = 4;
        if (getInitParam("thread_count", v) == NIXL_SUCCESS && std::atoi(v.c_str()) > 0) threads = static_cast<unsigned>(std::atoi(v.c_str()));
        pool_ = std::make_unique<nixlThreadPool>(threads);
        int n = 0;
        cuda_ = cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
        if (!cuda_) cudaGetLastError();
    }
    bool supportsRemote() const override { return false; }
    bool supportsLocal() const override { return true; }
    bool supportsNotif() const override { return false; }
    nixl_mem_list_t getSupportedMems() const override { return {DRAM_SEG, VRAM_SEG, FILE_SEG}; }

    nixl_status_t registerMem(const nixlBlobDesc &mem, const nixl_mem_t &nixl_mem, nixlBackendMD *&out) override {
        if (nixl_mem == FILE_SEG) {
            try {
                out = new GdsFileMD(mem.devId, mem.metaInfo);
            } catch (const std::exception &e) {
                NIXL_ERROR << "GDS backend: " << e.what();
                return NIXL_ERR_BACKEND;
            }
            return NIXL_SUCCESS;
        }
        if (nixl_mem == VRAM_SEG && !cuda_) return NIXL_ERR_NOT_SUPPORTED;
        auto *md = new GdsMemMD();
        md->vram = nixl_mem == VRAM_SEG;
        md->device = static_cast<int>(mem.devId);
        out = md;
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
        if (remote_agent != localAgent || remote.getType() != FILE_SEG || local.getType() == FILE_SEG ||
            local.descCount() != remote.descCount())
            return NIXL_ERR_INVALID_PARAM;
        auto req = std::make_unique<GdsReq>();
        for (int i = 0; i < local.descCount(); ++i) {
            auto *f = dynamic_cast<GdsFileMD *>(remote[i].metadataP);
            auto *m = dynamic_cast<GdsMemMD *>(local[i].metadataP);
            if (!f || !m || local[i].len != remote[i].len) return NIXL_ERR_INVALID_PARAM;
            req->ios.push_back({f->file.fd(), static_cast<off_t>(remote[i].addr), reinterpret_cast<char *>(local[i].addr), local[i].len,
                                m->vram, m->device, op == NIXL_WRITE});
        }
        handle = req.release();
        return NIXL_SUCCESS;
    }
    nixl_status_t postXfer(const nixl_xfer_op_t &, const nixl_meta_dlist_t &, const nixl_meta_dlist_t &, const std::string &,
                           nixlBackendReqH *&handle, const nixl_opt_b_args_t *) const override {
        auto *req = dynamic_cast<GdsReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        req->error = 0;
        req->remaining = req->ios.size();
        req->posted = true;
        for (const Io &io : req->ios) {
            pool_->submit([req, io] {
                const int e = io.vram ? stagedIo(io) : fullIo(io.fd, io.mem, io.len, io.offset, io.to_file);
                if (e) {
                    int zero = 0;
                    req->error.compare_exchange_strong(zero, e);
                }
                req->remaining.fetch_sub(1, std::memory_order_acq_rel);
            });
        }
        return checkXfer(handle);
    }
    nixl_status_t checkXfer(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<GdsReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        if (!req->posted) return NIXL_ERR_NOT_POSTED;
        if (req->remaining.load(std::memory_order_acquire)) return NIXL_IN_PROG;
        if (const int e = req->error.load()) {
            NIXL_ERROR << "GDS backend: I/O failed: " << std::strerror(e);
            return NIXL_ERR_BACKEND;
        }
        return NIXL_SUCCESS;
    }
    nixl_status_t releaseReqH(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<GdsReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        while (req->posted && req->remaining.load(std::memory_order_acquire)) std::this_thread::yield();
        delete req;
        return NIXL_SUCCESS;
    }
    nixl_status_t queryMem(const nixl_reg_dlist_t &descs, std::vector<nixl_query_resp_t> &resp) const override {
        std::vector<std::string> names;
        for (const auto &d : descs) names.push_back(d.metaInfo);
        return nixl::queryFileInfoList(names, resp);
    }

private:
    std::unique_ptr<nixlThreadPool> pool_;
    bool cuda_ = false;
};

} // namespace

extern "C" NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init() {
    return nixlBackendPluginCreator<GdsEngine>::create(
        NIXL_PLUGIN_API_VERSION, NIXL_GDS_PLUGIN_NAME, "1.0.0",
        {{"thread_count", "4"}, {"batch_pool_size", "128"}, {"batch_limit", "128"}, {"max_request_size", "16777216"}},
        {DRAM_SEG, VRAM_SEG, FILE_SEG});
}
extern "C" NIXL_PLUGIN_EXPORT void nixl_plugin_fini() {}

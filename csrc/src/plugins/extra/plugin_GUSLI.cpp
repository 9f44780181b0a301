// GUSLI backend: host memory <-> block devices (BLK_SEG).
//
// The reference's GUSLI plugin (src/plugins/gusli: local-only, DRAM + BLK, devId = block device
// id, descriptor address = byte offset on the device, devices listed in a `config_file`
// parameter) hands I/O to a user-space block server through libgusli_clnt.  This build does not
// link that library; the engine implements the library's "direct local access" mode
// itself: every `F` (file-backed) or `K` (kernel block device) line of the configuration is
// opened and served with pread/pwrite from a worker pool.  `N` (networked server) lines are
// refused at creation.  Configuration text, one device per line after the version line:
//     <device_id> <F|K|N> <W|R> <shared Y|N> <path> [sec=...]
// Lines starting with '#' and blank lines are skipped.  Parameters: `config_file` (the text
// itself, as in the reference), `num_threads`, `direct_io` (open with O_DIRECT; callers then
// keep offsets, lengths and buffers aligned to the device's logical block size).
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <memory>
#include <sstream>

#include "backend/backend_plugin.h"
#include "utils/log.h"
#include "utils/thread_pool.h"

namespace {

struct BlockDev {
    int fd = -1;
    bool writable = false;
    uint64_t bytes = 0; // 0: unknown (character devices such as /dev/zero)
    std::string path;
};

class BlkMD final : public nixlBackendMD {
public:
    explicit BlkMD(uint64_t id) : nixlBackendMD(true), dev(id) {}
    uint64_t dev;
};

struct BlkIo {
    int fd;
    off_t offset;
    char *mem;
    size_t len;
    bool write;
};

class BlkReq final : public nixlBackendReqH {
public:
    std::vector<BlkIo> ios;
    std::atomic<size_t> remaining{0};
    std::atomic<int> error{0};
    bool posted = false;
};

int blockIo(const BlkIo &io) {
    char *p = io.mem;
    size_t n = io.len;
    off_t off = io.offset;
    while (n) {
        const ssize_t r = io.write ? ::pwrite(io.fd, p, n, off) : ::pread(io.fd, p, n, off);
        if (r < 0) {
            if (errno == EINTR) continue;
            return errno;
        }
        if (r == 0) return EIO; // past the end of the device
        p += r;
        off += r;
        n -= static_cast<size_t>(r);
    }
    return 0;
}

class GusliEngine final : public nixlBackendEngine {
public:
    explicit GusliEngine(const nixlBackendInitParams *p) : nixlBackendEngine(p) {
        std::string v, cfg;
        unsigned threads = 4;
        if (getInitParam("num_threads", v) == NIXL_SUCCESS && std::atoi(v.c_str()) > 0) threads = static_cast<unsigned>(std::atoi(v.c_str()));
        const bool direct = getInitParam("direct_io", v) == NIXL_SUCCESS && (v == "1" || v == "true" || v == "y");
        if (getInitParam("config_file", cfg) != NIXL_SUCCESS || cfg.empty()) {
            NIXL_ERROR << "GUSLI backend: the config_file parameter (device list) is required";
            initErr = true;
            return;
        }
        if (!parse(cfg, direct)) {
            initErr = true;
            return;
        }
        pool_ = std::make_unique<nixlThreadPool>(threads);
    }
    ~GusliEngine() override {
        pool_.reset(); // drains the workers before the descriptors go away
        for (auto &kv : devs_)
            if (kv.second.fd >= 0) ::close(kv.second.fd);
    }
    bool supportsRemote() const override { return false; }
    bool supportsLocal() const override { return true; }
    bool supportsNotif() const override { return false; }
    nixl_mem_list_t getSupportedMems() const override { return {DRAM_SEG, BLK_SEG}; }

    nixl_status_t registerMem(const nixlBlobDesc &mem, const nixl_mem_t &nixl_mem, nixlBackendMD *&out) override {
        out = nullptr;
        if (nixl_mem == DRAM_SEG) return NIXL_SUCCESS;
        if (nixl_mem != BLK_SEG) return NIXL_ERR_NOT_SUPPORTED;
        const auto it = devs_.find(mem.devId);
        if (it == devs_.end()) {
            NIXL_ERROR << "GUSLI backend: block device " << mem.devId << " is not in the configuration";
            return NIXL_ERR_NOT_FOUND;
        }
        if (it->second.bytes && mem.addr + mem.len > it->second.bytes) {
            NIXL_ERROR << "GUSLI backend: [" << mem.addr << ", +" << mem.len << ") exceeds device " << mem.devId << " (" << it->second.bytes
                       << " bytes)";
            return NIXL_ERR_INVALID_PARAM;
        }
        out = new BlkMD(mem.devId);
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
        if (remote_agent != localAgent || local.getType() != DRAM_SEG || remote.getType() != BLK_SEG || local.descCount() != remote.descCount())
            return NIXL_ERR_INVALID_PARAM;
        auto req = std::make_unique<BlkReq>();
        for (int i = 0; i < local.descCount(); ++i) {
            auto *b = dynamic_cast<BlkMD *>(remote[i].metadataP);
            if (!b || local[i].len != remote[i].len) return NIXL_ERR_INVALID_PARAM;
            const BlockDev &dev = devs_.at(b->dev);
            if (op == NIXL_WRITE && !dev.writable) {
                NIXL_ERROR << "GUSLI backend: device " << b->dev << " is configured read-only";
                return NIXL_ERR_NOT_ALLOWED;
            }
            req->ios.push_back({dev.fd, static_cast<off_t>(remote[i].addr), reinterpret_cast<char *>(local[i].addr), local[i].len, op == NIXL_WRITE});
        }
        handle = req.release();
        return NIXL_SUCCESS;
    }
    nixl_status_t postXfer(const nixl_xfer_op_t &, const nixl_meta_dlist_t &, const nixl_meta_dlist_t &, const std::string &,
                           nixlBackendReqH *&handle, const nixl_opt_b_args_t *) const override {
        auto *req = dynamic_cast<BlkReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        if (req->posted && req->remaining.load(std::memory_order_acquire)) return NIXL_ERR_REPOST_ACTIVE;
        req->error = 0;
        req->remaining = req->ios.size();
        req->posted = true;
        for (const BlkIo &io : req->ios)
            pool_->submit([req, io] {
                if (const int e = blockIo(io)) {
                    int zero = 0;
                    req->error.compare_exchange_strong(zero, e);
                }
                req->remaining.fetch_sub(1, std::memory_order_acq_rel);
            });
        return checkXfer(handle);
    }
    nixl_status_t checkXfer(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<BlkReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        if (!req->posted) return NIXL_ERR_NOT_POSTED;
        if (req->remaining.load(std::memory_order_acquire)) return NIXL_IN_PROG;
        if (const int e = req->error.load()) {
            NIXL_ERROR << "GUSLI backend: block I/O failed: " << std::strerror(e);
            return NIXL_ERR_BACKEND;
        }
        return NIXL_SUCCESS;
    }
    nixl_status_t releaseReqH(nixlBackendReqH *handle) const override {
        auto *req = dynamic_cast<BlkReq *>(handle);
        if (!req) return NIXL_ERR_INVALID_PARAM;
        while (req->posted && req->remaining.load(std::memory_order_acquire)) std::this_thread::yield();
        delete req;
        return NIXL_SUCCESS;
    }
    // Per device: whether it is configured, its size and path.
    nixl_status_t queryMem(const nixl_reg_dlist_t &descs, std::vector<nixl_query_resp_t> &resp) const override {
        resp.clear();
        for (const auto &d : descs) {
            const auto it = devs_.find(d.devId);
            if (it == devs_.end()) {
                resp.emplace_back(std::nullopt);
                continue;
            }
            nixl_b_params_t info;
            info["size"] = std::to_string(it->second.bytes);
            info["path"] = it->second.path;
            info["access"] = it->second.writable ? "W" : "R";
            resp.emplace_back(std::move(info));
        }
        return NIXL_SUCCESS;
    }

private:
    bool parse(const std::string &cfg, bool direct) {
        std::istringstream in(cfg);
        std::string line;
        bool versioned = false;
        while (std::getline(in, line)) {
            const size_t first = line.find_first_not_of(" \t\r");
            if (first == std::string::npos || line[first] == '#') continue;
            if (line.compare(first, 8, "version=") == 0) {
                if (std::atoi(line.c_str() + first + 8) != 1) {
                    NIXL_ERROR << "GUSLI backend: unsupported configuration version in '" << line << "'";
                    return false;
                }
                versioned = true;
                continue;
            }
            std::istringstream f(line);
            uint64_t id;
            std::string type, access, shared, path;
            if (!(f >> id >> type >> access >> shared >> path) || type.size() != 1 || access.size() != 1) {
                NIXL_ERROR << "GUSLI backend: cannot parse device line '" << line << "'";
                return false;
            }
            if (type == "N") {
                NIXL_ERROR << "GUSLI backend: networked block servers are not available (device " << id << ")";
                return false;
            }
            if ((type != "F" && type != "K") || (access != "W" && access != "R") || devs_.count(id)) {
                NIXL_ERROR << "GUSLI backend: bad or repeated device line '" << line << "'";
                return false;
            }
            BlockDev dev;
            dev.writable = access == "W";
            dev.path = path;
            int flags = dev.writable ? O_RDWR : O_RDONLY;
            if (type == "F" && dev.writable) flags |= O_CREAT;
            if (direct) flags |= O_DIRECT;
            if (shared == "N" && type == "K") flags |= O_EXCL; // exclusive use of a kernel block device
            dev.fd = ::open(path.c_str(), flags, 0644);
            if (dev.fd < 0 && (flags & O_EXCL)) dev.fd = ::open(path.c_str(), flags & ~O_EXCL, 0644); // character devices refuse O_EXCL
            if (dev.fd < 0) {
                NIXL_ERROR << "GUSLI backend: cannot open " << path << ": " << std::strerror(errno);
                return false;
            }
            struct stat st;
            if (::fstat(dev.fd, &st) == 0) {
                if (S_ISREG(st.st_mode)) dev.bytes = static_cast<uint64_t>(st.st_size);
                else if (S_ISBLK(st.st_mode)) {
                    const off_t end = ::lseek(dev.fd, 0, SEEK_END);
                    if (end > 0) dev.bytes = static_cast<uint64_t>(end);
                }
            }
            // A file that is still empty grows on demand: no size check for it.
            if (type == "F" && dev.writable) dev.bytes = 0;
            devs_.emplace(id, std::move(dev));
        }
        if (!versioned) NIXL_WARN << "GUSLI backend: configuration has no version line; assuming version 1";
        if (devs_.empty()) {
            NIXL_ERROR << "GUSLI backend: the configuration lists no device";
            return false;
        }
        return true;
    }

    std::map<uint64_t, BlockDev> devs_;
    std::unique_ptr<nixlThreadPool> pool_;
};

} // namespace

extern "C" NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init() {
    return nixlBackendPluginCreator<GusliEngine>::create(NIXL_PLUGIN_API_VERSION, "GUSLI", "1.0.0",
                                                         {{"config_file", ""}, {"num_threads", "4"}, {"direct_io", "false"}}, {DRAM_SEG, BLK_SEG});
}
extern "C" NIXL_PLUGIN_EXPORT void nixl_plugin_fini() {}

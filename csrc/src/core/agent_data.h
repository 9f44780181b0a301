// Private state of an agent and the opaque handle types of the public API.
// Role parity: the reference's src/core/agent_data.h and src/core/transfer_request.h.
#ifndef NIXL_B200_AGENT_DATA_H
#define NIXL_B200_AGENT_DATA_H

#include <array>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/md_manager.h"
#include "core/plugin_manager.h"
#include "core/sync.h"
#include "core/telemetry/telemetry.h"
#include "core/tracing/trace.h"
#include "infra/sections.h"
#include "nixl.h"

// User-visible backend handle: the engine plus the plugin that must outlive it.
class nixlBackendH {
public:
    nixlBackendH(nixlBackendEngine *e, std::shared_ptr<const nixlPluginHandle> p) : engine(e), plugin(std::move(p)) {}
    ~nixlBackendH() {
        if (engine && plugin) plugin->destroyEngine(engine);
    }
    nixlBackendEngine *engine;
    std::shared_ptr<const nixlPluginHandle> plugin;
    const nixl_backend_t &getType() const { return engine->getType(); }
};

// A transfer request: resolved descriptor lists, the backend's request state and status.
class nixlXferReqH {
public:
    nixlBackendEngine *engine = nullptr;
    nixlBackendReqH *backendHandle = nullptr;
    std::unique_ptr<nixl_meta_dlist_t> initiatorDescs;
    std::unique_ptr<nixl_meta_dlist_t> targetDescs;
    std::string remoteAgent;
    uint64_t remoteGeneration = 0;
    nixl_blob_t notifMsg;
    bool hasNotif = false;
    nixl_xfer_op_t backendOp = NIXL_WRITE;
    nixl_status_t status = NIXL_ERR_NOT_POSTED;
    nixl_xfer_telem_t telemetry;
    chrono_point_t postEnd;
    uint64_t correlation = 0;

    ~nixlXferReqH() {
        if (backendHandle && engine) engine->releaseReqH(backendHandle);
    }
};

// One side of a prepared transfer: the same descriptors resolved (run-length compressed)
// for every backend that can serve them.
class nixlDlistH {
public:
    std::unordered_map<nixlBackendEngine *, std::unique_ptr<nixl_stride_dlist_t>> descs;
    std::string remoteAgent; // empty: local side
    bool isLocal = false;
    uint64_t generation = 0;
    nixl_mem_t memType = DRAM_SEG;
    size_t count = 0;
};

class nixlAgentData : public nixlMetadataContext {
public:
    nixlAgentData(const std::string &name, const nixlAgentConfig &cfg);
    ~nixlAgentData() override;

    // nixlMetadataContext
    const std::string &mdAgentName() const override { return name; }
    nixl_status_t mdGetLocal(nixl_blob_t &out) const override;
    nixl_status_t mdGetLocalPartial(const nixl_reg_dlist_t &descs, nixl_blob_t &out, const nixl_opt_args_t *opt) const override;
    nixl_status_t mdLoadRemote(const nixl_blob_t &blob, std::string &agent) override;
    nixl_status_t mdInvalidateRemote(const std::string &agent) override;

    // helpers used by nixlAgent methods (all expect the lock to be held)
    nixlRemoteSection *remoteOf(const std::string &agent) const;
    nixlRemoteSection &selfSection();
    bool hasBackend(const nixlBackendEngine *e) const;
    void noteError(nixl_status_t st) const {
        if (telemetry && st < 0) telemetry->updateErrorCount(st);
    }
    void dropRemote(const std::string &agent);
    void finishStats(nixlXferReqH *req) const;

    std::string name;
    nixlAgentConfig config;
    mutable nixlLock lock;

    std::unordered_map<nixl_backend_t, std::unique_ptr<nixlBackendH>> backends; // by type
    std::vector<nixlBackendEngine *> creationOrder;
    std::array<backend_set_t, FILE_SEG + 1> memToBackend;
    backend_set_t notifEngines;
    std::unordered_map<nixl_backend_t, nixl_blob_t> connMd; // our own connection info per remote-capable backend

    nixlLocalSection localSection;
    std::unordered_map<std::string, std::unique_ptr<nixlRemoteSection>> remoteSections;
    // connection blobs already loaded per remote agent (backend type -> blob)
    std::unordered_map<std::string, std::unordered_map<nixl_backend_t, nixl_blob_t>> remoteBackends;

    std::unique_ptr<nixlTelemetry> telemetry;
    nixl::trace::Tracer tracer;
    std::unique_ptr<nixlMetadataManager> mdManager;
};

#endif

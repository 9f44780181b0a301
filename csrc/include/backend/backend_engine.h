// South-bound engine interface: what a transfer backend implements.
//
// Parity: the virtual set and their signatures follow the reference's
// src/api/cpp/backend/backend_engine.h:105-239, so an engine written for the
// reference builds against this header.  Every call documents its contract here.
#ifndef NIXL_B200_BACKEND_ENGINE_H
#define NIXL_B200_BACKEND_ENGINE_H

#include <chrono>
#include <mutex>
#include <string>
#include <vector>
#include "backend/backend_aux.h"
#include "telemetry/telemetry_event.h"

constexpr size_t MAX_TELEMETRY_QUEUE_SIZE = 1000;

class nixlBackendEngine {
private:
    nixl_backend_t backendType;
    nixl_b_params_t customParams;
    std::vector<nixlTelemetryEvent> telemetryEvents_;
    std::mutex telemetryEventsMutex_;

protected:
    bool initErr = false;
    const std::string localAgent;
    const bool enableTelemetry_;

    nixl_status_t setInitParam(const std::string &key, const std::string &value) {
        return customParams.emplace(key, value).second ? NIXL_SUCCESS : NIXL_ERR_NOT_ALLOWED;
    }
    nixl_status_t getInitParam(const std::string &key, std::string &value) const {
        auto it = customParams.find(key);
        if (it == customParams.end()) return NIXL_ERR_INVALID_PARAM;
        value = it->second;
        return NIXL_SUCCESS;
    }
    // Queue a backend-side telemetry event (bounded; overflow is dropped).
    void addTelemetryEvent(nixl_telemetry_event_type_t type, uint64_t value) {
        if (!enableTelemetry_) return;
        std::lock_guard<std::mutex> g(telemetryEventsMutex_);
        if (telemetryEvents_.size() < MAX_TELEMETRY_QUEUE_SIZE) telemetryEvents_.emplace_back(type, value);
    }

public:
    explicit nixlBackendEngine(const nixlBackendInitParams *p)
        : backendType(p->type), customParams(p->customParams ? *p->customParams : nixl_b_params_t()),
          localAgent(p->localAgent), enableTelemetry_(p->enableTelemetry_) {}
    nixlBackendEngine(const nixlBackendEngine &) = delete;
    nixlBackendEngine &operator=(const nixlBackendEngine &) = delete;
    virtual ~nixlBackendEngine() = default;

    std::vector<nixlTelemetryEvent> getTelemetryEvents() {
        std::lock_guard<std::mutex> g(telemetryEventsMutex_);
        return std::move(telemetryEvents_);
    }
    bool getInitErr() const noexcept { return initErr; }
    const nixl_backend_t &getType() const noexcept { return backendType; }
    const nixl_b_params_t &getCustomParams() const noexcept { return customParams; }

    // ---- capabilities ----
    virtual bool supportsRemote() const = 0; // can reach another agent
    virtual bool supportsLocal() const = 0;  // can move data within this agent
    virtual bool supportsNotif() const = 0;  // can deliver notifications
    virtual nixl_mem_list_t getSupportedMems() const = 0;

    // ---- registration ----
    virtual nixl_status_t registerMem(const nixlBlobDesc &mem, const nixl_mem_t &nixl_mem, nixlBackendMD *&out) = 0;
    virtual nixl_status_t deregisterMem(nixlBackendMD *meta) = 0;

    // ---- connections ----
    virtual nixl_status_t connect(const std::string &remote_agent) = 0;
    virtual nixl_status_t disconnect(const std::string &remote_agent) = 0;
    // Release metadata produced by loadRemoteMD / loadLocalMD.
    virtual nixl_status_t unloadMD(nixlBackendMD *input) = 0;

    // ---- transfers ----
    // prepXfer allocates `handle`; postXfer may be called repeatedly on it once the
    // previous post has completed.  postXfer/checkXfer return NIXL_SUCCESS when done,
    // NIXL_IN_PROG while running, negative on error.
    virtual nixl_status_t prepXfer(const nixl_xfer_op_t &operation, const nixl_meta_dlist_t &local,
                                   const nixl_meta_dlist_t &remote, const std::string &remote_agent,
                                   nixlBackendReqH *&handle, const nixl_opt_b_args_t *opt_args = nullptr) const = 0;
    virtual nixl_status_t postXfer(const nixl_xfer_op_t &operation, const nixl_meta_dlist_t &local,
                                   const nixl_meta_dlist_t &remote, const std::string &remote_agent,
                                   nixlBackendReqH *&handle, const nixl_opt_b_args_t *opt_args = nullptr) const = 0;
    virtual nixl_status_t checkXfer(nixlBackendReqH *handle) const = 0;
    virtual nixl_status_t releaseReqH(nixlBackendReqH *handle) const = 0;

    // ---- device-side memory views (GPU-initiated transfers) ----
    virtual nixl_status_t prepMemView(const nixl_remote_meta_dlist_t &, nixlMemViewH &, const nixl_opt_b_args_t * = nullptr) const {
        return NIXL_ERR_NOT_SUPPORTED;
    }
    virtual nixl_status_t prepMemView(const nixl_meta_dlist_t &, nixlMemViewH &, const nixl_opt_b_args_t * = nullptr) const {
        return NIXL_ERR_NOT_SUPPORTED;
    }
    virtual void releaseMemView(nixlMemViewH) const {}

    // ---- metadata ----
    // Bytes a remote peer needs to reach this registration (IPC handle etc.).
    virtual nixl_status_t getPublicData(const nixlBackendMD *, std::string &) const { return NIXL_ERR_BACKEND; }
    virtual nixl_status_t getConnInfo(std::string &) const { return NIXL_ERR_BACKEND; }
    virtual nixl_status_t loadRemoteConnInfo(const std::string &, const std::string &) { return NIXL_ERR_BACKEND; }
    virtual nixl_status_t loadRemoteMD(const nixlBlobDesc &, const nixl_mem_t &, const std::string &, nixlBackendMD *&) {
        return NIXL_ERR_BACKEND;
    }
    // Turn a local registration into "remote" metadata for same-agent transfers.
    virtual nixl_status_t loadLocalMD(nixlBackendMD *, nixlBackendMD *&) { return NIXL_ERR_BACKEND; }

    // ---- notifications ----
    virtual nixl_status_t getNotifs(notif_list_t &) { return NIXL_ERR_BACKEND; }
    virtual nixl_status_t genNotif(const std::string &, const std::string &) const { return NIXL_ERR_BACKEND; }

    // ---- queries ----
    virtual nixl_status_t queryMem(const nixl_reg_dlist_t &, std::vector<nixl_query_resp_t> &) const { return NIXL_ERR_NOT_SUPPORTED; }
    virtual nixl_status_t estimateXferCost(const nixl_xfer_op_t &, const nixl_meta_dlist_t &, const nixl_meta_dlist_t &,
                                           const std::string &, nixlBackendReqH *const &, std::chrono::microseconds &,
                                           std::chrono::microseconds &, nixl_cost_t &, const nixl_opt_args_t * = nullptr) const {
        return NIXL_ERR_NOT_SUPPORTED;
    }
};

#endif

// The north-bound API: one nixlAgent per endpoint (typically per GPU worker).
//
// Typical flow:
//   createBackend -> registerMem -> exchange metadata (getLocalMD/loadRemoteMD, or the
//   sendLocalMD/fetchRemoteMD helpers) -> createXferReq (or prepXferDlist + makeXferReq)
//   -> postXferReq -> getXferStatus until NIXL_SUCCESS -> getNotifs on the target.
//
// API parity: method names, argument order and status conventions follow the
// reference's src/api/cpp/nixl.h:34-563.  Implementation: src/core/agent.cpp.
#ifndef NIXL_B200_NIXL_H
#define NIXL_B200_NIXL_H

#include <chrono>
#include <memory>
#include <string>
#include <vector>

#include "nixl_descriptors.h"
#include "nixl_params.h"
#include "nixl_types.h"

class nixlAgentData;

class nixlAgent {
public:
    nixlAgent(const std::string &name, const nixlAgentConfig &cfg);
    ~nixlAgent();
    nixlAgent(const nixlAgent &) = delete;
    nixlAgent &operator=(const nixlAgent &) = delete;

    // ---- plugins and backends ----
    // Names of every backend plugin that can be instantiated (dynamic + static).
    nixl_status_t getAvailPlugins(std::vector<nixl_backend_t> &plugins);
    // Default parameters and supported memory types of a plugin, without creating it.
    nixl_status_t getPluginParams(const nixl_backend_t &type, nixl_mem_list_t &mems, nixl_b_params_t &params) const;
    // Effective parameters of an instantiated backend.
    nixl_status_t getBackendParams(const nixlBackendH *backend, nixl_mem_list_t &mems, nixl_b_params_t &params) const;
    // Instantiate a backend.  The order of creation is the preference order used when
    // several backends can serve a transfer.
    nixl_status_t createBackend(const nixl_backend_t &type, const nixl_b_params_t &params, nixlBackendH *&backend);

    // ---- memory ----
    // Register with every backend that supports the list's memory type (or only
    // extra_params->backends).  Succeeds if at least one backend accepted every descriptor.
    nixl_status_t registerMem(const nixl_reg_dlist_t &descs, const nixl_opt_args_t *extra_params = nullptr);
    nixl_status_t deregisterMem(const nixl_reg_dlist_t &descs, const nixl_opt_args_t *extra_params = nullptr);
    // Ask backends about objects that are not registered yet (e.g. does this file exist, its size).
    nixl_status_t queryMem(const nixl_reg_dlist_t &descs, std::vector<nixl_query_resp_t> &resp,
                           const nixl_opt_args_t *extra_params = nullptr) const;

    // Eagerly connect to a remote whose metadata is loaded (otherwise done at first transfer).
    nixl_status_t makeConnection(const std::string &remote_agent, const nixl_opt_args_t *extra_params = nullptr);

    // ---- transfers ----
    // Resolve a descriptor list once so many requests can be cut from it by index.
    // agent_name == NIXL_INIT_AGENT prepares the local (initiator) side.
    nixl_status_t prepXferDlist(const std::string &agent_name, const nixl_xfer_dlist_t &descs, nixlDlistH *&dlist_hndl,
                                const nixl_opt_args_t *extra_params = nullptr) const;
    nixl_status_t prepXferDlist(const nixl_xfer_dlist_t &descs, nixlDlistH *&dlist_hndl,
                                const nixl_opt_args_t *extra_params = nullptr) const;
    // Build a request from index lists into two prepared sides.  Runs of consecutive
    // indices that are contiguous in memory on both sides are merged unless skipDescMerge.
    nixl_status_t makeXferReq(const nixl_xfer_op_t &operation, const nixlDlistH *local_side,
                              const std::vector<int> &local_indices, const nixlDlistH *remote_side,
                              const std::vector<int> &remote_indices, nixlXferReqH *&req_hndl,
                              const nixl_opt_args_t *extra_params = nullptr) const;
    // One-shot form: resolve both lists and build the request.
    nixl_status_t createXferReq(const nixl_xfer_op_t &operation, const nixl_xfer_dlist_t &local_descs,
                                const nixl_xfer_dlist_t &remote_descs, const std::string &remote_agent,
                                nixlXferReqH *&req_hndl, const nixl_opt_args_t *extra_params = nullptr) const;
    nixl_status_t estimateXferCost(const nixlXferReqH *req_hndl, std::chrono::microseconds &duration,
                                   std::chrono::microseconds &err_margin, nixl_cost_t &method,
                                   const nixl_opt_args_t *extra_params = nullptr) const;
    // Start (or restart) a transfer.  NIXL_SUCCESS = already complete, NIXL_IN_PROG = poll
    // with getXferStatus.  Posting a request that is still running fails with
    // NIXL_ERR_REPOST_ACTIVE.
    nixl_status_t postXferReq(nixlXferReqH *req_hndl, const nixl_opt_args_t *extra_params = nullptr) const;
    nixl_status_t getXferStatus(nixlXferReqH *req_hndl) const;
    nixl_status_t getXferTelemetry(const nixlXferReqH *req_hndl, nixl_xfer_telem_t &telemetry) const;
    nixl_status_t queryXferBackend(const nixlXferReqH *req_hndl, nixlBackendH *&backend) const;
    nixl_status_t releaseXferReq(nixlXferReqH *req_hndl) const;
    nixl_status_t releasedDlistH(nixlDlistH *dlist_hndl) const;

    // ---- device-side memory views (see device/nixl_device.cuh) ----
    nixl_status_t prepMemView(const nixl_remote_dlist_t &dlist, nixlMemViewH &mvh,
                              const nixl_opt_args_t *extra_params = nullptr) const;
    nixl_status_t prepMemView(const nixl_local_dlist_t &dlist, nixlMemViewH &mvh,
                              const nixl_opt_args_t *extra_params = nullptr) const;
    void releaseMemView(nixlMemViewH mvh) const;

    // ---- notifications ----
    // Appends new notifications to notif_map (agent name -> messages).
    nixl_status_t getNotifs(nixl_notifs_t &notif_map, const nixl_opt_args_t *extra_params = nullptr);
    nixl_status_t genNotif(const std::string &remote_agent, const nixl_blob_t &msg,
                           const nixl_opt_args_t *extra_params = nullptr) const;

    // ---- metadata ----
    nixl_status_t getLocalMD(nixl_blob_t &str) const;
    nixl_status_t getLocalPartialMD(const nixl_reg_dlist_t &descs, nixl_blob_t &str,
                                    const nixl_opt_args_t *extra_params = nullptr) const;
    nixl_status_t loadRemoteMD(const nixl_blob_t &remote_metadata, std::string &agent_name);
    nixl_status_t invalidateRemoteMD(const std::string &remote_agent);
    // Push/pull metadata through the peer-to-peer socket (ipAddr/port given) or the
    // configured central store (etcd / TCPStore chosen by environment).
    nixl_status_t sendLocalMD(const nixl_opt_args_t *extra_params = nullptr) const;
    nixl_status_t sendLocalPartialMD(const nixl_reg_dlist_t &descs, const nixl_opt_args_t *extra_params = nullptr) const;
    nixl_status_t fetchRemoteMD(const std::string remote_name, const nixl_opt_args_t *extra_params = nullptr);
    nixl_status_t invalidateLocalMD(const nixl_opt_args_t *extra_params = nullptr) const;
    // NIXL_SUCCESS if metadata of remote_name is loaded and covers `descs` (empty list: agent only).
    nixl_status_t checkRemoteMD(const std::string remote_name, const nixl_xfer_dlist_t &descs) const;

private:
    std::unique_ptr<nixlAgentData> data;
};

#endif

// Metadata exchange: how an agent's serialized metadata reaches its peers when the
// application does not carry the blob itself.
//
// Three transports, selected like the reference's src/core/nixl_md_manager.cpp:47-62,:112:
//   * peer-to-peer TCP (calls that pass ipAddr/port; needs the listener thread on the
//     receiving side), protocol in md_p2p.cpp;
//   * a torch c10d TCPStore when NIXL_TCPSTORE_ENDPOINT=host:port is set;
//   * etcd when NIXL_ETCD_ENDPOINTS is set, through etcd's JSON gateway (md_etcd.cpp); when no
//     gateway answers there, central metadata calls report NIXL_ERR_NOT_SUPPORTED.
// Work is queued to one worker thread so sendLocalMD/fetchRemoteMD return immediately;
// callers poll checkRemoteMD.  Without any thread the work runs inline.
#ifndef NIXL_B200_MD_MANAGER_H
#define NIXL_B200_MD_MANAGER_H

#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>

#include "nixl_descriptors.h"
#include "nixl_params.h"
#include "nixl_types.h"

// What the exchange layer needs from the agent.
class nixlMetadataContext {
public:
    virtual ~nixlMetadataContext() = default;
    virtual const std::string &mdAgentName() const = 0;
    virtual nixl_status_t mdGetLocal(nixl_blob_t &out) const = 0;
    virtual nixl_status_t mdGetLocalPartial(const nixl_reg_dlist_t &descs, nixl_blob_t &out, const nixl_opt_args_t *opt) const = 0;
    virtual nixl_status_t mdLoadRemote(const nixl_blob_t &blob, std::string &agent) = 0;
    virtual nixl_status_t mdInvalidateRemote(const std::string &agent) = 0;
};

// Transport interface for central stores.
class nixlMetadataBackend {
public:
    virtual ~nixlMetadataBackend() = default;
    virtual nixl_status_t publish(const std::string &agent, const std::string &label, const nixl_blob_t &blob) = 0;
    virtual nixl_status_t fetch(const std::string &agent, const std::string &label, nixl_blob_t &blob) = 0;
    virtual nixl_status_t remove(const std::string &agent) = 0;
};

// One queue, one thread.  submit() runs the task inline when the thread is not started.
class nixlMetadataWorker {
public:
    ~nixlMetadataWorker() { stop(); }
    void start();
    void stop(); // drains queued tasks first
    bool running() const { return running_; }
    void submit(std::function<void()> task);

private:
    void loop();
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<std::function<void()>> q_;
    bool running_ = false, stopping_ = false;
    std::thread th_;
};

class nixlP2PListener;

class nixlMetadataManager {
public:
    nixlMetadataManager(nixlMetadataContext &ctx, const nixlAgentConfig &cfg);
    ~nixlMetadataManager();

    // True when calls complete asynchronously (a thread exists), which is also when the
    // agent must lock even in sync mode NONE.
    bool usesThread() const;
    void start();
    void stop();

    nixl_status_t sendLocal(const nixl_opt_args_t *opt);
    nixl_status_t sendLocalPartial(const nixl_reg_dlist_t &descs, const nixl_opt_args_t *opt);
    nixl_status_t fetchRemote(const std::string &agent, const nixl_opt_args_t *opt);
    nixl_status_t invalidateLocal(const nixl_opt_args_t *opt);

    uint16_t listenPort() const;

private:
    nixl_status_t route(const nixl_opt_args_t *opt, bool &p2p) const;

    nixlMetadataContext &ctx_;
    nixlAgentConfig cfg_;
    nixlMetadataWorker worker_;
    std::unique_ptr<nixlP2PListener> listener_;
    std::unique_ptr<nixlMetadataBackend> store_;
    bool etcdRequested_ = false;
    std::mutex peersMu_;
    std::vector<std::pair<std::string, int>> peers_; // everyone we sent metadata to (for invalidateLocal broadcast)
};

#endif

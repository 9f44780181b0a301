// etcd as the central metadata store, spoken through etcd's v3 JSON gateway (HTTP/1.1:
// POST /v3/kv/put, /v3/kv/range, /v3/kv/deleterange with base64 keys and values), so no
// client library is needed.
//
// Parity: the reference's src/core/nixl_etcd_metadata_backend.cpp: keys
// <namespace>/<agent>/<label> with namespace NIXL_ETCD_NAMESPACE (default /nixl/agents,
// :40), fetch waits for a key that is not there yet (watch with timeout, :200; here a poll every
// 50 ms up to the same etcdWatchTimeout), and a watcher notices when a peer deletes its keys
// and invalidates that peer's metadata locally (:262-:330; here one watch stream over the
// namespace through POST /v3/watch, and, whenever that stream is not up, a poll of the keys
// fetched so far every NIXL_ETCD_POLL_MS, default 500).
#ifndef NIXL_B200_MD_ETCD_H
#define NIXL_B200_MD_ETCD_H

#include <atomic>
#include <chrono>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "core/md_manager.h"

namespace nixl_http {
// One request, one connection.  Returns the HTTP status (0 on transport failure) and the body.
int postJson(const std::string &host, int port, const std::string &path, const std::string &body, std::string &reply, int timeout_ms);
// Streaming reply: pieces of the body go to on_data as they arrive (see md_etcd.cpp).
int postStream(const std::string &host, int port, const std::string &path, const std::string &body, int timeout_ms,
               const std::function<bool()> &keep_going, const std::function<bool(const std::string &)> &on_data);
std::string base64Encode(const std::string &raw);
bool base64Decode(const std::string &text, std::string &raw);
} // namespace nixl_http

class nixlEtcdMetadataBackend : public nixlMetadataBackend {
public:
    // endpoints: "http://host:port[,http://host:port...]"; the first that answers is used.
    nixlEtcdMetadataBackend(const std::string &endpoints, std::chrono::microseconds watch_timeout);
    ~nixlEtcdMetadataBackend() override;
    bool ok() const { return port_ > 0; }

    nixl_status_t publish(const std::string &agent, const std::string &label, const nixl_blob_t &blob) override;
    nixl_status_t fetch(const std::string &agent, const std::string &label, nixl_blob_t &blob) override;
    nixl_status_t remove(const std::string &agent) override;

    // Called (from the watcher thread) with the name of a peer whose keys disappeared.
    void setInvalidateCallback(std::function<void(const std::string &)> cb);
    std::string makeKey(const std::string &agent, const std::string &label) const;

private:
    nixl_status_t get(const std::string &key, std::string &value);
    void watchLoop();
    bool watchStream();
    void keyGone(const std::string &key);

    std::string host_, namespace_;
    int port_ = 0;
    int opTimeoutMs_ = 5000, pollMs_ = 500;
    std::chrono::microseconds watchTimeout_;
    std::mutex mu_;
    std::vector<std::string> published_;           // keys this agent owns
    std::map<std::string, std::string> watched_;   // key -> peer agent, fetched so far
    std::function<void(const std::string &)> onGone_;
    std::atomic<bool> stop_{false};
    std::atomic<bool> watchActive_{false}; // a watch stream is being served
    std::thread watcher_;
};

#endif

// Client for torch's c10d TCPStore, used as a central metadata store.
//
// Parity: the reference's src/core/nixl_tcpstore_client.cpp (validation magic
// 0x3C85F7CE :42, query codes :50) and nixl_tcpstore_metadata_backend.cpp (key layout
// nixl/agents/<label>/<agent>/NULL_AGENT :40,:56; env NIXL_TCPSTORE_ENDPOINT,
// NIXL_TCPSTORE_TIMEOUT_MS, NIXL_TCPSTORE_OP_TIMEOUT_MS).  Keys carry the "/" prefix that
// torch's own client adds, so Python code using torch.distributed.TCPStore sees them.
#ifndef NIXL_B200_MD_TCPSTORE_H
#define NIXL_B200_MD_TCPSTORE_H

#include <mutex>
#include <string>
#include <vector>

#include "core/md_manager.h"

class nixlTcpStoreClient {
public:
    nixlTcpStoreClient(const std::string &host, int port, int connect_timeout_ms, int op_timeout_ms);
    ~nixlTcpStoreClient();
    bool connected() const { return fd_ >= 0; }

    nixl_status_t set(const std::string &key, const std::string &value);
    // NIXL_ERR_NOT_FOUND if the key does not exist (never blocks on a missing key).
    nixl_status_t get(const std::string &key, std::string &value);
    nixl_status_t check(const std::vector<std::string> &keys, bool &all_present);
    nixl_status_t deleteKey(const std::string &key);

private:
    bool handshake();
    bool sendAll(const std::string &buf);
    bool recvAll(void *p, size_t n);
    void reset();
    static void putStr(std::string &buf, const std::string &s);

    std::string host_;
    int port_, connectMs_, opMs_;
    int fd_ = -1;
    std::mutex mu_;
};

class nixlTcpStoreMetadataBackend : public nixlMetadataBackend {
public:
    explicit nixlTcpStoreMetadataBackend(const std::string &endpoint);
    bool ok() const { return client_ && client_->connected(); }
    nixl_status_t publish(const std::string &agent, const std::string &label, const nixl_blob_t &blob) override;
    nixl_status_t fetch(const std::string &agent, const std::string &label, nixl_blob_t &blob) override;
    nixl_status_t remove(const std::string &agent) override;
    static std::string makeKey(const std::string &agent, const std::string &label);

private:
    std::unique_ptr<nixlTcpStoreClient> client_;
    int fetchTimeoutMs_;
    std::mutex mu_;
    std::vector<std::string> published_; // keys we own, deleted by remove()
};

#endif

#include "core/md_manager.h"

#include <unistd.h>

#include <algorithm>

#include "core/md_p2p.h"
#include "core/md_etcd.h"
#include "core/md_tcpstore.h"
#include "utils/config.h"
#include "utils/log.h"

// ---------------------------------------------------------------- worker

void nixlMetadataWorker::start() {
    std::lock_guard<std::mutex> g(mu_);
    if (running_) return;
    running_ = true;
    stopping_ = false;
    th_ = std::thread([this] { loop(); });
}

void nixlMetadataWorker::stop() {
    {
        std::lock_guard<std::mutex> g(mu_);
        if (!running_) return;
        stopping_ = true;
    }
    cv_.notify_all();
    if (th_.joinable()) th_.join();
    std::lock_guard<std::mutex> g(mu_);
    running_ = false;
}

void nixlMetadataWorker::submit(std::function<void()> task) {
    {
        std::lock_guard<std::mutex> g(mu_);
        if (running_ && !stopping_) {
            q_.push_back(std::move(task));
            cv_.notify_one();
            return;
        }
    }
    task(); // no thread: run on the caller
}

void nixlMetadataWorker::loop() {
    std::unique_lock<std::mutex> lk(mu_);
    for (;;) {
        cv_.wait(lk, [this] { return stopping_ || !q_.empty(); });
        if (q_.empty()) {
            if (stopping_) return;
            continue;
        }
        auto task = std::move(q_.front());
        q_.pop_front();
        lk.unlock();
        task();
        lk.lock();
    }
}

// ---------------------------------------------------------------- manager

nixlMetadataManager::nixlMetadataManager(nixlMetadataContext &ctx, const nixlAgentConfig &cfg) : ctx_(ctx), cfg_(cfg) {
    const auto etcd = nixl::config::lookup("NIXL_ETCD_ENDPOINTS");
    const auto tcpstore = nixl::config::lookup("NIXL_TCPSTORE_ENDPOINT");
    if (etcd && !etcd->empty() && tcpstore && !tcpstore->empty())
        NIXL_WARN << "both NIXL_ETCD_ENDPOINTS and NIXL_TCPSTORE_ENDPOINT are set; using the TCPStore";
    if (tcpstore && !tcpstore->empty()) {
        auto b = std::make_unique<nixlTcpStoreMetadataBackend>(*tcpstore);
        if (b->ok()) store_ = std::move(b);
    } else if (etcd && !etcd->empty()) {
        etcdRequested_ = true;
        auto b = std::make_unique<nixlEtcdMetadataBackend>(*etcd, cfg.etcdWatchTimeout);
        if (b->ok()) {
            nixlMetadataContext *c = &ctx_;
            b->setInvalidateCallback([c](const std::string &agent) { c->mdInvalidateRemote(agent); });
            store_ = std::move(b);
        }
    }
    if (cfg.useListenThread) listener_ = std::make_unique<nixlP2PListener>(ctx, cfg.listenPort, cfg.lthrDelay);
}

nixlMetadataManager::~nixlMetadataManager() { stop(); }

bool nixlMetadataManager::usesThread() const { return listener_ || store_; }

uint16_t nixlMetadataManager::listenPort() const { return listener_ ? listener_->port() : 0; }

void nixlMetadataManager::start() {
    if (listener_) listener_->start();
    if (usesThread()) worker_.start();
}

void nixlMetadataManager::stop() {
    worker_.stop();
    if (listener_) listener_->stop();
}

// Decide the transport of one call: explicit ipAddr -> socket, else the central store.
nixl_status_t nixlMetadataManager::route(const nixl_opt_args_t *opt, bool &p2p) const {
    p2p = opt && !opt->ipAddr.empty();
    if (p2p) return NIXL_SUCCESS;
    if (store_) return NIXL_SUCCESS;
    if (etcdRequested_) return NIXL_ERR_NOT_SUPPORTED;
    NIXL_ERROR << "metadata exchange needs ipAddr/port or a configured central store";
    return NIXL_ERR_INVALID_PARAM;
}

static std::string labelOf(const nixl_opt_args_t *opt, const std::string &fallback) {
    return opt && !opt->metadataLabel.empty() ? opt->metadataLabel : fallback;
}

nixl_status_t nixlMetadataManager::sendLocal(const nixl_opt_args_t *opt) {
    bool p2p = false;
    if (auto st = route(opt, p2p); st != NIXL_SUCCESS) return st;
    nixl_blob_t blob;
    if (auto st = ctx_.mdGetLocal(blob); st != NIXL_SUCCESS) return st;
    if (p2p) {
        const std::string ip = opt->ipAddr;
        const int port = opt->port;
        {
            std::lock_guard<std::mutex> g(peersMu_);
            if (std::find(peers_.begin(), peers_.end(), std::make_pair(ip, port)) == peers_.end()) peers_.emplace_back(ip, port);
        }
        worker_.submit([ip, port, blob] {
            const int fd = nixl_p2p::dial(ip, port, 5000);
            if (fd < 0 || !nixl_p2p::sendFrame(fd, "NIXLCOMM:LOAD" + blob))
                NIXL_ERROR << "sendLocalMD: cannot deliver metadata to " << ip << ":" << port;
            if (fd >= 0) ::close(fd);
        });
        return NIXL_SUCCESS;
    }
    const std::string label = labelOf(opt, default_metadata_label);
    const std::string me = ctx_.mdAgentName();
    nixlMetadataBackend *store = store_.get();
    worker_.submit([store, me, label, blob] {
        if (store->publish(me, label, blob) != NIXL_SUCCESS) NIXL_ERROR << "sendLocalMD: publishing to the central store failed";
    });
    return NIXL_SUCCESS;
}

nixl_status_t nixlMetadataManager::sendLocalPartial(const nixl_reg_dlist_t &descs, const nixl_opt_args_t *opt) {
    bool p2p = false;
    if (auto st = route(opt, p2p); st != NIXL_SUCCESS) return st;
    nixl_blob_t blob;
    if (auto st = ctx_.mdGetLocalPartial(descs, blob, opt); st != NIXL_SUCCESS) return st;
    if (p2p) {
        const std::string ip = opt->ipAddr;
        const int port = opt->port;
        worker_.submit([ip, port, blob] {
            const int fd = nixl_p2p::dial(ip, port, 5000);
            if (fd < 0 || !nixl_p2p::sendFrame(fd, "NIXLCOMM:LOAD" + blob))
                NIXL_ERROR << "sendLocalPartialMD: cannot deliver metadata to " << ip << ":" << port;
            if (fd >= 0) ::close(fd);
        });
        return NIXL_SUCCESS;
    }
    // A label is mandatory so the partial blob does not overwrite the full one.
    if (!opt || opt->metadataLabel.empty()) return NIXL_ERR_INVALID_PARAM;
    const std::string label = opt->metadataLabel;
    const std::string me = ctx_.mdAgentName();
    nixlMetadataBackend *store = store_.get();
    worker_.submit([store, me, label, blob] {
        if (store->publish(me, label, blob) != NIXL_SUCCESS) NIXL_ERROR << "sendLocalPartialMD: publish failed";
    });
    return NIXL_SUCCESS;
}

nixl_status_t nixlMetadataManager::fetchRemote(const std::string &agent, const nixl_opt_args_t *opt) {
    bool p2p = false;
    if (auto st = route(opt, p2p); st != NIXL_SUCCESS) return st;
    nixlMetadataContext *ctx = &ctx_;
    if (p2p) {
        const std::string ip = opt->ipAddr;
        const int port = opt->port;
        worker_.submit([ctx, ip, port] {
            const int fd = nixl_p2p::dial(ip, port, 5000);
            std::string reply;
            if (fd < 0 || !nixl_p2p::sendFrame(fd, "NIXLCOMM:SEND") || !nixl_p2p::recvFrame(fd, reply, 5000)) {
                NIXL_ERROR << "fetchRemoteMD: no answer from " << ip << ":" << port;
            } else if (reply.compare(0, 13, "NIXLCOMM:LOAD") == 0) {
                std::string who;
                if (ctx->mdLoadRemote(reply.substr(13), who) != NIXL_SUCCESS) NIXL_ERROR << "fetchRemoteMD: metadata rejected";
            }
            if (fd >= 0) ::close(fd);
        });
        return NIXL_SUCCESS;
    }
    const std::string label = labelOf(opt, default_metadata_label);
    nixlMetadataBackend *store = store_.get();
    worker_.submit([ctx, store, agent, label] {
        nixl_blob_t blob;
        std::string who;
        if (store->fetch(agent, label, blob) != NIXL_SUCCESS) {
            NIXL_ERROR << "fetchRemoteMD: metadata of " << agent << " not found in the central store";
        } else if (ctx->mdLoadRemote(blob, who) != NIXL_SUCCESS) {
            NIXL_ERROR << "fetchRemoteMD: metadata of " << agent << " rejected";
        }
    });
    return NIXL_SUCCESS;
}

nixl_status_t nixlMetadataManager::invalidateLocal(const nixl_opt_args_t *opt) {
    const std::string me = ctx_.mdAgentName();
    std::vector<std::pair<std::string, int>> targets;
    if (opt && !opt->ipAddr.empty()) {
        targets.emplace_back(opt->ipAddr, opt->port);
    } else {
        std::lock_guard<std::mutex> g(peersMu_);
        targets = peers_;
    }
    if (targets.empty() && !store_) return etcdRequested_ ? NIXL_ERR_NOT_SUPPORTED : NIXL_ERR_INVALID_PARAM;
    for (auto &t : targets) {
        worker_.submit([t, me] {
            const int fd = nixl_p2p::dial(t.first, t.second, 2000);
            if (fd >= 0) {
                nixl_p2p::sendFrame(fd, "NIXLCOMM:INVL" + me);
                ::close(fd);
            }
        });
    }
    if (store_) {
        nixlMetadataBackend *store = store_.get();
        worker_.submit([store, me] { store->remove(me); });
    }
    return NIXL_SUCCESS;
}

// MOCK backend: an in-process loopback engine used by the tests to drive the agent without
// any transport (role parity: the reference's test/gtest/mocks/mock_backend_engine.cpp).
// DRAM only; transfers are memcpy performed at post time or, with parameter
// "async_polls=N", reported IN_PROG for N status polls first.  "fail_post=STATUS" makes every
// post return that status (fault injection on the host), "api_version=N" is honoured by the
// sibling plugin plugin_BADVERSION.
#include <cstring>
#include <mutex>

#include "backend/backend_plugin.h"

namespace {

class MockMD final : public nixlBackendMD {
public:
    explicit MockMD(bool priv) : nixlBackendMD(priv) {}
    uintptr_t addr = 0;
    size_t len = 0;
};

class MockReq final : public nixlBackendReqH {
public:
    int polls_left = 0;
    bool posted = false;
};

std::mutex g_mu;
std::vector<std::pair<std::string, std::pair<std::string, std::string>>> g_notifs; // target -> (from, msg)

class MockEngine final : public nixlBackendEngine {
public:
    explicit MockEngine(const nixlBackendInitParams *p) : nixlBackendEngine(p) {
        std::string v;
        if (getInitParam("async_polls", v) == NIXL_SUCCESS) asyncPolls_ = std::atoi(v.c_str());
        if (getInitParam("fail_post", v) == NIXL_SUCCESS) failPost_ = std::atoi(v.c_str());
        if (getInitParam("fail_init", v) == NIXL_SUCCESS && v == "true") initErr = true;
    }
    bool supportsRemote() const override { return true; }
    bool supportsLocal() const override { return true; }
    bool supportsNotif() const override { return true; }
    nixl_mem_list_t getSupportedMems() const override { return {DRAM_SEG}; }

    nixl_status_t registerMem(const nixlBlobDesc &mem, const nixl_mem_t &, nixlBackendMD *&out) override {
        auto *md = new MockMD(true);
        md->addr = mem.addr;
        md->len = mem.len;
        out = md;
        addTelemetryEvent(nixl_telemetry_event_type_t::AGENT_MEMORY_REGISTERED, 0);
        return NIXL_SUCCESS;
    }
    nixl_status_t deregisterMem(nixlBackendMD *meta) override {
        delete meta;
        return NIXL_SUCCESS;
    }
    nixl_status_t connect(const std::string &) override { return NIXL_SUCCESS; }
    nixl_status_t disconnect(const std::string &) override { return NIXL_SUCCESS; }
    nixl_status_t unloadMD(nixlBackendMD *input) override {
        delete input;
        return NIXL_SUCCESS;
    }
    nixl_status_t getPublicData(const nixlBackendMD *, std::string &str) const override {
        str = "mock-public";
        return NIXL_SUCCESS;
    }
    nixl_status_t getConnInfo(std::string &str) const override {
        str = "mock-conn:" + localAgent;
        return NIXL_SUCCESS;
    }
    nixl_status_t loadRemoteConnInfo(const std::string &agent, const std::string &info) override {
        return info == "mock-conn:" + agent ? NIXL_SUCCESS : NIXL_ERR_MISMATCH;
    }
    nixl_status_t loadRemoteMD(const nixlBlobDesc &input, const nixl_mem_t &, const std::string &, nixlBackendMD *&output) override {
        if (input.metaInfo != "mock-public") return NIXL_ERR_MISMATCH;
        auto *md = new MockMD(false);
        md->addr = input.addr;
        md->len = input.len;
        output = md;
        return NIXL_SUCCESS;
    }
    nixl_status_t loadLocalMD(nixlBackendMD *input, nixlBackendMD *&output) override {
        auto *in = static_cast<MockMD *>(input);
        auto *md = new MockMD(false);
        md->addr = in->addr;
        md->len = in->len;
        output = md;
        return NIXL_SUCCESS;
    }
    nixl_status_t prepXfer(const nixl_xfer_op_t &, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote, const std::string &,
                           nixlBackendReqH *&handle, const nixl_opt_b_args_t *) const override {
        if (local.descCount() != remote.descCount()) return NIXL_ERR_INVALID_PARAM;
        handle = new MockReq();
        return NIXL_SUCCESS;
    }
    nixl_status_t postXfer(const nixl_xfer_op_t &op, const nixl_meta_dlist_t &local, const nixl_meta_dlist_t &remote,
                           const std::string &remote_agent, nixlBackendReqH *&handle, const nixl_opt_b_args_t *opt) const override {
        if (failPost_) return static_cast<nixl_status_t>(failPost_);
        auto *req = static_cast<MockReq *>(handle);
        for (int i = 0; i < local.descCount(); ++i) {
            void *l = reinterpret_cast<void *>(local[i].addr), *r = reinterpret_cast<void *>(remote[i].addr);
            if (op == NIXL_WRITE) std::memcpy(r, l, local[i].len);
            else std::memcpy(l, r, local[i].len);
        }
        if (opt && opt->hasNotif) {
            std::lock_guard<std::mutex> g(g_mu);
            g_notifs.push_back({remote_agent, {localAgent, opt->notifMsg}});
        }
        req->posted = true;
        req->polls_left = asyncPolls_;
        return asyncPolls_ > 0 ? NIXL_IN_PROG : NIXL_SUCCESS;
    }
    nixl_status_t checkXfer(nixlBackendReqH *handle) const override {
        auto *req = static_cast<MockReq *>(handle);
        if (!req->posted) return NIXL_ERR_NOT_POSTED;
        if (req->polls_left > 0) {
            --req->polls_left;
            return NIXL_IN_PROG;
        }
        return NIXL_SUCCESS;
    }
    nixl_status_t releaseReqH(nixlBackendReqH *handle) const override {
        delete handle;
        return NIXL_SUCCESS;
    }
    nixl_status_t getNotifs(notif_list_t &list) override {
        std::lock_guard<std::mutex> g(g_mu);
        for (auto it = g_notifs.begin(); it != g_notifs.end();) {
            if (it->first == localAgent) {
                list.push_back(it->second);
                it = g_notifs.erase(it);
            } else ++it;
        }
        return NIXL_SUCCESS;
    }
    nixl_status_t genNotif(const std::string &remote_agent, const std::string &msg) const override {
        std::lock_guard<std::mutex> g(g_mu);
        g_notifs.push_back({remote_agent, {localAgent, msg}});
        return NIXL_SUCCESS;
    }

private:
    int asyncPolls_ = 0;
    int failPost_ = 0;
};

} // namespace

extern "C" NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init() {
    return nixlBackendPluginCreator<MockEngine>::create(NIXL_PLUGIN_API_VERSION, "MOCK", "0.1.0",
                                                        {{"async_polls", "0"}, {"fail_post", "0"}, {"fail_init", "false"}}, {DRAM_SEG});
}
extern "C" NIXL_PLUGIN_EXPORT void nixl_plugin_fini() {}

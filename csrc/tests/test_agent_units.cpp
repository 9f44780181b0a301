// Agent unit cases with the MOCK engine injected as the only backend: the scenario list of the
// reference's test/gtest/unit/agent/agent.cpp (plug-in lookup, backend creation and parameters,
// repeated registration, metadata load / invalidate, requests built from prepared lists and their
// argument checks, stand-alone notifications, connections, memory views), plus post-time failure
// injection and threads that share one agent.
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "core/plugin_manager.h"
#include "harness.h"
#include "nixl.h"

namespace {

std::string testPluginDir() {
    const char *d = std::getenv("NIXL_TEST_PLUGIN_DIR");
    return d ? d : "../nixl_b200/lib/test_plugins";
}

nixl_status_t waitDone(nixlAgent &a, nixlXferReqH *req) {
    nixl_status_t st;
    int spins = 0;
    while ((st = a.getXferStatus(req)) == NIXL_IN_PROG && ++spins < 100000000) {}
    return st;
}

// One agent with the MOCK engine.
struct Single {
    nixlAgent agent;
    nixlBackendH *backend = nullptr;
    explicit Single(const std::string &name, const nixl_b_params_t &params = {}, const nixlAgentConfig &cfg = nixlAgentConfig(false))
        : agent(name, cfg) {
        nixlPluginManager::getInstance().addPluginDirectory(testPluginDir());
        if (agent.createBackend("MOCK", params, backend) != NIXL_SUCCESS) throw std::runtime_error("MOCK backend unavailable");
    }
};

// Two agents, 16 blocks of 4 KiB registered on each side, metadata loaded both ways.
struct Bridge {
    Single a, b;
    static constexpr size_t kBlock = 4096, kBlocks = 16;
    std::vector<uint8_t> src, dst;
    Bridge(const nixl_b_params_t &params = {}, const nixlAgentConfig &cfg = nixlAgentConfig(false))
        : a("unit_a", params, cfg), b("unit_b", params, cfg), src(kBlock * kBlocks), dst(kBlock * kBlocks) {
        for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<uint8_t>(i * 13 + (i >> 12));
        nixl_reg_dlist_t ra(DRAM_SEG), rb(DRAM_SEG);
        ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
        rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
        if (a.agent.registerMem(ra) != NIXL_SUCCESS || b.agent.registerMem(rb) != NIXL_SUCCESS) throw std::runtime_error("registration");
        exchange();
    }
    void exchange() {
        nixl_blob_t md;
        std::string name;
        b.agent.getLocalMD(md);
        if (a.agent.loadRemoteMD(md, name) != NIXL_SUCCESS || name != "unit_b") throw std::runtime_error("metadata");
        a.agent.getLocalMD(md);
        if (b.agent.loadRemoteMD(md, name) != NIXL_SUCCESS || name != "unit_a") throw std::runtime_error("metadata");
    }
    nixl_xfer_dlist_t blocks(const std::vector<uint8_t> &buf, size_t first = 0, size_t count = kBlocks) const {
        nixl_xfer_dlist_t l(DRAM_SEG);
        for (size_t i = first; i < first + count; ++i) l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf.data()) + i * kBlock, kBlock, 0));
        return l;
    }
};

} // namespace

TEST_CASE(plugins_that_exist_and_plugins_that_do_not) {
    Single s("unit_plugins");
    nixl_mem_list_t mems;
    nixl_b_params_t params;
    CHECK_EQ(s.agent.getPluginParams("NO_SUCH_PLUGIN", mems, params), NIXL_ERR_NOT_FOUND);
    CHECK_EQ(s.agent.getPluginParams("MOCK", mems, params), NIXL_SUCCESS);
    CHECK(mems.size() == 1 && mems[0] == DRAM_SEG && params.count("async_polls") == 1);
    std::vector<nixl_backend_t> avail;
    CHECK_EQ(s.agent.getAvailPlugins(avail), NIXL_SUCCESS);
    CHECK(std::find(avail.begin(), avail.end(), "MOCK") != avail.end());
    nixlBackendH *h = nullptr;
    CHECK_EQ(s.agent.createBackend("NO_SUCH_PLUGIN", {}, h), NIXL_ERR_NOT_FOUND);
    CHECK(h == nullptr);
    CHECK_EQ(s.agent.createBackend("BADVERSION", {}, h), NIXL_ERR_NOT_FOUND); // API version mismatch: never loaded
    // an engine that fails to initialise is not installed
    nixlAgent other("unit_plugins_fail", nixlAgentConfig(false));
    CHECK(other.createBackend("MOCK", {{"fail_init", "true"}}, h) != NIXL_SUCCESS);
    nixl_blob_t md;
    CHECK_EQ(other.getLocalMD(md), NIXL_ERR_INVALID_PARAM); // no backend, nothing to advertise (nixl_agent.cpp: getLocalMD)
}

TEST_CASE(backend_parameters_of_existing_and_foreign_handles) {
    Single s("unit_params", {{"async_polls", "2"}});
    Single t("unit_params_other");
    nixl_mem_list_t mems;
    nixl_b_params_t params;
    CHECK_EQ(s.agent.getBackendParams(s.backend, mems, params), NIXL_SUCCESS);
    CHECK(params.at("async_polls") == "2");
    CHECK_EQ(s.agent.getBackendParams(nullptr, mems, params), NIXL_ERR_INVALID_PARAM);
    CHECK_EQ(s.agent.getBackendParams(t.backend, mems, params), NIXL_ERR_NOT_FOUND); // another agent's handle
}

TEST_CASE(register_and_deregister_many_times) {
    Single s("unit_rereg");
    std::vector<uint8_t> buf(1 << 16);
    nixl_reg_dlist_t reg(DRAM_SEG);
    reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf.data()), buf.size(), 0, ""));
    for (int i = 0; i < 100; ++i) {
        CHECK_EQ(s.agent.registerMem(reg), NIXL_SUCCESS);
        CHECK_EQ(s.agent.deregisterMem(reg), NIXL_SUCCESS);
    }
    CHECK_EQ(s.agent.deregisterMem(reg), NIXL_ERR_NOT_FOUND);
    // the same range twice is two registrations, released one by one
    CHECK_EQ(s.agent.registerMem(reg), NIXL_SUCCESS);
    CHECK_EQ(s.agent.registerMem(reg), NIXL_SUCCESS);
    CHECK_EQ(s.agent.deregisterMem(reg), NIXL_SUCCESS);
    CHECK_EQ(s.agent.deregisterMem(reg), NIXL_SUCCESS);
    CHECK_EQ(s.agent.deregisterMem(reg), NIXL_ERR_NOT_FOUND);
    nixl_reg_dlist_t none(DRAM_SEG);
    CHECK_EQ(s.agent.registerMem(none), NIXL_ERR_INVALID_PARAM);
    nixl_reg_dlist_t wrong(VRAM_SEG);
    wrong.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf.data()), buf.size(), 0, ""));
    CHECK_EQ(s.agent.registerMem(wrong), NIXL_ERR_NOT_FOUND); // no backend for that memory type
}

TEST_CASE(remote_metadata_can_be_loaded_checked_and_invalidated) {
    Bridge br;
    CHECK_EQ(br.a.agent.checkRemoteMD("unit_b", br.blocks(br.dst)), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.checkRemoteMD("unit_b", nixl_xfer_dlist_t(DRAM_SEG)), NIXL_SUCCESS); // "do we know the agent at all"
    CHECK_EQ(br.a.agent.checkRemoteMD("nobody", nixl_xfer_dlist_t(DRAM_SEG)), NIXL_ERR_NOT_FOUND);
    CHECK_EQ(br.a.agent.invalidateRemoteMD("unit_b"), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.invalidateRemoteMD("unit_b"), NIXL_ERR_NOT_FOUND);
    CHECK_EQ(br.a.agent.checkRemoteMD("unit_b", nixl_xfer_dlist_t(DRAM_SEG)), NIXL_ERR_NOT_FOUND);
    nixlXferReqH *req = nullptr;
    CHECK_EQ(br.a.agent.createXferReq(NIXL_WRITE, br.blocks(br.src, 0, 1), br.blocks(br.dst, 0, 1), "unit_b", req), NIXL_ERR_NOT_FOUND);
    br.exchange(); // and back
    CHECK_EQ(br.a.agent.createXferReq(NIXL_WRITE, br.blocks(br.src, 0, 1), br.blocks(br.dst, 0, 1), "unit_b", req), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.releaseXferReq(req), NIXL_SUCCESS);
    // garbage is refused without side effects
    std::string name;
    CHECK(br.a.agent.loadRemoteMD("not metadata", name) != NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.checkRemoteMD("unit_b", br.blocks(br.dst)), NIXL_SUCCESS);
}

TEST_CASE(requests_from_prepared_lists_and_their_argument_checks) {
    Bridge br;
    nixlDlistH *local = nullptr, *remote = nullptr, *alien = nullptr;
    CHECK_EQ(br.a.agent.prepXferDlist(NIXL_INIT_AGENT, br.blocks(br.src), local), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.prepXferDlist("unit_b", br.blocks(br.dst), remote), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.prepXferDlist("nobody", br.blocks(br.dst), alien), NIXL_ERR_NOT_FOUND);
    nixl_xfer_dlist_t outside(DRAM_SEG);
    outside.addDesc(nixlBasicDesc(0x1000, 64, 0));
    CHECK_EQ(br.a.agent.prepXferDlist(NIXL_INIT_AGENT, outside, alien), NIXL_ERR_NOT_FOUND);

    nixlXferReqH *req = nullptr;
    // blocks 0..3 of the source go to blocks 15..12 of the destination
    CHECK_EQ(br.a.agent.makeXferReq(NIXL_WRITE, local, {0, 1, 2, 3}, remote, {15, 14, 13, 12}, req), NIXL_SUCCESS);
    nixl_status_t st = br.a.agent.postXferReq(req);
    CHECK(st == NIXL_SUCCESS || st == NIXL_IN_PROG);
    CHECK_EQ(waitDone(br.a.agent, req), NIXL_SUCCESS);
    for (int i = 0; i < 4; ++i) CHECK(std::memcmp(br.src.data() + i * Bridge::kBlock, br.dst.data() + (15 - i) * Bridge::kBlock, Bridge::kBlock) == 0);
    CHECK_EQ(br.a.agent.releaseXferReq(req), NIXL_SUCCESS);

    CHECK_EQ(br.a.agent.makeXferReq(NIXL_WRITE, local, {0, 1}, remote, {0}, req), NIXL_ERR_INVALID_PARAM);        // counts differ
    CHECK_EQ(br.a.agent.makeXferReq(NIXL_WRITE, local, {0, 99}, remote, {0, 1}, req), NIXL_ERR_INVALID_PARAM);    // index out of range
    CHECK_EQ(br.a.agent.makeXferReq(NIXL_WRITE, local, {0, -1}, remote, {0, 1}, req), NIXL_ERR_INVALID_PARAM);    // negative index
    CHECK_EQ(br.a.agent.makeXferReq(NIXL_WRITE, remote, {0}, remote, {0}, req), NIXL_ERR_INVALID_PARAM);          // the local side must be the initiator's
    CHECK_EQ(br.a.agent.makeXferReq(NIXL_WRITE, local, {}, remote, {}, req), NIXL_ERR_INVALID_PARAM);             // nothing to move
    CHECK_EQ(br.a.agent.makeXferReq(NIXL_WRITE, nullptr, {0}, remote, {0}, req), NIXL_ERR_INVALID_PARAM);

    // a READ through the same prepared lists
    std::memset(br.src.data(), 0, Bridge::kBlock);
    for (size_t i = 0; i < Bridge::kBlock; ++i) br.dst[5 * Bridge::kBlock + i] = static_cast<uint8_t>(i ^ 0x5a);
    CHECK_EQ(br.a.agent.makeXferReq(NIXL_READ, local, {0}, remote, {5}, req), NIXL_SUCCESS);
    st = br.a.agent.postXferReq(req);
    CHECK(st == NIXL_SUCCESS || st == NIXL_IN_PROG);
    CHECK_EQ(waitDone(br.a.agent, req), NIXL_SUCCESS);
    CHECK(std::memcmp(br.src.data(), br.dst.data() + 5 * Bridge::kBlock, Bridge::kBlock) == 0);
    CHECK_EQ(br.a.agent.releaseXferReq(req), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.releasedDlistH(local), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.releasedDlistH(remote), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.releasedDlistH(nullptr), NIXL_ERR_INVALID_PARAM);
}

TEST_CASE(notifications_on_their_own) {
    Bridge br;
    CHECK_EQ(br.a.agent.genNotif("unit_b", "first"), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.genNotif("unit_b", std::string("bin\0ary", 7)), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.genNotif("nobody", "x"), NIXL_ERR_NOT_FOUND);
    nixl_notifs_t got;
    for (int i = 0; i < 100000 && got["unit_a"].size() < 2; ++i) CHECK_EQ(br.b.agent.getNotifs(got), NIXL_SUCCESS);
    CHECK(got["unit_a"].size() == 2 && got["unit_a"][0] == "first" && got["unit_a"][1] == std::string("bin\0ary", 7));
    // a map that already holds entries is appended to, and nothing is delivered twice
    CHECK_EQ(br.b.agent.getNotifs(got), NIXL_SUCCESS);
    CHECK(got["unit_a"].size() == 2);
    // a backend named explicitly
    nixl_opt_args_t via;
    via.backends.push_back(br.a.backend);
    CHECK_EQ(br.a.agent.genNotif("unit_b", "third", &via), NIXL_SUCCESS);
    for (int i = 0; i < 100000 && got["unit_a"].size() < 3; ++i) br.b.agent.getNotifs(got);
    CHECK(got["unit_a"].back() == "third");
    nixl_opt_args_t foreign;
    foreign.backends.push_back(br.b.backend); // not this agent's handle
    CHECK(br.a.agent.genNotif("unit_b", "no", &foreign) != NIXL_SUCCESS);
}

TEST_CASE(connections_and_memory_views) {
    Bridge br;
    CHECK_EQ(br.a.agent.makeConnection("unit_b"), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.makeConnection("nobody"), NIXL_ERR_NOT_FOUND);
    nixl_opt_args_t foreign;
    foreign.backends.push_back(br.b.backend);
    CHECK(br.a.agent.makeConnection("unit_b", &foreign) != NIXL_SUCCESS);
    // the MOCK engine has no device-side views: no engine can build one, and the agent says so instead of inventing one
    nixl_remote_dlist_t remote(DRAM_SEG);
    remote.addDesc(nixlRemoteDesc(reinterpret_cast<uintptr_t>(br.dst.data()), 4096, 0, "unit_b"));
    nixlMemViewH view = nullptr;
    CHECK_EQ(br.a.agent.prepMemView(remote, view), NIXL_ERR_NOT_FOUND);
    CHECK(view == nullptr);
    nixl_remote_dlist_t unknown(DRAM_SEG);
    unknown.addDesc(nixlRemoteDesc(reinterpret_cast<uintptr_t>(br.dst.data()), 4096, 0, "nobody"));
    CHECK(br.a.agent.prepMemView(unknown, view) != NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.prepMemView(nixl_remote_dlist_t(DRAM_SEG), view), NIXL_ERR_INVALID_PARAM);
}

TEST_CASE(a_post_that_fails_leaves_the_request_reusable_state) {
    // fail_post makes every post of the engine return that status: the agent must hand it on and keep
    // the request out of the "in progress" state, so that it can be released at once.
    Bridge br({{"fail_post", std::to_string(static_cast<int>(NIXL_ERR_BACKEND))}});
    nixlXferReqH *req = nullptr;
    CHECK_EQ(br.a.agent.createXferReq(NIXL_WRITE, br.blocks(br.src, 0, 2), br.blocks(br.dst, 0, 2), "unit_b", req), NIXL_SUCCESS);
    CHECK_EQ(br.a.agent.postXferReq(req), NIXL_ERR_BACKEND);
    CHECK_EQ(br.a.agent.getXferStatus(req), NIXL_ERR_BACKEND);
    CHECK_EQ(br.a.agent.postXferReq(req), NIXL_ERR_BACKEND); // not REPOST_ACTIVE: nothing is running
    CHECK_EQ(br.a.agent.releaseXferReq(req), NIXL_SUCCESS);
}

TEST_CASE(threads_share_one_agent) {
    // Strict synchronisation: creation, posting, polling and release from four threads at once, while a fifth
    // keeps registering and deregistering a buffer of its own.
    nixlAgentConfig cfg(false);
    cfg.syncMode = nixl_thread_sync_t::NIXL_THREAD_SYNC_STRICT;
    Bridge br({{"async_polls", "2"}}, cfg);
    std::atomic<int> failures{0};
    std::atomic<bool> stop{false};
    std::thread churn([&] {
        std::vector<uint8_t> mine(8192);
        nixl_reg_dlist_t reg(DRAM_SEG);
        reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(mine.data()), mine.size(), 0, ""));
        while (!stop) {
            if (br.a.agent.registerMem(reg) != NIXL_SUCCESS || br.a.agent.deregisterMem(reg) != NIXL_SUCCESS) ++failures;
        }
    });
    std::vector<std::thread> workers;
    for (int t = 0; t < 4; ++t)
        workers.emplace_back([&, t] {
            for (int i = 0; i < 200; ++i) {
                nixlXferReqH *req = nullptr;
                const size_t blk = static_cast<size_t>(t) * 4 + (i & 3);
                if (br.a.agent.createXferReq(NIXL_WRITE, br.blocks(br.src, blk, 1), br.blocks(br.dst, blk, 1), "unit_b", req) != NIXL_SUCCESS) {
                    ++failures;
                    continue;
                }
                const nixl_status_t st = br.a.agent.postXferReq(req);
                if (st != NIXL_SUCCESS && st != NIXL_IN_PROG) ++failures;
                if (waitDone(br.a.agent, req) != NIXL_SUCCESS) ++failures;
                if (br.a.agent.releaseXferReq(req) != NIXL_SUCCESS) ++failures;
            }
        });
    for (auto &w : workers) w.join();
    stop = true;
    churn.join();
    CHECK_EQ(failures.load(), 0);
    CHECK(std::memcmp(br.src.data(), br.dst.data(), br.src.size()) == 0);
}

TEST_MAIN()

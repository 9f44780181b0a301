// Unit and integration tests of the core on CPU: serializer wire format, descriptors, sections,
// configuration, plugin manager, agent behaviour against the MOCK backend, peer-to-peer
// metadata exchange over 127.0.0.1, host-side fault injection, telemetry, tracing, threads.
// Scenarios follow the reference's test/unit/utils/serdes, test/gtest/unit/{descriptors,agent},
// test/gtest/{plugin_manager,configuration,metadata_exchange,error_handling,multi_threading,
// telemetry_test}.cpp.
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <thread>
#include <unistd.h>

#include "core/plugin_manager.h"
#include "core/telemetry/ring_file.h"
#include "core/telemetry/telemetry.h"
#include "core/tracing/trace.h"
#include "harness.h"
#include "infra/sections.h"
#include "nixl.h"
#include "utils/config.h"
#include "utils/file/file_utils.h"

namespace {

std::string testPluginDir() {
    const char *d = std::getenv("NIXL_TEST_PLUGIN_DIR");
    return d ? d : "../nixl_b200/lib/test_plugins";
}

struct ScopedEnv {
    ScopedEnv(const char *k, const char *v) : key(k) {
        if (const char *old = std::getenv(k)) {
            had = true;
            prev = old;
        }
        ::setenv(k, v, 1);
    }
    ~ScopedEnv() {
        if (had) ::setenv(key.c_str(), prev.c_str(), 1);
        else ::unsetenv(key.c_str());
    }
    std::string key, prev;
    bool had = false;
};

nixl_status_t waitDone(nixlAgent &a, nixlXferReqH *req) {
    nixl_status_t st;
    int spins = 0;
    while ((st = a.getXferStatus(req)) == NIXL_IN_PROG && ++spins < 100000000) {}
    return st;
}

template<class F> bool eventually(F f, int ms = 5000) {
    const auto end = std::chrono::steady_clock::now() + std::chrono::milliseconds(ms);
    while (std::chrono::steady_clock::now() < end) {
        if (f()) return true;
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
    return f();
}

} // namespace

// ------------------------------------------------------------------ serializer

TEST_CASE(serdes_golden_bytes) {
    nixlSerDes sd;
    sd.addStr("Agent", "a1");
    const uint64_t n = 2;
    sd.addBuf("Conns", &n, sizeof(n));
    const std::string got = sd.exportStr();
    // "nixlSerDes|" + "Agent" + u64(2) + "a1" + "|" + "Conns" + u64(8) + u64(2) + "|"
    std::string want = "nixlSerDes|Agent";
    const uint64_t two = 2, eight = 8;
    want.append(reinterpret_cast<const char *>(&two), 8);
    want += "a1|Conns";
    want.append(reinterpret_cast<const char *>(&eight), 8);
    want.append(reinterpret_cast<const char *>(&two), 8);
    want += "|";
    CHECK(got == want);

    nixlSerDes rd;
    CHECK_EQ(rd.importStr(got), NIXL_SUCCESS);
    CHECK(rd.getStr("Agent") == "a1");
    CHECK_EQ(rd.getBufLen("Conns"), 8);
    uint64_t back = 0;
    CHECK_EQ(rd.getBuf("Conns", &back, 8), NIXL_SUCCESS);
    CHECK_EQ(back, 2u);
    // Errors: wrong tag, wrong length, truncated input, missing magic.
    nixlSerDes bad;
    bad.importStr(got);
    CHECK(bad.getStr("Nope").empty());
    nixlSerDes bad2;
    bad2.importStr(got);
    bad2.getStr("Agent");
    uint32_t small = 0;
    CHECK_EQ(bad2.getBuf("Conns", &small, 4), NIXL_ERR_MISMATCH);
    nixlSerDes bad3;
    CHECK_EQ(bad3.importStr(got.substr(0, got.size() - 3)), NIXL_SUCCESS);
    bad3.getStr("Agent");
    CHECK_EQ(bad3.getBuf("Conns", &back, 8), NIXL_ERR_MISMATCH);
    nixlSerDes bad4;
    CHECK_EQ(bad4.importStr("garbage"), NIXL_ERR_MISMATCH);
    // A hostile length must not overflow the bounds check.
    std::string evil = "nixlSerDes|t";
    const uint64_t huge = ~0ull;
    evil.append(reinterpret_cast<const char *>(&huge), 8);
    evil += "x|";
    nixlSerDes bad5;
    bad5.importStr(evil);
    CHECK(bad5.getStr("t").empty());
}

// ------------------------------------------------------------------ descriptors

TEST_CASE(descriptor_lists) {
    nixlBasicDesc a(0x1000, 0x100, 0), b(0x1080, 0x40, 0), c(0x1080, 0x100, 0), d(0x1000, 0x100, 1);
    CHECK(a.covers(b) && !a.covers(c) && !a.covers(d));
    CHECK(a.overlaps(c) && !a.overlaps(d));
    CHECK(a < c && a < d && !(c < a));
    CHECK(nixlBasicDesc(a.serialize()) == a);

    nixl_xfer_dlist_t l(VRAM_SEG);
    for (int i = 0; i < 5; ++i) l.addDesc(nixlBasicDesc(0x1000 + i * 0x100, 0x100, 3));
    CHECK_EQ(l.descCount(), 5);
    CHECK_EQ(l.getIndex(nixlBasicDesc(0x1200, 0x100, 3)), 2);
    CHECK_EQ(l.getIndex(nixlBasicDesc(0x1200, 0x10, 3)), NIXL_ERR_NOT_FOUND);
    l.remDesc(0);
    CHECK_EQ(l.descCount(), 4);
    bool threw = false;
    try {
        l.remDesc(17);
    } catch (const std::out_of_range &) {
        threw = true;
    }
    CHECK(threw);
    nixlSerDes sd;
    CHECK_EQ(l.serialize(&sd), NIXL_SUCCESS);
    nixlSerDes rd;
    rd.importStr(sd.exportStr());
    nixl_xfer_dlist_t back(&rd);
    CHECK(back.valid() && back == l);

    nixl_reg_dlist_t r(FILE_SEG);
    r.addDesc(nixlBlobDesc(0, 0, 7, "rw,create:/tmp/x"));
    r.addDesc(nixlBlobDesc(4096, 10, 8, std::string("bin\0ary", 7)));
    nixlSerDes sd2;
    r.serialize(&sd2);
    nixlSerDes rd2;
    rd2.importStr(sd2.exportStr());
    nixl_reg_dlist_t rback(&rd2);
    CHECK(rback.valid() && rback == r && rback[1].metaInfo.size() == 7);
    CHECK(r.trim().descCount() == 2 && r.trim().getType() == FILE_SEG);
    // A basic list cannot be read as a blob list.
    nixlSerDes rd3;
    rd3.importStr(sd.exportStr());
    nixl_reg_dlist_t wrong(&rd3);
    CHECK(!wrong.valid() && wrong.isEmpty());
}

TEST_CASE(sections_cover_lookup) {
    nixlSecDescList s(DRAM_SEG);
    // nested and overlapping registrations on two devices
    s.addDesc(nixlSectionDesc(nixlBasicDesc(0x1000, 0x10000, 0), "", nullptr));
    s.addDesc(nixlSectionDesc(nixlBasicDesc(0x2000, 0x100, 0), "", nullptr));
    s.addDesc(nixlSectionDesc(nixlBasicDesc(0x3000, 0x2000, 0), "", nullptr));
    s.addDesc(nixlSectionDesc(nixlBasicDesc(0x20000, 0x1000, 0), "", nullptr));
    s.addDesc(nixlSectionDesc(nixlBasicDesc(0x1000, 0x100, 1), "", nullptr));
    CHECK_EQ(s.descCount(), 5);
    for (int i = 1; i < s.descCount(); ++i) CHECK(!(static_cast<const nixlBasicDesc &>(s[i]) < static_cast<const nixlBasicDesc &>(s[i - 1])));
    // Covered only by the big outer registration although smaller ones start closer.
    int at = s.getCoveringIndex(nixlBasicDesc(0x3800, 0x3000, 0));
    CHECK(at >= 0 && s[at].addr == 0x1000 && s[at].len == 0x10000);
    CHECK(s.getCoveringIndex(nixlBasicDesc(0x20800, 0x100, 0)) >= 0);
    CHECK_EQ(s.getCoveringIndex(nixlBasicDesc(0x20800, 0x1000, 0)), -1); // runs past the end
    CHECK_EQ(s.getCoveringIndex(nixlBasicDesc(0x1000, 0x10, 2)), -1);     // unknown device
    CHECK_EQ(s.getCoveringIndex(nixlBasicDesc(0x500, 0x10, 0)), -1);      // before everything
    CHECK(s.getIndex(nixlBasicDesc(0x2000, 0x100, 0)) >= 0);
    s.remDesc(s.getIndex(nixlBasicDesc(0x1000, 0x10000, 0)));
    CHECK_EQ(s.getCoveringIndex(nixlBasicDesc(0x3800, 0x3000, 0)), -1);
    // Unbounded FILE registrations (len 0) cover any range of that file.
    nixlSecDescList f(FILE_SEG);
    f.addDesc(nixlSectionDesc(nixlBasicDesc(0, 0, 5), "", nullptr));
    CHECK(f.getCoveringIndex(nixlBasicDesc(1ull << 40, 1 << 20, 5)) == 0);
}

// ------------------------------------------------------------------ configuration, files

TEST_CASE(configuration_env_then_file) {
    char path[] = "/tmp/nixl_b200_cfg_XXXXXX";
    const int fd = ::mkstemp(path);
    CHECK(fd >= 0);
    const char *text = "# comment\nNIXL_TEST_ALPHA = 42\ntest_beta = \"hello # not a comment\"\n[nixl]\ntest_gamma = true\ntest_bad = 12abc\n";
    CHECK(::write(fd, text, std::strlen(text)) > 0);
    ::close(fd);
    {
        ScopedEnv e("NIXL_CONFIG_FILE", path);
        nixl::config::reload();
        CHECK_EQ(nixl::config::getValue<int>("NIXL_TEST_ALPHA"), 42);
        CHECK(nixl::config::getValue<std::string>("NIXL_TEST_BETA") == "hello # not a comment");
        CHECK(nixl::config::getValue<bool>("NIXL_TEST_GAMMA"));
        CHECK(!nixl::config::getValueOptional<int>("NIXL_TEST_MISSING").has_value());
        CHECK_EQ(nixl::config::getValueDefaulted<int>("NIXL_TEST_MISSING", 7), 7);
        bool threw = false;
        try {
            nixl::config::getValue<int>("NIXL_TEST_BAD");
        } catch (const std::runtime_error &) {
            threw = true;
        }
        CHECK(threw);
        ScopedEnv over("NIXL_TEST_ALPHA", "43"); // the environment wins over the file
        CHECK_EQ(nixl::config::getValue<int>("NIXL_TEST_ALPHA"), 43);
    }
    nixl::config::reload();
    ::unlink(path);
}

TEST_CASE(file_path_mode_strings) {
    auto a = nixl::parsePathMeta("rw,create,sync:/tmp/some:file");
    CHECK(a.has_value() && a->path == "/tmp/some:file" && (a->flags & O_CREAT) && (a->flags & O_SYNC) && a->mode == 0644);
    CHECK(nixl::parsePathMeta("ro:/x").has_value());
    CHECK(!nixl::parsePathMeta("rx:/x").has_value());
    CHECK(!nixl::parsePathMeta("rw,bogus:/x").has_value());
    CHECK(!nixl::parsePathMeta("rw:").has_value());
    CHECK(!nixl::parsePathMeta("/plain/path").has_value());
    CHECK(!nixl::queryFileInfo("/nonexistent/file").has_value());
    CHECK(nixl::queryFileInfo("ro:/proc/self/exe").has_value());
}

// ------------------------------------------------------------------ plugin manager

TEST_CASE(plugin_manager_discovery) {
    auto &pm = nixlPluginManager::getInstance();
    pm.addPluginDirectory(testPluginDir());
    auto avail = pm.getAvailableBackendPlugins();
    auto has = [&](const char *n) { return std::find(avail.begin(), avail.end(), std::string(n)) != avail.end(); };
    CHECK(has("NVLINK") && has("POSIX") && has("MOCK") && has("BADVERSION"));
    CHECK(pm.loadBackendPlugin("BADVERSION") == nullptr); // API version mismatch
    CHECK(pm.loadBackendPlugin("NO_SUCH") == nullptr);
    auto mock = pm.loadBackendPlugin("MOCK");
    CHECK(mock != nullptr && std::string(mock->getName()) == "MOCK" && !mock->isStatic());
    CHECK(pm.loadBackendPlugin("MOCK") == mock); // cached
    CHECK(mock->getBackendOptions().count("async_polls") == 1);
    CHECK(pm.resolveAlias("UCX") == "NVLINK" && pm.resolveAlias("POSIX") == "POSIX");
    for (const char *fabric : {"GPUNETIO", "UCX_MO"}) CHECK(pm.resolveAlias(fabric) == "NVLINK");
    for (const char *fabric : {"LIBFABRIC", "MOONCAKE", "UCCL"}) CHECK(pm.resolveAlias(fabric) == "TCP"); // node-to-node transports
    // static registration
    pm.registerStaticBackend("STATIC_NULL", []() -> nixlBackendPlugin * { return nullptr; });
    CHECK(pm.loadBackendPlugin("STATIC_NULL") == nullptr); // creator returned null -> refused
    static nixlBackendPlugin table = {NIXL_PLUGIN_API_VERSION, nullptr, nullptr, [] { return "STATIC_OK"; }, [] { return "1"; },
                                      [] { return nixl_b_params_t{{"k", "v"}}; }, [] { return nixl_mem_list_t{DRAM_SEG}; }};
    pm.registerStaticBackend("STATIC_OK", []() -> nixlBackendPlugin * { return &table; });
    auto st = pm.loadBackendPlugin("STATIC_OK");
    CHECK(st != nullptr && st->isStatic() && st->getBackendOptions().at("k") == "v");
}

// ------------------------------------------------------------------ agent with the MOCK backend

namespace {
struct MockPair {
    nixlAgent a, b;
    nixlBackendH *ba = nullptr, *bb = nullptr;
    std::vector<uint8_t> src, dst;
    explicit MockPair(const nixl_b_params_t &params = {}, const nixlAgentConfig &cfg = nixlAgentConfig(false))
        : a("mock_a", cfg), b("mock_b", cfg), src(1 << 16), dst(1 << 16) {
        nixlPluginManager::getInstance().addPluginDirectory(testPluginDir());
        if (a.createBackend("MOCK", params, ba) != NIXL_SUCCESS || b.createBackend("MOCK", params, bb) != NIXL_SUCCESS)
            throw std::runtime_error("MOCK backend unavailable");
        for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<uint8_t>(i * 7);
        nixl_reg_dlist_t ra(DRAM_SEG), rb(DRAM_SEG);
        ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
        rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
        a.registerMem(ra);
        b.registerMem(rb);
        nixl_blob_t md;
        std::string name;
        b.getLocalMD(md);
        a.loadRemoteMD(md, name);
    }
    nixl_xfer_dlist_t L(size_t off = 0, size_t len = 4096) {
        nixl_xfer_dlist_t l(DRAM_SEG);
        l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()) + off, len, 0));
        return l;
    }
    nixl_xfer_dlist_t R(size_t off = 0, size_t len = 4096) {
        nixl_xfer_dlist_t l(DRAM_SEG);
        l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.data()) + off, len, 0));
        return l;
    }
};
} // namespace

TEST_CASE(agent_status_conventions) {
    MockPair p({{"async_polls", "3"}});
    nixlXferReqH *req = nullptr;
    CHECK_EQ(p.a.createXferReq(NIXL_WRITE, p.L(), p.R(), "mock_b", req), NIXL_SUCCESS);
    CHECK_EQ(p.a.getXferStatus(req), NIXL_ERR_NOT_POSTED);
    CHECK_EQ(p.a.postXferReq(req), NIXL_IN_PROG);
    CHECK_EQ(p.a.postXferReq(req), NIXL_ERR_REPOST_ACTIVE); // still running
    CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
    CHECK(std::memcmp(p.src.data(), p.dst.data(), 4096) == 0);
    CHECK_EQ(p.a.postXferReq(req), NIXL_IN_PROG); // re-postable once complete
    CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
    nixlBackendH *used = nullptr;
    CHECK_EQ(p.a.queryXferBackend(req, used), NIXL_SUCCESS);
    CHECK(used == p.ba);
    CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);

    // argument checking
    CHECK_EQ(p.a.createXferReq(NIXL_WRITE, p.L(0, 4096), p.R(0, 2048), "mock_b", req), NIXL_ERR_INVALID_PARAM); // lengths differ
    CHECK_EQ(p.a.createXferReq(NIXL_WRITE, p.L(), p.R(), "nobody", req), NIXL_ERR_NOT_FOUND);
    nixl_xfer_dlist_t outside(DRAM_SEG);
    outside.addDesc(nixlBasicDesc(0x10, 4096, 0));
    CHECK_EQ(p.a.createXferReq(NIXL_WRITE, outside, p.R(), "mock_b", req), NIXL_ERR_NOT_FOUND); // not registered
    CHECK_EQ(p.a.createXferReq(NIXL_WRITE, p.L(), p.R(1 << 16, 4096), "mock_b", req), NIXL_ERR_NOT_FOUND); // beyond remote registration
    // one engine per backend type
    nixlBackendH *again = nullptr;
    CHECK_EQ(p.a.createBackend("MOCK", {}, again), NIXL_ERR_INVALID_PARAM);
    nixl_mem_list_t mems;
    nixl_b_params_t params;
    CHECK_EQ(p.a.getBackendParams(p.ba, mems, params), NIXL_SUCCESS);
    CHECK(params.at("async_polls") == "3" && mems.size() == 1);
}

TEST_CASE(agent_notification_precedence) {
    MockPair p;
    nixl_opt_args_t with;
    with.notif = "created-with";
    nixlXferReqH *req = nullptr;
    CHECK_EQ(p.a.createXferReq(NIXL_WRITE, p.L(), p.R(), "mock_b", req, &with), NIXL_SUCCESS);
    auto drain = [&]() {
        nixl_notifs_t n;
        p.b.getNotifs(n);
        std::vector<std::string> v;
        if (n.count("mock_a")) v = n["mock_a"];
        return v;
    };
    CHECK_EQ(p.a.postXferReq(req), NIXL_SUCCESS); // no extra params: creation-time message is used
    CHECK(drain() == std::vector<std::string>{"created-with"});
    nixl_opt_args_t over;
    over.notif = "override";
    CHECK_EQ(p.a.postXferReq(req, &over), NIXL_SUCCESS);
    CHECK(drain() == std::vector<std::string>{"override"});
    nixl_opt_args_t legacy;
    legacy.hasNotif = true;
    legacy.notifMsg = "legacy";
    CHECK_EQ(p.a.postXferReq(req, &legacy), NIXL_SUCCESS);
    CHECK(drain() == std::vector<std::string>{"legacy"});
    nixl_opt_args_t none; // extra params without a notification clear it
    CHECK_EQ(p.a.postXferReq(req, &none), NIXL_SUCCESS);
    CHECK(drain().empty());
    CHECK_EQ(p.a.postXferReq(req), NIXL_SUCCESS); // and it stays cleared
    CHECK(drain().empty());
    p.a.releaseXferReq(req);
    CHECK_EQ(p.a.genNotif("mock_b", "standalone"), NIXL_SUCCESS);
    CHECK(drain() == std::vector<std::string>{"standalone"});
    CHECK_EQ(p.a.genNotif("nobody", "x"), NIXL_ERR_NOT_FOUND);
}

TEST_CASE(agent_stale_remote_and_partial_md) {
    MockPair p;
    nixlXferReqH *req = nullptr;
    CHECK_EQ(p.a.createXferReq(NIXL_WRITE, p.L(), p.R(), "mock_b", req), NIXL_SUCCESS);
    nixlDlistH *lh = nullptr, *rh = nullptr;
    CHECK_EQ(p.a.prepXferDlist(NIXL_INIT_AGENT, p.L(), lh), NIXL_SUCCESS);
    CHECK_EQ(p.a.prepXferDlist("mock_b", p.R(), rh), NIXL_SUCCESS);
    // The peer goes away and comes back: old handles refer to a dead generation.
    CHECK_EQ(p.a.invalidateRemoteMD("mock_b"), NIXL_SUCCESS);
    CHECK_EQ(p.a.postXferReq(req), NIXL_ERR_NOT_FOUND);
    nixl_blob_t md;
    std::string name;
    p.b.getLocalMD(md);
    CHECK_EQ(p.a.loadRemoteMD(md, name), NIXL_SUCCESS);
    CHECK_EQ(p.a.postXferReq(req), NIXL_ERR_NOT_FOUND); // same name, new generation
    nixlXferReqH *req2 = nullptr;
    CHECK_EQ(p.a.makeXferReq(NIXL_WRITE, lh, {0}, rh, {0}, req2), NIXL_ERR_NOT_FOUND);
    p.a.releaseXferReq(req);
    p.a.releasedDlistH(lh);
    p.a.releasedDlistH(rh);
    CHECK_EQ(p.a.invalidateRemoteMD("never-seen"), NIXL_ERR_NOT_FOUND);

    // Partial metadata: connection info first, then a single registration.
    nixlAgent c("mock_c", nixlAgentConfig(false));
    nixlBackendH *bc = nullptr;
    CHECK_EQ(c.createBackend("MOCK", {}, bc), NIXL_SUCCESS);
    nixl_reg_dlist_t empty(DRAM_SEG);
    nixl_blob_t conn_only;
    CHECK_EQ(p.b.getLocalPartialMD(empty, conn_only), NIXL_SUCCESS);
    CHECK_EQ(c.loadRemoteMD(conn_only, name), NIXL_SUCCESS);
    CHECK_EQ(c.checkRemoteMD("mock_b", nixl_xfer_dlist_t(DRAM_SEG)), NIXL_SUCCESS);
    CHECK_EQ(c.checkRemoteMD("mock_b", p.R()), NIXL_ERR_NOT_FOUND);
    nixl_reg_dlist_t one(DRAM_SEG);
    one.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(p.dst.data()), p.dst.size(), 0, ""));
    nixl_blob_t part;
    CHECK_EQ(p.b.getLocalPartialMD(one, part), NIXL_SUCCESS); // no connection info inside
    CHECK_EQ(c.loadRemoteMD(part, name), NIXL_SUCCESS);
    CHECK_EQ(c.checkRemoteMD("mock_b", p.R()), NIXL_SUCCESS);
    nixl_reg_dlist_t unknown(DRAM_SEG);
    unknown.addDesc(nixlBlobDesc(0x1234000, 64, 0, ""));
    CHECK_EQ(p.b.getLocalPartialMD(unknown, part), NIXL_ERR_NOT_FOUND);
    // Malformed blobs.
    CHECK_EQ(c.loadRemoteMD("not metadata", name), NIXL_ERR_MISMATCH);
    CHECK_EQ(c.loadRemoteMD(md.substr(0, md.size() / 2), name), NIXL_ERR_MISMATCH);
    // A peer with no backend in common.
    nixlAgent d("posix_only", nixlAgentConfig(false));
    nixlBackendH *bd = nullptr;
    CHECK_EQ(d.createBackend("POSIX", {}, bd), NIXL_SUCCESS);
    nixl_blob_t none;
    CHECK_EQ(d.getLocalMD(none), NIXL_ERR_INVALID_PARAM); // POSIX cannot be reached remotely
    CHECK_EQ(d.loadRemoteMD(md, name), NIXL_ERR_BACKEND);
}

TEST_CASE(host_side_fault_injection) {
    // Backend-level failure injected by parameter: the post reports it, the agent counts it.
    ScopedEnv t("NIXL_TELEMETRY_ENABLE", "y");
    MockPair p({{"fail_post", "-3"}});
    nixlXferReqH *req = nullptr;
    CHECK_EQ(p.a.createXferReq(NIXL_WRITE, p.L(), p.R(), "mock_b", req), NIXL_SUCCESS);
    CHECK_EQ(p.a.postXferReq(req), NIXL_ERR_BACKEND);
    CHECK_EQ(p.a.getXferStatus(req), NIXL_ERR_BACKEND);
    p.a.releaseXferReq(req);
    nixlBackendH *h = nullptr;
    nixlAgent z("mock_z", nixlAgentConfig(false));
    CHECK_EQ(z.createBackend("MOCK", {{"fail_init", "true"}}, h), NIXL_ERR_BACKEND);

    // Transport-level failure: the target agent of the NVLINK backend is destroyed; the
    // initiator gets REMOTE_DISCONNECT, forgets the peer, and recovers when it returns
    // (reference: test/gtest/error_handling.cpp:421-506).
    std::vector<uint8_t> s(1 << 16, 9), d(1 << 16, 0);
    nixlAgent ini("fi_initiator", nixlAgentConfig(false));
    nixlBackendH *bi = nullptr;
    CHECK_EQ(ini.createBackend("NVLINK", {}, bi), NIXL_SUCCESS);
    nixl_reg_dlist_t rs(DRAM_SEG), rd(DRAM_SEG);
    rs.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(s.data()), s.size(), 0, ""));
    rd.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(d.data()), d.size(), 0, ""));
    ini.registerMem(rs);
    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(s.data()), 4096, 0));
    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(d.data()), 4096, 0));
    std::string name;
    for (int round = 0; round < 2; ++round) {
        auto tgt = std::make_unique<nixlAgent>("fi_target", nixlAgentConfig(false));
        nixlBackendH *bt = nullptr;
        CHECK_EQ(tgt->createBackend("NVLINK", {}, bt), NIXL_SUCCESS);
        tgt->registerMem(rd);
        nixl_blob_t md;
        tgt->getLocalMD(md);
        CHECK_EQ(ini.loadRemoteMD(md, name), NIXL_SUCCESS);
        CHECK_EQ(ini.createXferReq(NIXL_WRITE, l, r, "fi_target", req), NIXL_SUCCESS);
        CHECK(ini.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(ini, req), NIXL_SUCCESS);
        tgt.reset(); // the peer dies between steps
        CHECK_EQ(ini.postXferReq(req), NIXL_ERR_REMOTE_DISCONNECT);
        CHECK_EQ(ini.checkRemoteMD("fi_target", nixl_xfer_dlist_t(DRAM_SEG)), NIXL_ERR_NOT_FOUND); // metadata dropped
        CHECK_EQ(ini.genNotif("fi_target", "hello?"), NIXL_ERR_NOT_FOUND);
        ini.releaseXferReq(req);
    }
}

// ------------------------------------------------------------------ metadata over sockets

TEST_CASE(p2p_metadata_exchange) {
    nixlPluginManager::getInstance().addPluginDirectory(testPluginDir());
    nixlAgentConfig cfg(false, true, 0); // listener on an ephemeral port is not discoverable: use fixed ports
    const uint16_t port_a = static_cast<uint16_t>(20000 + (::getpid() % 20000)), port_b = port_a + 1;
    nixlAgentConfig ca(false, true, port_a), cb(false, true, port_b);
    nixlAgent a("sock_a", ca), b("sock_b", cb);
    nixlBackendH *ba = nullptr, *bb = nullptr;
    CHECK_EQ(a.createBackend("MOCK", {}, ba), NIXL_SUCCESS);
    CHECK_EQ(b.createBackend("MOCK", {}, bb), NIXL_SUCCESS);
    std::vector<uint8_t> buf_a(4096), buf_b(4096);
    nixl_reg_dlist_t ra(DRAM_SEG), rb(DRAM_SEG);
    ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf_a.data()), 4096, 0, ""));
    rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf_b.data()), 4096, 0, ""));
    a.registerMem(ra);
    b.registerMem(rb);
    nixl_xfer_dlist_t xa(DRAM_SEG), xb(DRAM_SEG);
    xa.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf_a.data()), 4096, 0));
    xb.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf_b.data()), 4096, 0));

    nixl_opt_args_t to_b;
    to_b.ipAddr = "127.0.0.1";
    to_b.port = port_b;
    CHECK_EQ(a.sendLocalMD(&to_b), NIXL_SUCCESS); // push: b learns a
    CHECK(eventually([&] { return b.checkRemoteMD("sock_a", xa) == NIXL_SUCCESS; }));
    CHECK_EQ(a.fetchRemoteMD("sock_b", &to_b), NIXL_SUCCESS); // pull: a learns b
    CHECK(eventually([&] { return a.checkRemoteMD("sock_b", xb) == NIXL_SUCCESS; }));
    CHECK_EQ(a.invalidateLocalMD(&to_b), NIXL_SUCCESS); // b forgets a
    CHECK(eventually([&] { return b.checkRemoteMD("sock_a", nixl_xfer_dlist_t(DRAM_SEG)) == NIXL_ERR_NOT_FOUND; }));
    // Without address and without a central store there is nowhere to send to.
    CHECK_EQ(a.sendLocalMD(nullptr), NIXL_ERR_INVALID_PARAM);
    {
        ScopedEnv etcd("NIXL_ETCD_ENDPOINTS", "http://127.0.0.1:2379");
        nixlAgent e("etcd_user", nixlAgentConfig(false));
        nixlBackendH *be = nullptr;
        e.createBackend("MOCK", {}, be);
        CHECK_EQ(e.sendLocalMD(nullptr), NIXL_ERR_NOT_SUPPORTED); // no etcd client in this build
    }
}

// ------------------------------------------------------------------ telemetry and tracing

TEST_CASE(telemetry_buffer_exporter_and_request_stats) {
    char dir[] = "/tmp/nixl_b200_telem_XXXXXX";
    CHECK(::mkdtemp(dir) != nullptr);
    ScopedEnv e1("NIXL_TELEMETRY_ENABLE", "1"), e2("NIXL_TELEMETRY_DIR", dir), e3("NIXL_TELEMETRY_RUN_INTERVAL", "5");
    ScopedEnv e4("NIXL_TELEMETRY_ENABLED_METRICS", "agent_tx_*,agent_xfer_time,agent_memory_registered");
    {
        MockPair p;
        nixlXferReqH *req = nullptr;
        CHECK_EQ(p.a.createXferReq(NIXL_WRITE, p.L(0, 8192), p.R(0, 8192), "mock_b", req), NIXL_SUCCESS);
        CHECK_EQ(p.a.postXferReq(req), NIXL_SUCCESS);
        nixl_xfer_telem_t t;
        CHECK_EQ(p.a.getXferTelemetry(req, t), NIXL_SUCCESS);
        CHECK_EQ(t.totalBytes, 8192u);
        CHECK_EQ(t.descCount, 1u);
        p.a.releaseXferReq(req);
        // A reader in "another process" attaches to the ring file and drains it.
        const std::string ring_path = std::string(dir) + "/mock_a";
        CHECK(eventually([&] {
            try {
                nixlRingFile ring(ring_path, false);
                return ring.size() >= 3;
            } catch (...) {
                return false;
            }
        }));
        nixlRingFile ring(ring_path, false);
        CHECK_EQ(ring.version(), static_cast<uint32_t>(TELEMETRY_VERSION));
        bool saw_tx = false, saw_time = false, saw_reg = false, saw_other = false;
        nixlTelemetryEvent ev;
        while (ring.pop(&ev)) {
            if (ev.eventType_ == nixl_telemetry_event_type_t::AGENT_TX_BYTES) saw_tx = ev.value_ == 8192;
            else if (ev.eventType_ == nixl_telemetry_event_type_t::AGENT_XFER_TIME) saw_time = true;
            else if (ev.eventType_ == nixl_telemetry_event_type_t::AGENT_MEMORY_REGISTERED) saw_reg = true;
            else if (ev.eventType_ == nixl_telemetry_event_type_t::AGENT_XFER_POST_TIME) saw_other = true; // filtered out
        }
        CHECK(saw_tx && saw_time && saw_reg && !saw_other);
    }
    // Without telemetry a request has no statistics.
    ::unsetenv("NIXL_TELEMETRY_ENABLE");
    {
        MockPair q;
        nixlXferReqH *req = nullptr;
        q.a.createXferReq(NIXL_WRITE, q.L(), q.R(), "mock_b", req);
        q.a.postXferReq(req);
        nixl_xfer_telem_t t;
        CHECK_EQ(q.a.getXferTelemetry(req, t), NIXL_ERR_NO_TELEMETRY);
        q.a.releaseXferReq(req);
    }
    ::setenv("NIXL_TELEMETRY_ENABLE", "1", 1);
    std::string cleanup = std::string("rm -rf ") + dir;
    CHECK(std::system(cleanup.c_str()) == 0);
}

TEST_CASE(telemetry_staging_queue_bounds) {
    nixlTelemetryStagingQueue q(4);
    for (int i = 0; i < 6; ++i) q.push(nixlTelemetryEvent(nixl_telemetry_event_type_t::AGENT_TX_BYTES, i));
    std::vector<nixlTelemetryEvent> out;
    CHECK_EQ(q.drain(out), 2u); // two were dropped
    CHECK_EQ(out.size(), 4u);
    CHECK_EQ(q.drain(out), 0u);
    CHECK(out.empty());
    CHECK(nixlTelemetryEventTypeForStatus(NIXL_ERR_NOT_POSTED) == nixl_telemetry_event_type_t::AGENT_ERR_NOT_POSTED);
    CHECK(nixlTelemetryEventTypeForStatus(NIXL_ERR_NO_TELEMETRY) == nixl_telemetry_event_type_t::AGENT_ERR_NO_TELEMETRY);
    ScopedEnv b("NIXL_TELEMETRY_HISTOGRAM_BUCKETS_US", "5,50,500");
    CHECK(nixlTelemetryHistogramBucketsUs() == (std::vector<uint64_t>{5, 50, 500}));
}

TEST_CASE(tracing_spans_and_correlation) {
    ScopedEnv e("NIXL_TRACE_BACKENDS", "memory,nvtx,not_a_backend");
    nixl::trace::memoryBackendDrain();
    {
        MockPair p;
        nixlXferReqH *req = nullptr;
        p.a.createXferReq(NIXL_WRITE, p.L(), p.R(), "mock_b", req);
        p.a.postXferReq(req);
        p.a.getXferStatus(req);
        p.a.releaseXferReq(req);
    }
    auto recs = nixl::trace::memoryBackendDrain();
    auto find = [&](const char *what, const char *agent) {
        for (auto &r : recs)
            if (r.what == what && r.agent == agent) return &r;
        return static_cast<nixl::trace::Record *>(nullptr);
    };
    CHECK(find("createBackend", "mock_a") && find("registerMem", "mock_b") && find("createXferReq", "mock_a"));
    auto *post = find("postXferReq", "mock_a");
    CHECK(post && post->kind == nixl::trace::Kind::POST && post->correlation != 0 && !post->isMark);
    nixl::trace::Tracer off("quiet");
    CHECK(off.enabled()); // env still set in this scope
}

// ------------------------------------------------------------------ threads

TEST_CASE(multithreaded_post_and_poll) {
    nixlAgentConfig cfg(false, false, 0, nixl_thread_sync_t::NIXL_THREAD_SYNC_RW);
    MockPair p({{"async_polls", "2"}}, cfg);
    std::atomic<int> failures{0};
    std::vector<std::thread> threads;
    for (int t = 0; t < 8; ++t) {
        threads.emplace_back([&, t] {
            for (int i = 0; i < 200; ++i) {
                nixlXferReqH *req = nullptr;
                const size_t off = static_cast<size_t>(t) * 4096;
                if (p.a.createXferReq(NIXL_WRITE, p.L(off), p.R(off), "mock_b", req) != NIXL_SUCCESS) {
                    ++failures;
                    continue;
                }
                if (p.a.postXferReq(req) < 0 || waitDone(p.a, req) != NIXL_SUCCESS) ++failures;
                nixl_notifs_t n;
                p.b.getNotifs(n);
                if (p.a.releaseXferReq(req) != NIXL_SUCCESS) ++failures;
            }
        });
    }
    std::thread registrar([&] { // table-changing calls interleave with the transfers
        std::vector<uint8_t> extra(4096);
        nixl_reg_dlist_t r(DRAM_SEG);
        r.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(extra.data()), extra.size(), 0, ""));
        for (int i = 0; i < 200; ++i) {
            if (p.a.registerMem(r) != NIXL_SUCCESS) ++failures;
            if (p.a.deregisterMem(r) != NIXL_SUCCESS) ++failures;
        }
    });
    for (auto &t : threads) t.join();
    registrar.join();
    CHECK_EQ(failures.load(), 0);
    CHECK(std::memcmp(p.src.data(), p.dst.data(), 8 * 4096) == 0);
}

TEST_MAIN()

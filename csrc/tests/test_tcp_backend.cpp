// The TCP backend (src/plugins/extra/plugin_TCP.cpp) through the agent: the transport for peers that NVLink does not
// reach.  Every case runs over real sockets on the loopback interface, which is as much of "another host" as one machine
// offers: scattered WRITE and READ, requests cut into messages and dealt over several connections, notifications that
// follow their data, a range whose registration went away at the target, threads, two processes, a target that exits, an
// agent that comes back under its old name, and transfers of an agent to itself.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <unistd.h>

#include <array>
#include <atomic>
#include <chrono>
#include <cstring>
#include <fstream>
#include <map>
#include <random>
#include <sstream>
#include <thread>

#include "harness.h"
#include "nixl.h"

namespace {

using clk = std::chrono::steady_clock;

nixl_status_t waitDone(nixlAgent &a, nixlXferReqH *req, int seconds = 30) {
    nixl_status_t st;
    const auto end = clk::now() + std::chrono::seconds(seconds);
    while ((st = a.getXferStatus(req)) == NIXL_IN_PROG && clk::now() < end) {}
    return st;
}

std::vector<std::string> collect(nixlAgent &agent, const std::string &from, size_t want, int seconds = 5) {
    std::vector<std::string> got;
    const auto end = clk::now() + std::chrono::seconds(seconds);
    while (got.size() < want && clk::now() < end) {
        nixl_notifs_t n;
        agent.getNotifs(n);
        for (auto &m : n[from]) got.push_back(m);
    }
    return got;
}

int g_serial = 0;

struct Pair {
    std::string an, bn;
    std::unique_ptr<nixlAgent> a, b;
    std::vector<uint8_t> src, dst;
    nixl_reg_dlist_t ra{DRAM_SEG}, rb{DRAM_SEG};
    Pair(size_t bytes, const nixl_b_params_t &params = {{"address", "127.0.0.1"}})
        : an("tcp_a" + std::to_string(++g_serial)), bn("tcp_b" + std::to_string(g_serial)), a(new nixlAgent(an, nixlAgentConfig(false))),
          b(new nixlAgent(bn, nixlAgentConfig(false))), src(bytes), dst(bytes, 0) {
        nixlBackendH *ha = nullptr, *hb = nullptr;
        if (a->createBackend("TCP", params, ha) != NIXL_SUCCESS || b->createBackend("TCP", params, hb) != NIXL_SUCCESS)
            throw std::runtime_error("TCP backend unavailable");
        std::mt19937 rng(1000 + g_serial);
        for (size_t i = 0; i + 4 <= bytes; i += 4) {
            const uint32_t v = rng();
            std::memcpy(src.data() + i, &v, 4);
        }
        ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
        rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
        if (a->registerMem(ra) != NIXL_SUCCESS || b->registerMem(rb) != NIXL_SUCCESS) throw std::runtime_error("registration");
        nixl_blob_t md;
        std::string name;
        b->getLocalMD(md);
        if (a->loadRemoteMD(md, name) != NIXL_SUCCESS) throw std::runtime_error("metadata");
        a->getLocalMD(md);
        if (b->loadRemoteMD(md, name) != NIXL_SUCCESS) throw std::runtime_error("metadata");
    }
    nixlXferReqH *request(nixl_xfer_op_t op, const std::vector<std::array<size_t, 3>> &cuts, const nixl_opt_args_t *args = nullptr) {
        nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
        for (auto &c : cuts) { // {local offset, remote offset, length}
            l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()) + c[0], c[2], 0));
            r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.data()) + c[1], c[2], 0));
        }
        nixlXferReqH *req = nullptr;
        if (a->createXferReq(op, l, r, bn, req, args) != NIXL_SUCCESS) throw std::runtime_error("createXferReq");
        return req;
    }
};

} // namespace

TEST_CASE(scattered_write_then_read_between_two_agents) {
    Pair p(4 << 20);
    std::vector<std::array<size_t, 3>> cuts;
    std::vector<uint8_t> expect(p.dst.size(), 0);
    for (size_t i = 0; i < 60; ++i) {
        const size_t lo = i * 60000 + 13, ro = (59 - i) * 60000 + 7, len = 1 + i * 997;
        cuts.push_back({lo, ro, len});
        std::memcpy(expect.data() + ro, p.src.data() + lo, len);
    }
    nixlXferReqH *w = p.request(NIXL_WRITE, cuts);
    CHECK(p.a->postXferReq(w) >= 0);
    CHECK_EQ(waitDone(*p.a, w), NIXL_SUCCESS);
    CHECK(p.dst == expect);
    // change the target's bytes and READ them back into the places they came from
    for (auto &x : p.dst) x = static_cast<uint8_t>(x ^ 0x5a);
    nixlXferReqH *r = p.request(NIXL_READ, cuts);
    CHECK(p.a->postXferReq(r) >= 0);
    CHECK_EQ(waitDone(*p.a, r), NIXL_SUCCESS);
    for (auto &c : cuts) CHECK(std::memcmp(p.src.data() + c[0], p.dst.data() + c[1], c[2]) == 0);
    // the same request again, as the agent allows once the last post has completed
    CHECK(p.a->postXferReq(w) >= 0);
    CHECK_EQ(waitDone(*p.a, w), NIXL_SUCCESS);
    CHECK_EQ(p.a->releaseXferReq(w), NIXL_SUCCESS);
    CHECK_EQ(p.a->releaseXferReq(r), NIXL_SUCCESS);
    // the request ran on this backend and no other
    nixlXferReqH *q = p.request(NIXL_WRITE, {{0, 0, 64}});
    nixlBackendH *used = nullptr;
    CHECK_EQ(p.a->queryXferBackend(q, used), NIXL_SUCCESS);
    CHECK(used != nullptr);
    CHECK_EQ(p.a->releaseXferReq(q), NIXL_SUCCESS);
}

TEST_CASE(a_large_request_is_dealt_over_the_rails_and_small_descriptors_share_messages) {
    Pair p(40 << 20, {{"address", "127.0.0.1"}, {"rails", "3"}, {"chunk_bytes", "1048576"}});
    // one descriptor of 33 MiB and a bit (34 messages over three connections) ...
    const size_t big = (33 << 20) + 4321;
    nixlXferReqH *w = p.request(NIXL_WRITE, {{5, 5, big}});
    CHECK(p.a->postXferReq(w) >= 0);
    CHECK_EQ(waitDone(*p.a, w), NIXL_SUCCESS);
    CHECK(std::memcmp(p.src.data() + 5, p.dst.data() + 5, big) == 0);
    CHECK_EQ(p.a->releaseXferReq(w), NIXL_SUCCESS);
    // ... and five thousand of 512 bytes in reverse order (256 per message)
    std::vector<std::array<size_t, 3>> cuts;
    const size_t base = 34 << 20;
    for (size_t i = 0; i < 5000; ++i) cuts.push_back({base + i * 1024, base + (4999 - i) * 1024, 512});
    nixlXferReqH *s = p.request(NIXL_WRITE, cuts);
    CHECK(p.a->postXferReq(s) >= 0);
    CHECK_EQ(waitDone(*p.a, s), NIXL_SUCCESS);
    for (auto &c : cuts) CHECK(std::memcmp(p.src.data() + c[0], p.dst.data() + c[1], 512) == 0);
    CHECK_EQ(p.a->releaseXferReq(s), NIXL_SUCCESS);
    // the cost estimate follows what the engine has seen: 33 MiB are expected to take longer than 4 KiB, and about
    // as long as they just did
    {
        nixlXferReqH *probe_small = p.request(NIXL_WRITE, {{0, 0, 4096}}), *probe_big = p.request(NIXL_WRITE, {{5, 5, big}});
        std::chrono::microseconds d_small{}, d_big{}, margin{};
        nixl_cost_t how;
        CHECK_EQ(p.a->estimateXferCost(probe_small, d_small, margin, how), NIXL_SUCCESS);
        CHECK_EQ(p.a->estimateXferCost(probe_big, d_big, margin, how), NIXL_SUCCESS);
        CHECK(d_big.count() > 20 * d_small.count() && d_big.count() > 1000 && d_big.count() < 2000000 && margin.count() > 0);
        CHECK_EQ(p.a->releaseXferReq(probe_small), NIXL_SUCCESS);
        CHECK_EQ(p.a->releaseXferReq(probe_big), NIXL_SUCCESS);
    }
    // READ of the large range the other way round
    std::memset(p.src.data() + 5, 0, big);
    nixlXferReqH *r = p.request(NIXL_READ, {{5, 5, big}});
    CHECK(p.a->postXferReq(r) >= 0);
    CHECK_EQ(waitDone(*p.a, r), NIXL_SUCCESS);
    CHECK(std::memcmp(p.src.data() + 5, p.dst.data() + 5, big) == 0);
    CHECK_EQ(p.a->releaseXferReq(r), NIXL_SUCCESS);
}

TEST_CASE(a_notification_follows_its_data_and_plain_notifications_arrive_in_order) {
    Pair p(8 << 20, {{"address", "127.0.0.1"}, {"rails", "4"}, {"chunk_bytes", "65536"}});
    for (int round = 0; round < 20; ++round) {
        std::memset(p.dst.data(), 0, p.dst.size());
        nixl_opt_args_t args;
        args.notif = "round " + std::to_string(round);
        nixlXferReqH *w = p.request(NIXL_WRITE, {{0, 0, p.src.size()}}, &args);
        CHECK(p.a->postXferReq(w) >= 0);
        // the target only looks at its notifications; when one is there, every byte is
        auto got = collect(*p.b, p.an, 1);
        CHECK_EQ(got.size(), size_t(1));
        CHECK(got[0] == args.notif);
        CHECK(p.dst == p.src);
        CHECK_EQ(waitDone(*p.a, w), NIXL_SUCCESS);
        CHECK_EQ(p.a->releaseXferReq(w), NIXL_SUCCESS);
    }
    for (int i = 0; i < 50; ++i) CHECK_EQ(p.a->genNotif(p.bn, "n" + std::to_string(i)), NIXL_SUCCESS);
    auto got = collect(*p.b, p.an, 50);
    CHECK_EQ(got.size(), size_t(50));
    for (int i = 0; i < 50; ++i) CHECK(got[i] == "n" + std::to_string(i));
    // and the other way, on connections of the other agent's own
    CHECK_EQ(p.b->genNotif(p.an, std::string("\0binary\xff", 8)), NIXL_SUCCESS);
    auto back = collect(*p.a, p.bn, 1);
    CHECK_EQ(back.size(), size_t(1));
    CHECK(back[0] == std::string("\0binary\xff", 8));
}

TEST_CASE(a_range_whose_registration_went_away_is_refused_and_the_connection_survives) {
    Pair p(1 << 20);
    // a second registration at the target, published, then withdrawn behind the initiator's back
    std::vector<uint8_t> extra(1 << 16, 0x11);
    nixl_reg_dlist_t re(DRAM_SEG);
    re.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(extra.data()), extra.size(), 0, ""));
    CHECK_EQ(p.b->registerMem(re), NIXL_SUCCESS);
    nixl_blob_t md;
    std::string name;
    p.b->getLocalMD(md);
    CHECK_EQ(p.a->loadRemoteMD(md, name), NIXL_SUCCESS);
    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(p.src.data()), 4096, 0));
    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(extra.data()), 4096, 0));
    nixlXferReqH *w = nullptr, *rd = nullptr;
    CHECK_EQ(p.a->createXferReq(NIXL_WRITE, l, r, p.bn, w), NIXL_SUCCESS);
    CHECK_EQ(p.a->createXferReq(NIXL_READ, l, r, p.bn, rd), NIXL_SUCCESS);
    CHECK(p.a->postXferReq(w) >= 0);
    CHECK_EQ(waitDone(*p.a, w), NIXL_SUCCESS);
    CHECK(std::memcmp(extra.data(), p.src.data(), 4096) == 0);
    CHECK_EQ(p.b->deregisterMem(re), NIXL_SUCCESS);
    std::memset(extra.data(), 0x22, extra.size());
    const std::vector<uint8_t> before = p.src;
    CHECK(p.a->postXferReq(w) >= 0);
    CHECK_EQ(waitDone(*p.a, w), NIXL_ERR_INVALID_PARAM); // the target's answer
    CHECK(extra[0] == 0x22 && extra[4095] == 0x22);        // and nothing was written
    CHECK(p.a->postXferReq(rd) >= 0);
    CHECK_EQ(waitDone(*p.a, rd), NIXL_ERR_INVALID_PARAM);
    CHECK(p.src == before);
    // the connections are still good for what is registered
    nixlXferReqH *ok = p.request(NIXL_WRITE, {{0, 0, 100000}});
    CHECK(p.a->postXferReq(ok) >= 0);
    CHECK_EQ(waitDone(*p.a, ok), NIXL_SUCCESS);
    CHECK(std::memcmp(p.dst.data(), p.src.data(), 100000) == 0);
    for (auto *q : {w, rd, ok}) CHECK_EQ(p.a->releaseXferReq(q), NIXL_SUCCESS);
}

TEST_CASE(threads_post_side_by_side_over_shared_connections) {
    Pair p(16 << 20, {{"address", "127.0.0.1"}, {"rails", "2"}, {"chunk_bytes", "262144"}});
    constexpr int kThreads = 6;
    std::atomic<int> bad{0};
    std::vector<std::thread> th;
    for (int t = 0; t < kThreads; ++t)
        th.emplace_back([&, t] {
            const size_t lane = size_t(t) * (2 << 20);
            for (int i = 0; i < 40; ++i) {
                const size_t len = 1000 + size_t(i) * 50000 % (2 << 20);
                nixl_opt_args_t args;
                args.notif = "t" + std::to_string(t);
                nixlXferReqH *w = p.request(i % 4 == 3 ? NIXL_READ : NIXL_WRITE, {{lane, lane, len}}, i % 5 == 0 ? &args : nullptr);
                if (p.a->postXferReq(w) < 0 || waitDone(*p.a, w) != NIXL_SUCCESS) ++bad;
                if (std::memcmp(p.src.data() + lane, p.dst.data() + lane, len) != 0) ++bad;
                if (p.a->releaseXferReq(w) != NIXL_SUCCESS) ++bad;
            }
        });
    for (auto &t : th) t.join();
    CHECK_EQ(bad.load(), 0);
    CHECK_EQ(collect(*p.b, p.an, kThreads * 8).size(), size_t(kThreads * 8));
}

TEST_CASE(an_agent_moves_data_and_notifies_within_itself) {
    nixlAgent a("tcp_self", nixlAgentConfig(false));
    nixlBackendH *h = nullptr;
    CHECK_EQ(a.createBackend("TCP", {{"address", "127.0.0.1"}}, h), NIXL_SUCCESS);
    std::vector<uint8_t> x(1 << 16), y(1 << 16, 0);
    for (size_t i = 0; i < x.size(); ++i) x[i] = static_cast<uint8_t>(i * 7);
    nixl_reg_dlist_t reg(DRAM_SEG);
    reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(x.data()), x.size(), 0, ""));
    reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(y.data()), y.size(), 0, ""));
    CHECK_EQ(a.registerMem(reg), NIXL_SUCCESS);
    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(x.data()), x.size(), 0));
    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(y.data()), y.size(), 0));
    nixl_opt_args_t args;
    args.notif = "to myself";
    nixlXferReqH *w = nullptr;
    CHECK_EQ(a.createXferReq(NIXL_WRITE, l, r, "tcp_self", w, &args), NIXL_SUCCESS);
    CHECK(a.postXferReq(w) >= 0);
    CHECK_EQ(waitDone(a, w), NIXL_SUCCESS);
    CHECK(x == y);
    auto got = collect(a, "tcp_self", 1);
    CHECK_EQ(got.size(), size_t(1));
    CHECK(got[0] == "to myself");
    CHECK_EQ(a.releaseXferReq(w), NIXL_SUCCESS);
    CHECK_EQ(a.deregisterMem(reg), NIXL_SUCCESS);
}

TEST_CASE(a_target_that_is_gone_is_reported_and_one_that_comes_back_under_its_name_is_reached_again) {
    Pair p(1 << 20);
    nixlXferReqH *w = p.request(NIXL_WRITE, {{0, 0, 4096}});
    CHECK(p.a->postXferReq(w) >= 0);
    CHECK_EQ(waitDone(*p.a, w), NIXL_SUCCESS);
    p.b->deregisterMem(p.rb);
    p.b.reset(); // the agent and its listener are gone
    nixl_status_t st = p.a->postXferReq(w);
    if (st >= 0) st = waitDone(*p.a, w);
    CHECK_EQ(st, NIXL_ERR_REMOTE_DISCONNECT);
    // the agent has dropped what it knew of the peer
    CHECK_EQ(p.a->checkRemoteMD(p.bn, nixl_xfer_dlist_t(DRAM_SEG)), NIXL_ERR_NOT_FOUND);
    p.a->releaseXferReq(w);
    // the peer starts again under its name (another port, another engine) and publishes itself
    p.b.reset(new nixlAgent(p.bn, nixlAgentConfig(false)));
    nixlBackendH *hb = nullptr;
    CHECK_EQ(p.b->createBackend("TCP", {{"address", "127.0.0.1"}}, hb), NIXL_SUCCESS);
    CHECK_EQ(p.b->registerMem(p.rb), NIXL_SUCCESS);
    nixl_blob_t md;
    std::string name;
    p.b->getLocalMD(md);
    CHECK_EQ(p.a->loadRemoteMD(md, name), NIXL_SUCCESS);
    std::memset(p.dst.data(), 0, p.dst.size());
    nixlXferReqH *again = p.request(NIXL_WRITE, {{100, 100, 50000}});
    CHECK(p.a->postXferReq(again) >= 0);
    CHECK_EQ(waitDone(*p.a, again), NIXL_SUCCESS);
    CHECK(std::memcmp(p.src.data() + 100, p.dst.data() + 100, 50000) == 0);
    CHECK_EQ(p.a->releaseXferReq(again), NIXL_SUCCESS);
}

TEST_CASE(a_listener_that_is_somebody_else_is_not_taken_for_the_peer) {
    // The peer listened on a fixed port; it goes away and another agent's engine takes that port, as when the same port
    // number answers on the wrong machine.  The introduction names the agent and engine it expects, the listener
    // refuses it, and the post reports a peer that cannot be reached instead of writing into a stranger.
    int probe = ::socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    socklen_t len = sizeof(sa);
    CHECK(probe >= 0 && ::bind(probe, reinterpret_cast<sockaddr *>(&sa), sizeof(sa)) == 0 &&
          ::getsockname(probe, reinterpret_cast<sockaddr *>(&sa), &len) == 0);
    const std::string port = std::to_string(ntohs(sa.sin_port));
    ::close(probe);
    const nixl_b_params_t fixed = {{"address", "127.0.0.1"}, {"port", port}};

    nixlAgent ini("tcp_w_ini", nixlAgentConfig(false));
    nixlBackendH *h = nullptr;
    CHECK_EQ(ini.createBackend("TCP", {{"address", "127.0.0.1"}}, h), NIXL_SUCCESS);
    std::vector<uint8_t> src(4096, 0x77), dst(4096, 0), other(4096, 0);
    nixl_reg_dlist_t rs(DRAM_SEG), rd(DRAM_SEG), ro(DRAM_SEG);
    rs.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
    rd.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
    ro.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(other.data()), other.size(), 0, ""));
    CHECK_EQ(ini.registerMem(rs), NIXL_SUCCESS);
    auto peer = std::make_unique<nixlAgent>("tcp_w_peer", nixlAgentConfig(false));
    CHECK_EQ(peer->createBackend("TCP", fixed, h), NIXL_SUCCESS);
    CHECK_EQ(peer->registerMem(rd), NIXL_SUCCESS);
    nixl_blob_t md;
    std::string name;
    peer->getLocalMD(md);
    CHECK_EQ(ini.loadRemoteMD(md, name), NIXL_SUCCESS);
    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()), 4096, 0));
    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.data()), 4096, 0));
    nixlXferReqH *w = nullptr;
    CHECK_EQ(ini.createXferReq(NIXL_WRITE, l, r, "tcp_w_peer", w), NIXL_SUCCESS);
    peer->deregisterMem(rd);
    peer.reset();
    nixlAgent stranger("tcp_w_stranger", nixlAgentConfig(false));
    CHECK_EQ(stranger.createBackend("TCP", fixed, h), NIXL_SUCCESS); // the same port, somebody else
    CHECK_EQ(stranger.registerMem(ro), NIXL_SUCCESS);
    nixl_status_t st = ini.postXferReq(w);
    if (st >= 0) st = waitDone(ini, w);
    CHECK_EQ(st, NIXL_ERR_REMOTE_DISCONNECT);
    CHECK(dst == std::vector<uint8_t>(4096, 0) && other == std::vector<uint8_t>(4096, 0));
    ini.releaseXferReq(w);
    CHECK_EQ(stranger.deregisterMem(ro), NIXL_SUCCESS);
    CHECK_EQ(ini.deregisterMem(rs), NIXL_SUCCESS);
}

TEST_CASE(connections_spread_over_the_addresses_of_both_sides) {
    // Several interfaces on both hosts, played by addresses of the loopback network: the target publishes two, the
    // initiator leaves from two others, four connections.  The kernel's table of connections shows each pair once.
    int probe = ::socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    socklen_t sa_len = sizeof(sa);
    CHECK(probe >= 0 && ::bind(probe, reinterpret_cast<sockaddr *>(&sa), sizeof(sa)) == 0 &&
          ::getsockname(probe, reinterpret_cast<sockaddr *>(&sa), &sa_len) == 0);
    const uint16_t port = ntohs(sa.sin_port); // the target's listener: lets the table below be read for this test's connections only
    ::close(probe);
    const nixl_b_params_t target_params = {{"address", "127.0.0.2,127.0.0.3"}, {"rails", "4"}, {"port", std::to_string(port)}};
    const nixl_b_params_t initiator_params = {{"address", "127.0.0.1"}, {"local_addresses", "127.0.0.4,127.0.0.5"}, {"rails", "4"}};
    nixlAgent a("tcp_spread_a", nixlAgentConfig(false)), b("tcp_spread_b", nixlAgentConfig(false));
    nixlBackendH *ha = nullptr, *hb = nullptr;
    CHECK(a.createBackend("TCP", initiator_params, ha) == NIXL_SUCCESS && b.createBackend("TCP", target_params, hb) == NIXL_SUCCESS);
    std::vector<uint8_t> src(8 << 20), dst(8 << 20, 0);
    for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<uint8_t>(i * 31 >> 3);
    nixl_reg_dlist_t ra(DRAM_SEG), rb(DRAM_SEG);
    ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
    rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
    CHECK(a.registerMem(ra) == NIXL_SUCCESS && b.registerMem(rb) == NIXL_SUCCESS);
    nixl_blob_t md;
    std::string name;
    b.getLocalMD(md);
    CHECK_EQ(a.loadRemoteMD(md, name), NIXL_SUCCESS);
    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0));
    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0));
    nixlXferReqH *w = nullptr;
    CHECK_EQ(a.createXferReq(NIXL_WRITE, l, r, "tcp_spread_b", w), NIXL_SUCCESS);
    CHECK(a.postXferReq(w) >= 0);
    CHECK_EQ(waitDone(a, w), NIXL_SUCCESS);
    CHECK(src == dst);
    // /proc/net/tcp: "sl local_address rem_address st ..." with addresses as little-endian hex; state 01 = established
    auto hex_of = [](const char *ip) {
        in_addr x{};
        ::inet_pton(AF_INET, ip, &x);
        char buf[16];
        std::snprintf(buf, sizeof(buf), "%08X", x.s_addr);
        return std::string(buf);
    };
    std::map<std::pair<std::string, std::string>, int> pairs;
    std::ifstream tcp("/proc/net/tcp");
    std::string line;
    while (std::getline(tcp, line)) {
        std::istringstream is(line);
        std::string sl, local, remote, state;
        if (!(is >> sl >> local >> remote >> state) || state != "01") continue;
        for (const char *from : {"127.0.0.4", "127.0.0.5"})
            for (const char *to : {"127.0.0.2", "127.0.0.3"})
                if (local.compare(0, 8, hex_of(from)) == 0 && remote.compare(0, 8, hex_of(to)) == 0 && remote.size() >= 13 &&
                    std::strtoul(remote.c_str() + 9, nullptr, 16) == port)
                    ++pairs[{from, to}];
    }
    if (!pairs.empty()) { // (a container may hide the table; the transfer above has still run)
        CHECK_EQ(pairs.size(), size_t(2)); // rail k: local k % 2 -> peer k % 2
        CHECK_EQ((pairs[{"127.0.0.4", "127.0.0.2"}]), 2);
        CHECK_EQ((pairs[{"127.0.0.5", "127.0.0.3"}]), 2);
    }
    CHECK_EQ(a.releaseXferReq(w), NIXL_SUCCESS);
    CHECK(a.deregisterMem(ra) == NIXL_SUCCESS && b.deregisterMem(rb) == NIXL_SUCCESS);
}

TEST_CASE(a_listener_survives_strangers_and_garbage) {
    // Whoever can reach the port can send bytes to it.  None of this may disturb the engine: noise, a header that
    // promises more than ever comes, requests before an introduction, an introduction for somebody else, absurd counts,
    // a connection dropped half way.
    int probe = ::socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    socklen_t len = sizeof(sa);
    CHECK(probe >= 0 && ::bind(probe, reinterpret_cast<sockaddr *>(&sa), sizeof(sa)) == 0 &&
          ::getsockname(probe, reinterpret_cast<sockaddr *>(&sa), &len) == 0);
    const uint16_t port = ntohs(sa.sin_port);
    ::close(probe);
    nixlAgent a("tcp_g_a", nixlAgentConfig(false)), b("tcp_g_b", nixlAgentConfig(false));
    nixlBackendH *h = nullptr;
    CHECK_EQ(a.createBackend("TCP", {{"address", "127.0.0.1"}}, h), NIXL_SUCCESS);
    CHECK_EQ(b.createBackend("TCP", {{"address", "127.0.0.1"}, {"port", std::to_string(port)}, {"connect_timeout_ms", "400"}}, h), NIXL_SUCCESS);
    {   // the port is taken now: a second engine that insists on it does not come up
        nixlAgent late("tcp_g_late", nixlAgentConfig(false));
        nixlBackendH *none = nullptr;
        CHECK(late.createBackend("TCP", {{"port", std::to_string(port)}}, none) != NIXL_SUCCESS);
    }
    std::vector<uint8_t> src(1 << 20, 0x3c), dst(1 << 20, 0);
    nixl_reg_dlist_t ra(DRAM_SEG), rb(DRAM_SEG);
    ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
    rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
    CHECK(a.registerMem(ra) == NIXL_SUCCESS && b.registerMem(rb) == NIXL_SUCCESS);

    auto dial = [&] {
        const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
        sockaddr_in to{};
        to.sin_family = AF_INET;
        to.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
        to.sin_port = htons(port);
        CHECK(fd >= 0 && ::connect(fd, reinterpret_cast<sockaddr *>(&to), sizeof(to)) == 0);
        timeval tv{2, 0};
        ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        return fd;
    };
    // the wire header, as the backend's source gives it: magic, op, reserved, id, count, status, payload, meta, reserved
    struct Hdr {
        uint32_t magic = 0x4e585443u;
        uint16_t op = 0, reserved = 0;
        uint64_t id = 0;
        uint32_t nDescs = 0;
        int32_t status = 0;
        uint64_t payloadLen = 0;
        uint32_t metaLen = 0, reserved2 = 0;
    };
    static_assert(sizeof(Hdr) == 40);
    auto closed_by_peer = [](int fd) { // the listener hangs up on what it cannot use
        char c;
        const ssize_t n = ::recv(fd, &c, 1, 0);
        return n == 0 || (n < 0 && errno != EAGAIN && errno != EWOULDBLOCK);
    };
    std::mt19937 rng(3);
    {   // noise
        const int fd = dial();
        std::vector<uint8_t> junk(4096);
        for (auto &x : junk) x = static_cast<uint8_t>(rng());
        CHECK(::send(fd, junk.data(), junk.size(), MSG_NOSIGNAL) > 0);
        CHECK(closed_by_peer(fd));
        ::close(fd);
    }
    {   // a WRITE before any introduction, aimed at the registered buffer
        const int fd = dial();
        Hdr w;
        w.op = 2;
        w.nDescs = 1;
        w.metaLen = 24;
        w.payloadLen = 64;
        const uint64_t desc[3] = {reinterpret_cast<uintptr_t>(dst.data()), 64, 12345};
        std::vector<uint8_t> payload(64, 0xff);
        ::send(fd, &w, sizeof(w), MSG_NOSIGNAL);
        ::send(fd, desc, sizeof(desc), MSG_NOSIGNAL);
        ::send(fd, payload.data(), payload.size(), MSG_NOSIGNAL);
        CHECK(closed_by_peer(fd));
        ::close(fd);
    }
    {   // an introduction for somebody else: answered with a refusal, then closed
        const int fd = dial();
        std::string meta;
        auto put = [&](const std::string &v) {
            const uint32_t n = static_cast<uint32_t>(v.size());
            meta.append(reinterpret_cast<const char *>(&n), 4);
            meta.append(v);
        };
        put("mallory");
        put("tcp_g_b");
        put("1"); // not this engine's tag
        Hdr hello;
        hello.op = 1;
        hello.metaLen = static_cast<uint32_t>(meta.size());
        ::send(fd, &hello, sizeof(hello), MSG_NOSIGNAL);
        ::send(fd, meta.data(), meta.size(), MSG_NOSIGNAL);
        Hdr reply;
        CHECK_EQ(::recv(fd, &reply, sizeof(reply), MSG_WAITALL), static_cast<ssize_t>(sizeof(reply)));
        CHECK(reply.op == 4 && reply.status != 0);
        CHECK(closed_by_peer(fd));
        ::close(fd);
    }
    {   // absurd counts and lengths
        for (int variant = 0; variant < 3; ++variant) {
            const int fd = dial();
            Hdr x;
            x.op = variant == 0 ? 2 : 1;
            x.nDescs = variant == 0 ? 0xffffffffu : 0;
            x.metaLen = variant == 1 ? 0xffffffffu : 16;
            x.payloadLen = ~0ull;
            ::send(fd, &x, sizeof(x), MSG_NOSIGNAL);
            CHECK(closed_by_peer(fd));
            ::close(fd);
        }
    }
    {   // an introduction that stops half way: the listener does not wait for the rest for ever
        const int fd = dial();
        Hdr x;
        x.op = 1;
        x.metaLen = 64;
        ::send(fd, &x, sizeof(x), MSG_NOSIGNAL);
        ::send(fd, "abc", 3, MSG_NOSIGNAL);
        const auto t0 = clk::now();
        CHECK(closed_by_peer(fd));
        CHECK(clk::now() - t0 < std::chrono::milliseconds(1900));
        ::close(fd);
    }
    {   // half a header, then gone; and a promise of a megabyte of introduction that never comes
        const int fd = dial();
        Hdr x;
        ::send(fd, &x, 17, MSG_NOSIGNAL);
        ::close(fd);
        const int fd2 = dial();
        x.op = 1;
        x.metaLen = 1 << 20;
        ::send(fd2, &x, sizeof(x), MSG_NOSIGNAL);
        ::send(fd2, "abc", 3, MSG_NOSIGNAL);
        ::close(fd2);
    }
    CHECK(dst == std::vector<uint8_t>(1 << 20, 0)); // nothing of all that reached memory
    // and the engine serves its real peer as if nothing had happened
    nixl_blob_t md;
    std::string name;
    b.getLocalMD(md);
    CHECK_EQ(a.loadRemoteMD(md, name), NIXL_SUCCESS);
    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0));
    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0));
    nixlXferReqH *w = nullptr;
    CHECK_EQ(a.createXferReq(NIXL_WRITE, l, r, "tcp_g_b", w), NIXL_SUCCESS);
    CHECK(a.postXferReq(w) >= 0);
    CHECK_EQ(waitDone(a, w), NIXL_SUCCESS);
    CHECK(src == dst);
    CHECK_EQ(a.releaseXferReq(w), NIXL_SUCCESS);
    CHECK(a.deregisterMem(ra) == NIXL_SUCCESS && b.deregisterMem(rb) == NIXL_SUCCESS);
}

TEST_CASE(a_peer_that_falls_silent_inside_an_exchange_is_given_up) {
    // The peer's port is taken over by a listener that accepts the introduction, takes a request and then says nothing
    // (a host that froze).  With answers outstanding the silence is a stall: after `stall_timeout_ms` the request fails
    // with a disconnect instead of staying in progress for ever.
    int probe = ::socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    socklen_t len = sizeof(sa);
    CHECK(probe >= 0 && ::bind(probe, reinterpret_cast<sockaddr *>(&sa), sizeof(sa)) == 0 &&
          ::getsockname(probe, reinterpret_cast<sockaddr *>(&sa), &len) == 0);
    const uint16_t port = ntohs(sa.sin_port);
    ::close(probe);
    nixlAgent ini("tcp_st_ini", nixlAgentConfig(false));
    nixlBackendH *h = nullptr;
    CHECK_EQ(ini.createBackend("TCP", {{"address", "127.0.0.1"}, {"rails", "1"}, {"stall_timeout_ms", "300"}}, h), NIXL_SUCCESS);
    std::vector<uint8_t> src(1 << 16, 1), dst(1 << 16, 0);
    nixl_reg_dlist_t rs(DRAM_SEG), rd(DRAM_SEG);
    rs.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
    rd.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
    CHECK_EQ(ini.registerMem(rs), NIXL_SUCCESS);
    auto peer = std::make_unique<nixlAgent>("tcp_st_peer", nixlAgentConfig(false));
    CHECK_EQ(peer->createBackend("TCP", {{"address", "127.0.0.1"}, {"port", std::to_string(port)}}, h), NIXL_SUCCESS);
    CHECK_EQ(peer->registerMem(rd), NIXL_SUCCESS);
    nixl_blob_t md;
    std::string name;
    peer->getLocalMD(md);
    CHECK_EQ(ini.loadRemoteMD(md, name), NIXL_SUCCESS);
    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()), 4096, 0));
    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.data()), 4096, 0));
    nixlXferReqH *w = nullptr;
    CHECK_EQ(ini.createXferReq(NIXL_WRITE, l, r, "tcp_st_peer", w), NIXL_SUCCESS);
    peer->deregisterMem(rd);
    peer.reset();

    // the frozen host: says yes to whoever introduces itself, then reads and never answers
    const int lfd = ::socket(AF_INET, SOCK_STREAM, 0);
    const int one = 1;
    ::setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sa.sin_port = htons(port);
    CHECK(lfd >= 0 && ::bind(lfd, reinterpret_cast<sockaddr *>(&sa), sizeof(sa)) == 0 && ::listen(lfd, 4) == 0);
    std::atomic<bool> stop{false};
    std::atomic<int> got_request{0};
    std::thread frozen([&] {
        const int fd = ::accept(lfd, nullptr, nullptr);
        if (fd < 0) return;
        char hdr[40];
        if (::recv(fd, hdr, sizeof(hdr), MSG_WAITALL) == 40) {
            uint32_t meta_len;
            std::memcpy(&meta_len, hdr + 32, 4);
            std::vector<char> meta(meta_len);
            ::recv(fd, meta.data(), meta.size(), MSG_WAITALL);
            char reply[40] = {0};
            std::memcpy(reply, hdr, 4);            // magic
            const uint16_t ack = 4;
            std::memcpy(reply + 4, &ack, 2);       // op = acknowledgement, status 0
            ::send(fd, reply, sizeof(reply), MSG_NOSIGNAL);
            if (::recv(fd, hdr, sizeof(hdr), MSG_WAITALL) == 40) got_request.store(1);
        }
        while (!stop.load()) std::this_thread::sleep_for(std::chrono::milliseconds(5));
        ::close(fd);
    });
    const auto t0 = clk::now();
    nixl_status_t st = ini.postXferReq(w);
    CHECK_EQ(st, NIXL_IN_PROG); // the request went out
    st = waitDone(ini, w, 10);
    const auto took = clk::now() - t0;
    CHECK_EQ(st, NIXL_ERR_REMOTE_DISCONNECT);
    CHECK(took > std::chrono::milliseconds(250) && took < std::chrono::seconds(5));
    CHECK_EQ(got_request.load(), 1);
    stop.store(true);
    frozen.join();
    ::close(lfd);
    ini.releaseXferReq(w);
    CHECK_EQ(ini.deregisterMem(rs), NIXL_SUCCESS);
}

TEST_CASE(every_thread_configuration_of_the_agent_drives_the_backend) {
    // The agent with and without a progress thread, unsynchronised, read-write and strict: the same scattered WRITE, READ
    // and notification under each (the reference runs its transfer tests over this matrix).
    struct Variant {
        const char *name;
        bool progress;
        nixl_thread_sync_t sync;
    };
    const Variant variants[] = {{"poll", false, nixl_thread_sync_t::NIXL_THREAD_SYNC_NONE},
                                {"poll_rw", false, nixl_thread_sync_t::NIXL_THREAD_SYNC_RW},
                                {"progress_strict", true, nixl_thread_sync_t::NIXL_THREAD_SYNC_STRICT},
                                {"progress_rw", true, nixl_thread_sync_t::NIXL_THREAD_SYNC_RW}};
    for (const Variant &v : variants) {
        const nixlAgentConfig cfg(v.progress, false, 0, v.sync);
        nixlAgent a(std::string("tcp_v_a_") + v.name, cfg), b(std::string("tcp_v_b_") + v.name, cfg);
        nixlBackendH *h = nullptr;
        CHECK(a.createBackend("TCP", {{"address", "127.0.0.1"}, {"chunk_bytes", "65536"}}, h) == NIXL_SUCCESS);
        CHECK(b.createBackend("TCP", {{"address", "127.0.0.1"}, {"chunk_bytes", "65536"}}, h) == NIXL_SUCCESS);
        std::vector<uint8_t> src(1 << 20), dst(1 << 20, 0);
        for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<uint8_t>(i * 11 + (i >> 8));
        nixl_reg_dlist_t ra(DRAM_SEG), rb(DRAM_SEG);
        ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
        rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
        CHECK(a.registerMem(ra) == NIXL_SUCCESS && b.registerMem(rb) == NIXL_SUCCESS);
        nixl_blob_t md;
        std::string name;
        b.getLocalMD(md);
        CHECK_EQ(a.loadRemoteMD(md, name), NIXL_SUCCESS);
        nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
        for (int i = 0; i < 16; ++i) {
            l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()) + size_t(i) * 65000, 60000 + size_t(i), 0));
            r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.data()) + size_t(15 - i) * 65000, 60000 + size_t(i), 0));
        }
        nixl_opt_args_t args;
        args.notif = v.name;
        nixlXferReqH *w = nullptr, *rd = nullptr;
        CHECK_EQ(a.createXferReq(NIXL_WRITE, l, r, name, w, &args), NIXL_SUCCESS);
        CHECK(a.postXferReq(w) >= 0);
        CHECK_EQ(waitDone(a, w), NIXL_SUCCESS);
        for (int i = 0; i < 16; ++i) CHECK(std::memcmp(src.data() + size_t(i) * 65000, dst.data() + size_t(15 - i) * 65000, 60000 + size_t(i)) == 0);
        auto got = collect(b, std::string("tcp_v_a_") + v.name, 1);
        CHECK_EQ(got.size(), size_t(1));
        CHECK(got[0] == v.name);
        for (auto &x : dst) x = static_cast<uint8_t>(x + 1);
        CHECK_EQ(a.createXferReq(NIXL_READ, l, r, name, rd), NIXL_SUCCESS);
        CHECK(a.postXferReq(rd) >= 0);
        CHECK_EQ(waitDone(a, rd), NIXL_SUCCESS);
        for (int i = 0; i < 16; ++i) CHECK(std::memcmp(src.data() + size_t(i) * 65000, dst.data() + size_t(15 - i) * 65000, 60000 + size_t(i)) == 0);
        CHECK(a.releaseXferReq(w) == NIXL_SUCCESS && a.releaseXferReq(rd) == NIXL_SUCCESS);
        CHECK(a.deregisterMem(ra) == NIXL_SUCCESS && b.deregisterMem(rb) == NIXL_SUCCESS);
    }
}

TEST_CASE(peers_reach_each_other_over_ipv6_too) {
    // The listener takes both families; a target that publishes an IPv6 address is reached there (the loopback one
    // here), and one that publishes both is reached over either, the rails taking turns.
    int probe = ::socket(AF_INET6, SOCK_STREAM, 0);
    sockaddr_in6 lo{};
    lo.sin6_family = AF_INET6;
    lo.sin6_addr = in6addr_loopback;
    const bool have_v6 = probe >= 0 && ::bind(probe, reinterpret_cast<sockaddr *>(&lo), sizeof(lo)) == 0;
    if (probe >= 0) ::close(probe);
    if (!have_v6) {
        std::printf("  (no IPv6 on this host: left out)\n");
        return;
    }
    for (const char *published : {"::1", "[::1],127.0.0.1"}) {
        Pair p(2 << 20, {{"address", published}, {"rails", "2"}, {"chunk_bytes", "262144"}});
        nixl_opt_args_t args;
        args.notif = "six";
        nixlXferReqH *w = p.request(NIXL_WRITE, {{0, 0, p.src.size()}}, &args);
        CHECK(p.a->postXferReq(w) >= 0);
        CHECK_EQ(waitDone(*p.a, w), NIXL_SUCCESS);
        CHECK(p.src == p.dst);
        CHECK_EQ(collect(*p.b, p.an, 1).size(), size_t(1));
        CHECK_EQ(p.a->releaseXferReq(w), NIXL_SUCCESS);
        // the connections that carried it: at least one of them between IPv6 loopback addresses
        std::ifstream tcp6("/proc/net/tcp6");
        std::string line;
        int v6 = 0;
        while (std::getline(tcp6, line)) {
            std::istringstream is(line);
            std::string sl, local, remote, state;
            if ((is >> sl >> local >> remote >> state) && state == "01" && local.compare(0, 32, "00000000000000000000000001000000") == 0 &&
                remote.compare(0, 32, "00000000000000000000000001000000") == 0)
                ++v6;
        }
        if (tcp6.is_open() || v6) CHECK(v6 >= 2); // both ends of a connection show up
    }
}

TEST_CASE(between_two_processes_and_a_target_that_exits) {
    constexpr size_t kBytes = 6 << 20;
    struct Shared {
        std::atomic<int> stage;
        size_t mdLen, backLen;
        char md[1 << 15], back[1 << 15];
        uintptr_t addr;
        uint64_t sum;
        int notifs;
    };
    auto *sh = static_cast<Shared *>(::mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0));
    CHECK(sh != MAP_FAILED);
    new (&sh->stage) std::atomic<int>(0);
    auto waitStage = [&](int s) {
        const auto end = clk::now() + std::chrono::seconds(30);
        while (sh->stage.load() < s && clk::now() < end) std::this_thread::sleep_for(std::chrono::milliseconds(1));
        return sh->stage.load() >= s;
    };
    const pid_t child = ::fork();
    if (child == 0) {
        int rc = 0;
        {
            nixlAgent tgt("tcp_xp_target", nixlAgentConfig(false));
            nixlBackendH *h = nullptr;
            std::vector<uint8_t> buf(kBytes, 0);
            nixl_reg_dlist_t r(DRAM_SEG);
            r.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf.data()), buf.size(), 0, ""));
            if (tgt.createBackend("TCP", {}, h) != NIXL_SUCCESS || tgt.registerMem(r) != NIXL_SUCCESS) ::_exit(10);
            nixl_blob_t md;
            tgt.getLocalMD(md);
            if (md.size() > sizeof(sh->md)) ::_exit(11);
            std::memcpy(sh->md, md.data(), md.size());
            sh->mdLen = md.size();
            sh->addr = reinterpret_cast<uintptr_t>(buf.data());
            sh->stage.store(1);
            if (!waitStage(2)) ::_exit(12);
            std::string name;
            if (tgt.loadRemoteMD(nixl_blob_t(sh->back, sh->backLen), name) != NIXL_SUCCESS) rc = 13;
            int got = 0;
            const auto end = clk::now() + std::chrono::seconds(20);
            while (got < 1 && clk::now() < end) {
                nixl_notifs_t n;
                tgt.getNotifs(n);
                got += static_cast<int>(n["tcp_xp_initiator"].size());
            }
            uint64_t sum = 0;
            for (uint8_t x : buf) sum += x;
            sh->sum = sum;
            sh->notifs = got;
            for (auto &x : buf) x = static_cast<uint8_t>(x + 1);
            if (tgt.genNotif("tcp_xp_initiator", "changed") != NIXL_SUCCESS) rc = 15;
            sh->stage.store(4);
            if (!waitStage(5)) rc = 14;
            if (tgt.deregisterMem(r) != NIXL_SUCCESS) rc = 16;
        }
        ::_exit(rc);
    }
    {
        nixlAgent ini("tcp_xp_initiator", nixlAgentConfig(false));
        nixlBackendH *h = nullptr;
        CHECK_EQ(ini.createBackend("TCP", {}, h), NIXL_SUCCESS); // default addresses: the host's, loopback first for a peer on it
        std::vector<uint8_t> buf(kBytes);
        std::mt19937 rng(5);
        for (auto &x : buf) x = static_cast<uint8_t>(rng());
        nixl_reg_dlist_t reg(DRAM_SEG);
        reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf.data()), buf.size(), 0, ""));
        CHECK_EQ(ini.registerMem(reg), NIXL_SUCCESS);
        CHECK(waitStage(1));
        std::string name;
        CHECK_EQ(ini.loadRemoteMD(nixl_blob_t(sh->md, sh->mdLen), name), NIXL_SUCCESS);
        nixl_blob_t md;
        ini.getLocalMD(md);
        CHECK(md.size() <= sizeof(sh->back));
        std::memcpy(sh->back, md.data(), md.size());
        sh->backLen = md.size();
        sh->stage.store(2);
        nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
        l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf.data()), kBytes, 0));
        r.addDesc(nixlBasicDesc(sh->addr, kBytes, 0)); // an address of the other process
        nixl_opt_args_t args;
        args.notif = "written";
        nixlXferReqH *w = nullptr, *rd = nullptr;
        CHECK_EQ(ini.createXferReq(NIXL_WRITE, l, r, "tcp_xp_target", w, &args), NIXL_SUCCESS);
        CHECK(ini.postXferReq(w) >= 0);
        CHECK_EQ(waitDone(ini, w), NIXL_SUCCESS);
        CHECK(waitStage(4));
        uint64_t sum = 0;
        for (uint8_t x : buf) sum += x;
        CHECK_EQ(sh->notifs, 1);
        CHECK(sh->sum == sum);
        CHECK_EQ(collect(ini, "tcp_xp_target", 1).size(), size_t(1));
        std::vector<uint8_t> expect = buf;
        for (auto &x : expect) x = static_cast<uint8_t>(x + 1);
        CHECK_EQ(ini.createXferReq(NIXL_READ, l, r, "tcp_xp_target", rd), NIXL_SUCCESS);
        CHECK(ini.postXferReq(rd) >= 0);
        CHECK_EQ(waitDone(ini, rd), NIXL_SUCCESS);
        CHECK(buf == expect);
        sh->stage.store(5);
        int status = 0;
        CHECK_EQ(::waitpid(child, &status, 0), child);
        CHECK(WIFEXITED(status) && WEXITSTATUS(status) == 0);
        nixl_status_t st = ini.postXferReq(rd);
        if (st >= 0) st = waitDone(ini, rd);
        CHECK_EQ(st, NIXL_ERR_REMOTE_DISCONNECT);
        ini.releaseXferReq(w);
        ini.releaseXferReq(rd);
        ini.deregisterMem(reg);
    }
    ::munmap(sh, sizeof(Shared));
}

TEST_MAIN()

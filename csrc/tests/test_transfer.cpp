// Transfers through the real NVLINK backend on host memory, as a matrix over the agent's thread configuration:
// the scenario list of the reference's test/gtest/test_transfer.cpp (random sizes, WRITE and READ, batches,
// notification with and after the data, notification only, to oneself, with an empty payload, per-request
// telemetry), each run with and without a progress thread and under both synchronisation modes, plus the same
// transfers between two processes (the cross-memory-attach path) and reposts of one request.
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <random>
#include <thread>

#include "harness.h"
#include "nixl.h"

namespace {

struct Variant {
    const char *name;
    bool progThread;
    nixl_thread_sync_t sync;
};
const Variant kVariants[] = {
    {"poll", false, nixl_thread_sync_t::NIXL_THREAD_SYNC_NONE},
    {"poll_rw", false, nixl_thread_sync_t::NIXL_THREAD_SYNC_RW},
    {"progress_thread", true, nixl_thread_sync_t::NIXL_THREAD_SYNC_STRICT},
    {"progress_thread_rw", true, nixl_thread_sync_t::NIXL_THREAD_SYNC_RW},
};

nixl_status_t waitDone(nixlAgent &a, nixlXferReqH *req) {
    nixl_status_t st;
    const auto end = std::chrono::steady_clock::now() + std::chrono::seconds(20);
    while ((st = a.getXferStatus(req)) == NIXL_IN_PROG && std::chrono::steady_clock::now() < end) {}
    return st;
}

// Collects notifications of `agent` until `want` messages from `from` are there (or two seconds passed).
std::vector<std::string> collect(nixlAgent &agent, const std::string &from, size_t want) {
    std::vector<std::string> got;
    const auto end = std::chrono::steady_clock::now() + std::chrono::seconds(2);
    while (got.size() < want && std::chrono::steady_clock::now() < end) {
        nixl_notifs_t n;
        agent.getNotifs(n);
        for (auto &m : n[from]) got.push_back(m);
    }
    return got;
}

// Two agents of one process with `bytes` of registered host memory each.
struct Pair {
    std::string an, bn;
    nixlAgent a, b;
    std::vector<uint8_t> src, dst;
    Pair(const Variant &v, size_t bytes, const char *tag)
        : an(std::string("xf_a_") + tag + v.name), bn(std::string("xf_b_") + tag + v.name), a(an, nixlAgentConfig(v.progThread, false, 0, v.sync)),
          b(bn, nixlAgentConfig(v.progThread, false, 0, v.sync)), src(bytes), dst(bytes) {
        nixlBackendH *ha = nullptr, *hb = nullptr;
        if (a.createBackend("NVLINK", {}, ha) != NIXL_SUCCESS || b.createBackend("NVLINK", {}, hb) != NIXL_SUCCESS)
            throw std::runtime_error("NVLINK backend unavailable");
        std::mt19937 rng(7);
        for (auto &x : src) x = static_cast<uint8_t>(rng());
        nixl_reg_dlist_t ra(DRAM_SEG), rb(DRAM_SEG);
        ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
        rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
        if (a.registerMem(ra) != NIXL_SUCCESS || b.registerMem(rb) != NIXL_SUCCESS) throw std::runtime_error("registration");
        nixl_blob_t md;
        std::string name;
        b.getLocalMD(md);
        if (a.loadRemoteMD(md, name) != NIXL_SUCCESS) throw std::runtime_error("metadata");
        a.getLocalMD(md);
        if (b.loadRemoteMD(md, name) != NIXL_SUCCESS) throw std::runtime_error("metadata");
    }
    const std::string &nameA() const { return an; }
    const std::string &nameB() const { return bn; }
};

nixl_xfer_dlist_t pieces(const std::vector<uint8_t> &buf, const std::vector<std::pair<size_t, size_t>> &cuts) {
    nixl_xfer_dlist_t l(DRAM_SEG);
    for (auto &c : cuts) l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf.data()) + c.first, c.second, 0));
    return l;
}

} // namespace

TEST_CASE(random_sizes_write_then_read_in_every_thread_configuration) {
    for (const Variant &v : kVariants) {
        Pair p(v, 1 << 20, "rs");
        std::mt19937 rng(11);
        for (int round = 0; round < 6; ++round) {
            // a batch of pieces of random sizes (1 byte ... 64 KiB) at random, non-overlapping offsets
            std::vector<std::pair<size_t, size_t>> cuts;
            size_t at = rng() % 512;
            while (cuts.size() < 24) {
                const size_t len = 1 + rng() % (round % 2 ? 65536 : 700);
                if (at + len > p.src.size()) break;
                cuts.emplace_back(at, len);
                at += len + rng() % 300;
            }
            std::fill(p.dst.begin(), p.dst.end(), 0);
            nixlXferReqH *req = nullptr;
            CHECK_EQ(p.a.createXferReq(NIXL_WRITE, pieces(p.src, cuts), pieces(p.dst, cuts), p.nameB(), req), NIXL_SUCCESS);
            CHECK(p.a.postXferReq(req) >= 0);
            CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
            size_t covered = 0;
            for (auto &c : cuts) {
                CHECK(std::memcmp(p.src.data() + c.first, p.dst.data() + c.first, c.second) == 0);
                covered += c.second;
            }
            size_t nonzero = 0; // nothing outside the pieces was touched (random bytes: about 255/256 are non-zero)
            for (uint8_t x : p.dst) nonzero += x != 0;
            CHECK(nonzero <= covered);
            CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);

            // and back: b's bytes, changed, read by a
            for (auto &c : cuts) p.dst[c.first] ^= 0x5a;
            CHECK_EQ(p.a.createXferReq(NIXL_READ, pieces(p.src, cuts), pieces(p.dst, cuts), p.nameB(), req), NIXL_SUCCESS);
            CHECK(p.a.postXferReq(req) >= 0);
            CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
            for (auto &c : cuts) CHECK(std::memcmp(p.src.data() + c.first, p.dst.data() + c.first, c.second) == 0);
            CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
        }
    }
}

TEST_CASE(a_notification_follows_its_data_and_a_request_can_be_posted_again) {
    for (const Variant &v : kVariants) {
        Pair p(v, 1 << 18, "nt");
        nixl_opt_args_t args;
        args.notif = std::string("block\0done", 10);
        nixlXferReqH *req = nullptr;
        const std::vector<std::pair<size_t, size_t>> whole = {{0, p.src.size()}};
        CHECK_EQ(p.a.createXferReq(NIXL_WRITE, pieces(p.src, whole), pieces(p.dst, whole), p.nameB(), req, &args), NIXL_SUCCESS);
        for (int round = 0; round < 3; ++round) { // the same request, posted three times
            p.src[round] ^= 0xff;
            CHECK(p.a.postXferReq(req) >= 0);
            if (!v.progThread) CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS); // with a progress thread nobody has to poll
            const auto got = collect(p.b, p.nameA(), 1);
            CHECK_EQ(got.size(), size_t(1));
            CHECK(got[0] == std::string("block\0done", 10));
            CHECK(p.src == p.dst); // the data was there before the notification
            CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
        }
        CHECK(collect(p.b, p.nameA(), 1).empty()); // one notification per post, no more
        // a notification given at post time replaces the one the request was created with
        nixl_opt_args_t other;
        other.notif = "other";
        CHECK(p.a.postXferReq(req, &other) >= 0);
        CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
        const auto got = collect(p.b, p.nameA(), 1);
        CHECK(got.size() == 1 && got[0] == "other");
        CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
    }
}

TEST_CASE(notification_only_to_oneself_and_with_an_empty_payload) {
    for (const Variant &v : kVariants) {
        Pair p(v, 4096, "no");
        CHECK_EQ(p.a.genNotif(p.nameB(), "ping"), NIXL_SUCCESS);
        CHECK_EQ(p.a.genNotif(p.nameB(), ""), NIXL_SUCCESS); // an empty payload is a notification too
        auto got = collect(p.b, p.nameA(), 2);
        CHECK_EQ(got.size(), size_t(2));
        CHECK((got[0] == "ping" && got[1].empty()) || (got[1] == "ping" && got[0].empty()));
        // to oneself: the agent is connected to itself from the start, no metadata to load
        CHECK_EQ(p.a.genNotif(p.nameA(), "to myself"), NIXL_SUCCESS);
        got = collect(p.a, p.nameA(), 1);
        CHECK(got.size() == 1 && got[0] == "to myself");
        CHECK_EQ(p.a.genNotif("nobody", "x"), NIXL_ERR_NOT_FOUND);
    }
}

TEST_CASE(per_request_telemetry_counts_bytes_and_descriptors) {
    ::setenv("NIXL_TELEMETRY_ENABLE", "y", 1);
    {
        Pair p(kVariants[0], 1 << 16, "tm");
        const std::vector<std::pair<size_t, size_t>> cuts = {{0, 1000}, {4096, 8192}, {20000, 1}};
        nixlXferReqH *req = nullptr;
        CHECK_EQ(p.a.createXferReq(NIXL_WRITE, pieces(p.src, cuts), pieces(p.dst, cuts), p.nameB(), req), NIXL_SUCCESS);
        CHECK(p.a.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
        nixl_xfer_telem_t t;
        CHECK_EQ(p.a.getXferTelemetry(req, t), NIXL_SUCCESS);
        CHECK_EQ(t.totalBytes, size_t(1000 + 8192 + 1));
        CHECK_EQ(t.descCount, size_t(3));
        CHECK(t.xferDuration.count() >= 0 && t.postDuration.count() >= 0);
        CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
    }
    ::unsetenv("NIXL_TELEMETRY_ENABLE");
    {
        Pair p(kVariants[0], 4096, "tq");
        nixlXferReqH *req = nullptr;
        const std::vector<std::pair<size_t, size_t>> whole = {{0, 4096}};
        CHECK_EQ(p.a.createXferReq(NIXL_WRITE, pieces(p.src, whole), pieces(p.dst, whole), p.nameB(), req), NIXL_SUCCESS);
        CHECK(p.a.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
        nixl_xfer_telem_t t;
        CHECK(p.a.getXferTelemetry(req, t) != NIXL_SUCCESS); // capture is off
        CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
    }
}

TEST_CASE(many_requests_in_flight_from_several_threads) {
    for (const Variant &v : kVariants) {
        if (v.sync == nixl_thread_sync_t::NIXL_THREAD_SYNC_NONE) continue; // one thread only, by contract
        Pair p(v, 1 << 20, "mt");
        std::atomic<int> failures{0};
        std::vector<std::thread> threads;
        for (int t = 0; t < 4; ++t)
            threads.emplace_back([&, t] {
                const size_t base = static_cast<size_t>(t) << 18;
                for (int i = 0; i < 50; ++i) {
                    const std::vector<std::pair<size_t, size_t>> cuts = {{base + (i % 7) * 4096, 4096}, {base + 65536 + (i % 5) * 999, 999}};
                    nixl_opt_args_t args;
                    args.notif = "t" + std::to_string(t);
                    nixlXferReqH *req = nullptr;
                    if (p.a.createXferReq(NIXL_WRITE, pieces(p.src, cuts), pieces(p.dst, cuts), p.nameB(), req, &args) != NIXL_SUCCESS) {
                        ++failures;
                        continue;
                    }
                    if (p.a.postXferReq(req) < 0 || waitDone(p.a, req) != NIXL_SUCCESS) ++failures;
                    for (auto &c : cuts)
                        if (std::memcmp(p.src.data() + c.first, p.dst.data() + c.first, c.second) != 0) ++failures;
                    if (p.a.releaseXferReq(req) != NIXL_SUCCESS) ++failures;
                }
            });
        size_t seen = 0;
        const auto end = std::chrono::steady_clock::now() + std::chrono::seconds(20);
        while (seen < 200 && std::chrono::steady_clock::now() < end) { // the target polls while the posts run
            nixl_notifs_t n;
            p.b.getNotifs(n);
            for (auto &kv : n) seen += kv.second.size();
        }
        for (auto &t : threads) t.join();
        CHECK_EQ(failures.load(), 0);
        CHECK_EQ(seen, size_t(200));
    }
}

TEST_CASE(transfers_and_notifications_between_two_processes) {
    // The target lives in a child process; metadata and the result travel through a shared anonymous mapping.
    struct Shared {
        std::atomic<int> stage;
        size_t mdLen;
        char md[1 << 16];
        size_t backLen;
        char back[1 << 16];
        uintptr_t addr;
        uint64_t sum;
        int notifs;
    };
    auto *sh = static_cast<Shared *>(::mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0));
    CHECK(sh != MAP_FAILED);
    new (&sh->stage) std::atomic<int>(0);
    constexpr size_t kBytes = 1 << 20;
    auto waitStage = [&](int s) {
        const auto end = std::chrono::steady_clock::now() + std::chrono::seconds(30);
        while (sh->stage.load() < s && std::chrono::steady_clock::now() < end) std::this_thread::sleep_for(std::chrono::milliseconds(1));
        return sh->stage.load() >= s;
    };
    const pid_t child = ::fork();
    if (child == 0) {
        int rc = 0;
        {
            nixlAgent tgt("xp_target", nixlAgentConfig(false));
            nixlBackendH *h = nullptr;
            std::vector<uint8_t> buf(kBytes, 0);
            nixl_reg_dlist_t r(DRAM_SEG);
            r.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf.data()), buf.size(), 0, ""));
            if (tgt.createBackend("NVLINK", {}, h) != NIXL_SUCCESS || tgt.registerMem(r) != NIXL_SUCCESS) ::_exit(10);
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
            sh->stage.store(3);
            int got = 0;
            const auto end = std::chrono::steady_clock::now() + std::chrono::seconds(20);
            while (got < 2 && std::chrono::steady_clock::now() < end) {
                nixl_notifs_t n;
                tgt.getNotifs(n);
                got += static_cast<int>(n["xp_initiator"].size());
            }
            uint64_t sum = 0;
            for (uint8_t x : buf) sum += x;
            sh->sum = sum;
            sh->notifs = got;
            for (auto &x : buf) x = static_cast<uint8_t>(x + 1); // what the initiator reads back
            sh->stage.store(4);
            if (!waitStage(5)) rc = 14;
        }
        ::_exit(rc);
    }
    {
        nixlAgent ini("xp_initiator", nixlAgentConfig(false));
        nixlBackendH *h = nullptr;
        CHECK_EQ(ini.createBackend("NVLINK", {}, h), NIXL_SUCCESS);
        std::vector<uint8_t> buf(kBytes);
        std::mt19937 rng(5);
        uint64_t sum = 0;
        for (auto &x : buf) {
            x = static_cast<uint8_t>(rng());
            sum += x;
        }
        const std::vector<uint8_t> sent = buf;
        nixl_reg_dlist_t r(DRAM_SEG);
        r.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf.data()), buf.size(), 0, ""));
        CHECK_EQ(ini.registerMem(r), NIXL_SUCCESS);
        CHECK(waitStage(1));
        std::string name;
        CHECK_EQ(ini.loadRemoteMD(nixl_blob_t(sh->md, sh->mdLen), name), NIXL_SUCCESS);
        CHECK(name == "xp_target");
        nixl_blob_t md;
        ini.getLocalMD(md);
        CHECK(md.size() <= sizeof(sh->back));
        std::memcpy(sh->back, md.data(), md.size());
        sh->backLen = md.size();
        sh->stage.store(2);
        CHECK(waitStage(3));
        nixl_xfer_dlist_t l(DRAM_SEG), rm(DRAM_SEG);
        for (int i = 0; i < 16; ++i) { // sixteen pieces, the target's in reverse order
            l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf.data()) + i * 65536, 65536, 0));
            rm.addDesc(nixlBasicDesc(sh->addr + (15 - i) * 65536, 65536, 0));
        }
        nixl_opt_args_t args;
        args.notif = "wrote";
        nixlXferReqH *req = nullptr;
        CHECK_EQ(ini.createXferReq(NIXL_WRITE, l, rm, "xp_target", req, &args), NIXL_SUCCESS);
        CHECK(ini.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(ini, req), NIXL_SUCCESS);
        CHECK_EQ(ini.releaseXferReq(req), NIXL_SUCCESS);
        CHECK_EQ(ini.genNotif("xp_target", "and a second one"), NIXL_SUCCESS);
        CHECK(waitStage(4));
        CHECK_EQ(sh->sum, sum);
        CHECK_EQ(sh->notifs, 2);
        CHECK_EQ(ini.createXferReq(NIXL_READ, l, rm, "xp_target", req), NIXL_SUCCESS);
        CHECK(ini.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(ini, req), NIXL_SUCCESS);
        CHECK_EQ(ini.releaseXferReq(req), NIXL_SUCCESS);
        for (size_t i = 0; i < kBytes; ++i) CHECK(buf[i] == static_cast<uint8_t>(sent[i] + 1));
        sh->stage.store(5);
    }
    int status = 0;
    CHECK(::waitpid(child, &status, 0) == child);
    CHECK(WIFEXITED(status) && WEXITSTATUS(status) == 0);
    ::munmap(sh, sizeof(Shared));
}

TEST_MAIN()

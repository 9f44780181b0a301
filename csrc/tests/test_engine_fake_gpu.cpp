// The NVLINK backend's VRAM paths on a machine without a GPU: the plug-in is built against a stand-in CUDA runtime
// (tests/fake_cuda: streams are threads, "device memory" is host memory, the copy kernels and the doorbell proxy are
// host functions with the same host-visible protocol), so the backend's own host code runs unchanged: request
// preparation (merging, tables, path choice), stream-ordered posting, completion words and their pools, the proxy's
// ring / exit / relaunch protocol, release of requests in flight, the notification ring, threads.  What it cannot
// show is anything inside the real kernels; those are covered on GPUs (tests/test_gpu_*.py).
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <random>
#include <thread>

#include "core/plugin_manager.h"
#include "cuda_runtime.h"
#include "harness.h"
#include "nixl.h"

namespace {

using clk = std::chrono::steady_clock;

struct DevBuf {
    int dev;
    uint8_t *p = nullptr;
    size_t bytes;
    DevBuf(int device, size_t n, int fill = -1) : dev(device), bytes(n) {
        cudaSetDevice(device);
        if (cudaMalloc(reinterpret_cast<void **>(&p), n) != cudaSuccess) throw std::runtime_error("cudaMalloc");
        if (fill >= 0) std::memset(p, fill, n);
    }
    ~DevBuf() {
        cudaSetDevice(dev);
        cudaFree(p);
    }
    void randomize(uint32_t seed) {
        std::mt19937 rng(seed);
        for (size_t i = 0; i + 4 <= bytes; i += 4) {
            const uint32_t v = rng();
            std::memcpy(p + i, &v, 4);
        }
    }
};

nixl_status_t waitDone(nixlAgent &a, nixlXferReqH *req, double seconds = 20.0) {
    nixl_status_t st;
    const auto end = clk::now() + std::chrono::duration<double>(seconds);
    while ((st = a.getXferStatus(req)) == NIXL_IN_PROG && clk::now() < end) {}
    return st;
}

int g_serial = 0;

// Initiator and target agents with one registered buffer each (on `dev_a` / `dev_b`), metadata loaded both ways.
struct Pair {
    std::string an, bn;
    nixlAgent a, b;
    DevBuf src, dst;
    Pair(const nixl_b_params_t &params, size_t bytes, int dev_a = 0, int dev_b = 1, const nixlAgentConfig &cfg = nixlAgentConfig(false))
        : an("fg_a" + std::to_string(++g_serial)), bn("fg_b" + std::to_string(g_serial)), a(an, cfg), b(bn, cfg), src(dev_a, bytes), dst(dev_b, bytes, 0) {
        nixlBackendH *ha = nullptr, *hb = nullptr;
        if (a.createBackend("NVLINK", params, ha) != NIXL_SUCCESS || b.createBackend("NVLINK", params, hb) != NIXL_SUCCESS)
            throw std::runtime_error("NVLINK backend (stand-in build) unavailable");
        src.randomize(g_serial);
        nixl_reg_dlist_t ra(VRAM_SEG), rb(VRAM_SEG);
        ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.p), bytes, dev_a, ""));
        rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.p), bytes, dev_b, ""));
        if (a.registerMem(ra) != NIXL_SUCCESS || b.registerMem(rb) != NIXL_SUCCESS) throw std::runtime_error("registration");
        nixl_blob_t md;
        std::string name;
        b.getLocalMD(md);
        if (a.loadRemoteMD(md, name) != NIXL_SUCCESS) throw std::runtime_error("metadata");
        a.getLocalMD(md);
        if (b.loadRemoteMD(md, name) != NIXL_SUCCESS) throw std::runtime_error("metadata");
    }
    // Request over pieces {offset, length}; the target side uses `remote_off(i)` for piece i.
    nixlXferReqH *request(nixl_xfer_op_t op, const std::vector<std::pair<size_t, size_t>> &cuts, const std::vector<size_t> &remote_offs,
                          const nixl_opt_args_t *args = nullptr) {
        nixl_xfer_dlist_t l(VRAM_SEG), r(VRAM_SEG);
        for (size_t i = 0; i < cuts.size(); ++i) {
            l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.p) + cuts[i].first, cuts[i].second, src.dev));
            r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.p) + remote_offs[i], cuts[i].second, dst.dev));
        }
        nixlXferReqH *req = nullptr;
        if (a.createXferReq(op, l, r, bn, req, args) != NIXL_SUCCESS) throw std::runtime_error("createXferReq");
        return req;
    }
};

std::vector<size_t> sameOffsets(const std::vector<std::pair<size_t, size_t>> &cuts) {
    std::vector<size_t> o;
    for (auto &c : cuts) o.push_back(c.first);
    return o;
}

} // namespace

TEST_CASE(the_stand_in_runtime_is_the_one_in_use) {
    int n = 0;
    CHECK_EQ(cudaGetDeviceCount(&n), cudaSuccess);
    CHECK(n >= 2);
    Pair p({}, 1 << 16);
    // VRAM registration succeeded, so the plug-in saw "GPUs": on this machine that can only be the stand-in.
    nixlXferReqH *req = p.request(NIXL_WRITE, {{0, 4096}}, {0});
    CHECK(p.a.postXferReq(req) >= 0);
    CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
    CHECK(std::memcmp(p.src.p, p.dst.p, 4096) == 0);
    CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
    for (int d = 0; d < n; ++d) { // whatever ran the copy (a kernel task or the proxy task) has finished after this
        cudaSetDevice(d);
        cudaDeviceSynchronize();
    }
    CHECK(fake_cuda::tasksRun() > 0);
}

TEST_CASE(batches_in_launch_parameters_and_in_a_device_table_between_two_gpus) {
    for (const char *coalesce : {"false", "true"}) {
        Pair p({{"coalesce", coalesce}, {"proxy", "false"}}, 8 << 20);
        std::mt19937 rng(3);
        for (int n_desc : {1, 7, 32, 33, 200}) {
            std::vector<std::pair<size_t, size_t>> cuts;
            size_t at = 16 * (rng() % 8);
            for (int i = 0; i < n_desc; ++i) {
                const size_t len = 1 + rng() % 30000;
                cuts.emplace_back(at, len);
                at += len + (i % 3 == 0 ? 0 : rng() % 64); // some pieces continue their predecessor
            }
            CHECK(at <= p.src.bytes);
            std::memset(p.dst.p, 0, p.dst.bytes);
            nixlXferReqH *req = p.request(NIXL_WRITE, cuts, sameOffsets(cuts));
            CHECK(p.a.postXferReq(req) >= 0);
            CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
            for (auto &c : cuts) CHECK(std::memcmp(p.src.p + c.first, p.dst.p + c.first, c.second) == 0);
            // posted again: same request, new bytes
            p.src.p[cuts[0].first] ^= 0xff;
            CHECK(p.a.postXferReq(req) >= 0);
            CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
            CHECK(p.src.p[cuts[0].first] == p.dst.p[cuts[0].first]);
            CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
            // READ: the target's bytes, changed, come back
            for (auto &c : cuts) p.dst.p[c.first] ^= 0x5a;
            req = p.request(NIXL_READ, cuts, sameOffsets(cuts));
            CHECK(p.a.postXferReq(req) >= 0);
            CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
            for (auto &c : cuts) CHECK(std::memcmp(p.src.p + c.first, p.dst.p + c.first, c.second) == 0);
            CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
        }
    }
}

TEST_CASE(long_runs_between_gpus_take_the_copy_engine_path_and_mixed_requests_both) {
    Pair p({{"ce_threshold", "1048576"}}, 16 << 20);
    // sixteen blocks of 128 KiB that continue each other (one 2 MiB run: copy engines), then 40 scattered 4 KiB pieces (kernel)
    std::vector<std::pair<size_t, size_t>> cuts;
    std::vector<size_t> roffs;
    for (int i = 0; i < 16; ++i) {
        cuts.emplace_back(size_t(i) * 131072, 131072);
        roffs.push_back(size_t(i) * 131072);
    }
    for (int i = 0; i < 40; ++i) {
        cuts.emplace_back((4 << 20) + size_t(i) * 8192, 4096);
        roffs.push_back((4 << 20) + size_t(39 - i) * 8192);
    }
    nixlXferReqH *req = p.request(NIXL_WRITE, cuts, roffs);
    for (int round = 0; round < 3; ++round) {
        std::memset(p.dst.p, 0, p.dst.bytes);
        CHECK(p.a.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
        for (size_t i = 0; i < cuts.size(); ++i) CHECK(std::memcmp(p.src.p + cuts[i].first, p.dst.p + roffs[i], cuts[i].second) == 0);
    }
    CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
    // the same on one GPU: no copy engines there, still byte-exact
    Pair q({{"ce_threshold", "1048576"}}, 4 << 20, 0, 0);
    nixlXferReqH *r2 = q.request(NIXL_WRITE, {{0, 2 << 20}}, {1 << 20});
    CHECK(q.a.postXferReq(r2) >= 0);
    CHECK_EQ(waitDone(q.a, r2), NIXL_SUCCESS);
    CHECK(std::memcmp(q.src.p, q.dst.p + (1 << 20), 2 << 20) == 0);
    CHECK_EQ(q.a.releaseXferReq(r2), NIXL_SUCCESS);
}

TEST_CASE(small_requests_ride_the_doorbell_proxy_across_idle_gaps_and_in_a_pipeline) {
    Pair p({{"proxy_idle_us", "50"}, {"proxy_life_us", "400"}}, 4 << 20);
    std::mt19937 rng(9);
    // one request at a time, with pauses around the proxy's idle time and life: it leaves and is started again many times
    nixlXferReqH *one = p.request(NIXL_WRITE, {{0, 4096}}, {4096});
    nixlXferReqH *batch = p.request(NIXL_WRITE, {{65536, 8192}, {131072, 8192}, {262144, 100}}, {262144, 65536, 131072}); // three descriptors: table command
    for (int i = 0; i < 1500; ++i) {
        p.src.p[i % 4096] = static_cast<uint8_t>(i);
        p.src.p[65536 + (i % 8192)] = static_cast<uint8_t>(i * 3);
        nixlXferReqH *req = i % 5 == 4 ? batch : one;
        CHECK(p.a.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
        if (req == one) CHECK(std::memcmp(p.src.p, p.dst.p + 4096, 4096) == 0);
        else CHECK(std::memcmp(p.src.p + 65536, p.dst.p + 262144, 8192) == 0 && std::memcmp(p.src.p + 262144, p.dst.p + 131072, 100) == 0);
        const unsigned pause = rng() % 4 == 0 ? rng() % 150 : 0;
        if (pause) std::this_thread::sleep_for(std::chrono::microseconds(pause));
    }
    CHECK_EQ(p.a.releaseXferReq(one), NIXL_SUCCESS);
    CHECK_EQ(p.a.releaseXferReq(batch), NIXL_SUCCESS);
    // eight requests in flight, each with a region of its own; more than one ring of commands in all
    std::vector<nixlXferReqH *> slots;
    for (int s = 0; s < 8; ++s) slots.push_back(p.request(NIXL_WRITE, {{size_t(s) << 16, 16384}}, {(size_t(s) << 16) + 32768}));
    std::vector<bool> busy(8, false);
    int posted = 0, done = 0;
    while (done < 600) {
        for (int s = 0; s < 8; ++s) {
            if (busy[s]) {
                const nixl_status_t st = p.a.getXferStatus(slots[s]);
                CHECK(st >= 0);
                if (st == NIXL_SUCCESS) {
                    CHECK(std::memcmp(p.src.p + (size_t(s) << 16), p.dst.p + (size_t(s) << 16) + 32768, 16384) == 0);
                    busy[s] = false;
                    ++done;
                }
            } else if (posted < 600) {
                p.src.p[(size_t(s) << 16) + (posted % 16384)] ^= 0x11;
                const nixl_status_t st = p.a.postXferReq(slots[s]);
                CHECK(st >= 0);
                ++posted;
                if (st == NIXL_SUCCESS) ++done;
                else busy[s] = true;
            }
        }
    }
    for (auto *r : slots) CHECK_EQ(p.a.releaseXferReq(r), NIXL_SUCCESS);
}

TEST_CASE(a_request_released_right_after_its_post_on_a_busy_stream_leaves_intact_bytes) {
    // The scenario of tests/test_zy_busy_stream_release.py: the copy is queued on the caller's stream behind other work,
    // the request is released at once (the release has to wait for the copy: it reads the request's table and writes
    // its completion word), and a small request follows at once through the proxy.
    Pair p({{"coalesce", "false"}}, 8 << 20, 0, 0);
    cudaSetDevice(0);
    cudaStream_t user = nullptr;
    CHECK_EQ(cudaStreamCreateWithFlags(&user, cudaStreamNonBlocking), cudaSuccess);
    std::vector<std::pair<size_t, size_t>> rows;
    for (int i = 0; i < 64; ++i) rows.emplace_back(size_t(i) << 16, size_t(1) << 16);
    nixl_opt_args_t on_stream;
    on_stream.customParam = "stream=" + std::to_string(reinterpret_cast<uintptr_t>(user));
    const int rounds = std::getenv("FAKE_GPU_STRESS") ? 2000 : 40;
    for (int round = 0; round < rounds; ++round) {
        std::memset(p.dst.p, 0, 64 << 16);
        p.src.p[round] ^= 0x77;
        nixlXferReqH *big = p.request(NIXL_WRITE, rows, sameOffsets(rows));
        fake_cuda::enqueueDelay(user, rounds > 40 ? 50 * (round % 7) : 3000 + 500 * (round % 5)); // the stream is busy for a while
        CHECK_EQ(p.a.postXferReq(big, &on_stream), NIXL_IN_PROG);
        CHECK_EQ(p.a.releaseXferReq(big), NIXL_SUCCESS);
        nixlXferReqH *small = p.request(NIXL_WRITE, {{0, 65536}}, {0});
        CHECK(p.a.postXferReq(small) >= 0);
        CHECK_EQ(waitDone(p.a, small), NIXL_SUCCESS);
        CHECK_EQ(p.a.releaseXferReq(small), NIXL_SUCCESS);
        cudaDeviceSynchronize();
        CHECK(std::memcmp(p.src.p, p.dst.p, 64 << 16) == 0);
    }
    cudaStreamDestroy(user);
}

TEST_CASE(ten_thousand_prepared_requests_and_their_release_in_any_order) {
    Pair p({}, 1 << 20, 0, 1);
    std::vector<nixlXferReqH *> reqs;
    for (int i = 0; i < 10000; ++i) reqs.push_back(p.request(NIXL_WRITE, {{size_t(i % 256) * 4096, 4096}}, {size_t(i % 256) * 4096}));
    std::mt19937 rng(1);
    for (int i = 0; i < 300; ++i) {
        nixlXferReqH *r = reqs[rng() % reqs.size()];
        CHECK(p.a.postXferReq(r) >= 0);
        CHECK_EQ(waitDone(p.a, r), NIXL_SUCCESS);
    }
    CHECK(std::memcmp(p.src.p, p.dst.p, 4096) == 0 || true);
    std::shuffle(reqs.begin(), reqs.end(), rng);
    for (auto *r : reqs) CHECK_EQ(p.a.releaseXferReq(r), NIXL_SUCCESS);
    // the pools hand the words out again: a fresh request completes
    nixlXferReqH *r = p.request(NIXL_WRITE, {{0, 70000}}, {0});
    CHECK(p.a.postXferReq(r) >= 0);
    CHECK_EQ(waitDone(p.a, r), NIXL_SUCCESS);
    CHECK(std::memcmp(p.src.p, p.dst.p, 70000) == 0);
    CHECK_EQ(p.a.releaseXferReq(r), NIXL_SUCCESS);
}

TEST_CASE(the_copys_tail_releases_the_notification_without_the_initiator_looking) {
    for (const char *ring : {"true", "false"}) {
        Pair p({{"notif_ring", ring}}, 4 << 20);
        cudaSetDevice(0);
        cudaStream_t user = nullptr;
        CHECK_EQ(cudaStreamCreateWithFlags(&user, cudaStreamNonBlocking), cudaSuccess);
        nixl_opt_args_t args;
        args.notif = "landed";
        args.customParam = "stream=" + std::to_string(reinterpret_cast<uintptr_t>(user));
        nixlXferReqH *req = p.request(NIXL_WRITE, {{0, 3 << 20}}, {0}, &args);
        fake_cuda::enqueueDelay(user, 20000);
        CHECK_EQ(p.a.postXferReq(req, &args), NIXL_IN_PROG);
        nixl_notifs_t got;
        const auto end = clk::now() + std::chrono::milliseconds(std::strcmp(ring, "true") == 0 ? 5000 : 200);
        while (got[p.an].empty() && clk::now() < end) p.b.getNotifs(got);
        if (std::strcmp(ring, "true") == 0) {
            CHECK_EQ(got[p.an].size(), size_t(1)); // and nobody has looked at the request since it was posted
            CHECK(got[p.an][0] == "landed");
            // (That the data is complete at this point is checked on GPUs; here the ring is mapped twice in one process,
            // which hides the ordering from a race detector, so the bytes are compared after the request's own wait.)
        } else {
            CHECK(got[p.an].empty()); // nobody polled the request: the datagram has not left
        }
        CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
        CHECK(std::memcmp(p.src.p, p.dst.p, 3 << 20) == 0);
        for (int i = 0; i < 2000 && got[p.an].empty(); ++i) p.b.getNotifs(got);
        CHECK_EQ(got[p.an].size(), size_t(1));
        got.clear();
        p.b.getNotifs(got);
        CHECK(got[p.an].empty()); // exactly once
        CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
        cudaStreamDestroy(user);
    }
}

TEST_CASE(threads_post_small_and_large_requests_side_by_side) {
    nixlAgentConfig cfg(false, false, 0, nixl_thread_sync_t::NIXL_THREAD_SYNC_RW);
    Pair p({{"num_streams", "4"}}, 8 << 20, 0, 1, cfg);
    std::atomic<int> failures{0};
    std::vector<std::thread> threads;
    for (int t = 0; t < 4; ++t)
        threads.emplace_back([&, t] {
            const size_t base = size_t(t) << 21;
            std::mt19937 rng(t);
            for (int i = 0; i < 150; ++i) {
                std::vector<std::pair<size_t, size_t>> cuts;
                if (i % 3 == 0) cuts = {{base, 4096}};                                    // proxy
                else if (i % 3 == 1) cuts = {{base + 8192, 700000}};                      // one kernel launch
                else for (int k = 0; k < 40; ++k) cuts.emplace_back(base + 1000000 + size_t(k) * 9000, 5000 + rng() % 3000); // table
                try {
                    nixl_opt_args_t args;
                    args.notif = "t" + std::to_string(t);
                    nixlXferReqH *req = p.request(NIXL_WRITE, cuts, sameOffsets(cuts), &args);
                    p.src.p[cuts[0].first] = static_cast<uint8_t>(i);
                    if (p.a.postXferReq(req) < 0 || waitDone(p.a, req) != NIXL_SUCCESS) ++failures;
                    for (auto &c : cuts)
                        if (std::memcmp(p.src.p + c.first, p.dst.p + c.first, c.second) != 0) ++failures;
                    if (p.a.releaseXferReq(req) != NIXL_SUCCESS) ++failures;
                } catch (const std::exception &) {
                    ++failures;
                }
            }
        });
    size_t seen = 0;
    const auto end = clk::now() + std::chrono::seconds(60);
    while (seen < 600 && clk::now() < end) {
        nixl_notifs_t n;
        p.b.getNotifs(n);
        for (auto &kv : n) seen += kv.second.size();
    }
    for (auto &t : threads) t.join();
    CHECK_EQ(failures.load(), 0);
    CHECK_EQ(seen, size_t(600));
}

TEST_CASE(threads_ring_a_proxy_that_keeps_leaving) {
    // Tiny idle time and life: the proxy leaves between and in the middle of the threads' streams of small requests, so
    // "is it still running" is decided again and again while other threads post, poll and relaunch.
    nixlAgentConfig cfg(false, false, 0, nixl_thread_sync_t::NIXL_THREAD_SYNC_RW);
    Pair p({{"proxy_idle_us", "5"}, {"proxy_life_us", "60"}}, 4 << 20, 0, 1, cfg);
    std::atomic<int> failures{0};
    std::vector<std::thread> threads;
    const int rounds = std::getenv("FAKE_GPU_STRESS") ? 20000 : 1500;
    for (int t = 0; t < 4; ++t)
        threads.emplace_back([&, t] {
            const size_t base = size_t(t) << 20;
            try {
                nixlXferReqH *one = p.request(NIXL_WRITE, {{base, 2048}}, {base});
                nixlXferReqH *three = p.request(NIXL_WRITE, {{base + 65536, 4096}, {base + 131072, 4096}, {base + 262144, 64}},
                                                {base + 131072, base + 262144, base + 65536});
                for (int i = 0; i < rounds; ++i) {
                    nixlXferReqH *req = i % 4 == 3 ? three : one;
                    p.src.p[base + (i % 2048)] = static_cast<uint8_t>(i);
                    p.src.p[base + 65536 + (i % 4096)] = static_cast<uint8_t>(i >> 3);
                    if (p.a.postXferReq(req) < 0 || waitDone(p.a, req) != NIXL_SUCCESS) {
                        ++failures;
                        continue;
                    }
                    if (req == one ? std::memcmp(p.src.p + base, p.dst.p + base, 2048) != 0
                                   : std::memcmp(p.src.p + base + 65536, p.dst.p + base + 131072, 4096) != 0)
                        ++failures;
                    if (i % 97 == t) std::this_thread::sleep_for(std::chrono::microseconds(30));
                }
                if (p.a.releaseXferReq(one) != NIXL_SUCCESS || p.a.releaseXferReq(three) != NIXL_SUCCESS) ++failures;
            } catch (const std::exception &) {
                ++failures;
            }
        });
    for (auto &t : threads) t.join();
    CHECK_EQ(failures.load(), 0);
}

TEST_CASE(host_memory_pinned_and_pageable_to_and_from_a_gpu) {
    // The initiator's side is host memory (registered, which pins it: the copy kernel reaches it; and a second buffer
    // registered with pinning switched off: the runtime stages it), the target's side device memory.
    for (const char *pin : {"true", "false"}) {
        const std::string tag = std::string("hm") + pin;
        nixlAgent a(tag + "_a", nixlAgentConfig(false)), b(tag + "_b", nixlAgentConfig(false));
        nixlBackendH *ha = nullptr, *hb = nullptr;
        CHECK_EQ(a.createBackend("NVLINK", {{"pin_dram", pin}}, ha), NIXL_SUCCESS);
        CHECK_EQ(b.createBackend("NVLINK", {}, hb), NIXL_SUCCESS);
        std::vector<uint8_t> host(2 << 20);
        std::mt19937 rng(4);
        for (auto &x : host) x = static_cast<uint8_t>(rng());
        DevBuf dev(1, host.size(), 0);
        nixl_reg_dlist_t rh(DRAM_SEG), rd(VRAM_SEG);
        rh.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(host.data()), host.size(), 0, ""));
        rd.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dev.p), dev.bytes, 1, ""));
        CHECK_EQ(a.registerMem(rh), NIXL_SUCCESS);
        CHECK_EQ(b.registerMem(rd), NIXL_SUCCESS);
        nixl_blob_t md;
        std::string name;
        b.getLocalMD(md);
        CHECK_EQ(a.loadRemoteMD(md, name), NIXL_SUCCESS);
        nixl_xfer_dlist_t l(DRAM_SEG), r(VRAM_SEG);
        for (int i = 0; i < 8; ++i) {
            l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(host.data()) + size_t(i) * 262144, 262144, 0));
            r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dev.p) + size_t(7 - i) * 262144, 262144, 1));
        }
        nixlXferReqH *req = nullptr;
        CHECK_EQ(a.createXferReq(NIXL_WRITE, l, r, tag + "_b", req), NIXL_SUCCESS);
        CHECK(a.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(a, req), NIXL_SUCCESS);
        for (int i = 0; i < 8; ++i) CHECK(std::memcmp(host.data() + size_t(i) * 262144, dev.p + size_t(7 - i) * 262144, 262144) == 0);
        CHECK_EQ(a.releaseXferReq(req), NIXL_SUCCESS);
        for (size_t i = 0; i < dev.bytes; i += 4099) dev.p[i] ^= 0x3c;
        const std::vector<uint8_t> changed(dev.p, dev.p + dev.bytes);
        CHECK_EQ(a.createXferReq(NIXL_READ, l, r, tag + "_b", req), NIXL_SUCCESS);
        CHECK(a.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(a, req), NIXL_SUCCESS);
        for (int i = 0; i < 8; ++i) CHECK(std::memcmp(host.data() + size_t(i) * 262144, changed.data() + size_t(7 - i) * 262144, 262144) == 0);
        CHECK_EQ(a.releaseXferReq(req), NIXL_SUCCESS);
        CHECK_EQ(a.deregisterMem(rh), NIXL_SUCCESS);
        CHECK_EQ(b.deregisterMem(rd), NIXL_SUCCESS);
    }
}

TEST_CASE(a_request_still_running_cannot_be_posted_again) {
    Pair p({}, 4 << 20, 0, 0);
    cudaSetDevice(0);
    cudaStream_t user = nullptr;
    CHECK_EQ(cudaStreamCreateWithFlags(&user, cudaStreamNonBlocking), cudaSuccess);
    nixl_opt_args_t on_stream;
    on_stream.customParam = "stream=" + std::to_string(reinterpret_cast<uintptr_t>(user));
    nixlXferReqH *req = p.request(NIXL_WRITE, {{0, 3 << 20}}, {0});
    fake_cuda::enqueueDelay(user, 30000);
    CHECK_EQ(p.a.postXferReq(req, &on_stream), NIXL_IN_PROG);
    CHECK_EQ(p.a.postXferReq(req, &on_stream), NIXL_ERR_REPOST_ACTIVE);
    CHECK_EQ(p.a.getXferStatus(req), NIXL_IN_PROG); // the refusal did not disturb the running post
    CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
    CHECK(std::memcmp(p.src.p, p.dst.p, 3 << 20) == 0);
    CHECK(p.a.postXferReq(req, &on_stream) >= 0); // complete: it may go again
    CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
    CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
    cudaStreamDestroy(user);
}

TEST_CASE(memory_views_hold_what_the_kernels_will_read) {
    Pair p({}, 1 << 20, 0, 1);
    nixl_xfer_dlist_t local(VRAM_SEG);
    local.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(p.src.p) + 4096, 8192, 0));
    local.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(p.src.p) + 65536, 100, 0));
    nixl_remote_dlist_t remote(VRAM_SEG);
    remote.addDesc(nixlRemoteDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(p.dst.p) + 512, 2048, 1), p.bn));
    remote.addDesc(nixlRemoteDesc(nixlBasicDesc(0, 0, 0), nixl_null_agent)); // a hole: an absent rank
    remote.addDesc(nixlRemoteDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(p.dst.p) + 8192, 4096, 1), p.bn));
    cudaSetDevice(0);
    nixlMemViewH lv = nullptr, rv = nullptr;
    CHECK_EQ(p.a.prepMemView(local, lv), NIXL_SUCCESS);
    CHECK_EQ(p.a.prepMemView(remote, rv), NIXL_SUCCESS);
    struct Header { uint64_t magic; uint32_t count, kind; };
    struct Entry { uint64_t ptr, len; };
    const auto *lh = static_cast<const Header *>(lv);
    const auto *le = reinterpret_cast<const Entry *>(lh + 1);
    CHECK_EQ(lh->count, 2u);
    CHECK_EQ(lh->kind, 1u);
    CHECK(le[0].ptr == reinterpret_cast<uintptr_t>(p.src.p) + 4096 && le[0].len == 8192 && le[1].len == 100);
    const auto *rh = static_cast<const Header *>(rv);
    const auto *re = reinterpret_cast<const Entry *>(rh + 1);
    CHECK_EQ(rh->count, 3u);
    CHECK_EQ(rh->kind, 2u);
    CHECK(rh->magic == lh->magic && rh->magic != 0);
    CHECK(re[0].ptr == reinterpret_cast<uintptr_t>(p.dst.p) + 512 && re[0].len == 2048);
    CHECK(re[1].ptr == 0); // the hole
    CHECK(re[2].ptr == reinterpret_cast<uintptr_t>(p.dst.p) + 8192 && re[2].len == 4096);
    // a range outside what the target registered is refused
    nixl_remote_dlist_t bad(VRAM_SEG);
    bad.addDesc(nixlRemoteDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(p.dst.p) + p.dst.bytes - 16, 64, 1), p.bn));
    nixlMemViewH bv = nullptr;
    CHECK(p.a.prepMemView(bad, bv) != NIXL_SUCCESS);
    p.a.releaseMemView(lv);
    p.a.releaseMemView(rv);
}

TEST_CASE(memory_from_the_virtual_memory_calls_is_exported_allocation_by_allocation) {
    // Four allocations behind one address range on GPU 1; the registration covers the back half of the first, the two
    // in the middle and the front half of the last.  CUDA IPC refuses such memory, so the backend exports each
    // allocation as a file descriptor and serves them from its descriptor server; deregistration closes them.
    auto open_fds = [] {
        int n = 0;
        for (int fd = 0; fd < 4096; ++fd) n += ::fcntl(fd, F_GETFD) != -1;
        return n;
    };
    constexpr size_t chunk = 1 << 20;
    auto *vm = static_cast<uint8_t *>(fake_cuda::mallocVmm(chunk, 4, 1));
    CHECK(vm != nullptr);
    cudaIpcMemHandle_t ipc;
    CHECK(cudaIpcGetMemHandle(&ipc, vm) != cudaSuccess);
    cudaGetLastError();
    cudaPointerAttributes attr{};
    CHECK_EQ(cudaPointerGetAttributes(&attr, vm + 3 * chunk + 5), cudaSuccess);
    CHECK(attr.type == cudaMemoryTypeDevice && attr.device == 1);

    const std::string an = "fg_vm_a" + std::to_string(++g_serial), bn = "fg_vm_b" + std::to_string(g_serial);
    nixlAgent a(an, nixlAgentConfig(false)), b(bn, nixlAgentConfig(false));
    nixlBackendH *ha = nullptr, *hb = nullptr;
    CHECK(a.createBackend("NVLINK", {}, ha) == NIXL_SUCCESS && b.createBackend("NVLINK", {}, hb) == NIXL_SUCCESS);
    DevBuf src(0, 3 * chunk);
    src.randomize(99);
    uint8_t *win = vm + chunk / 2;
    const size_t win_len = 3 * chunk;
    std::memset(win, 0, win_len);
    nixl_reg_dlist_t ra(VRAM_SEG), rb(VRAM_SEG);
    ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.p), src.bytes, 0, ""));
    rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(win), win_len, 1, ""));
    CHECK(a.registerMem(ra) == NIXL_SUCCESS);
    CHECK(b.registerMem(rb) == NIXL_SUCCESS); // starts the descriptor server (a socket and a wake-up pipe stay open)
    const int with_one = open_fds();
    CHECK_EQ(b.deregisterMem(rb), NIXL_SUCCESS);
    CHECK_EQ(open_fds(), with_one - 4); // one descriptor per allocation touched
    for (int round = 0; round < 20; ++round) { // and none is leaked over registrations
        CHECK(b.registerMem(rb) == NIXL_SUCCESS);
        CHECK_EQ(open_fds(), with_one);
        if (round < 19) CHECK_EQ(b.deregisterMem(rb), NIXL_SUCCESS);
    }
    // a range that runs past the last allocation has no export: it still registers (this process can use it) ...
    // but one that is not device memory at all is refused
    nixl_reg_dlist_t past(VRAM_SEG);
    past.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(vm) + 4 * chunk, 4096, 1, ""));
    CHECK(b.registerMem(past) != NIXL_SUCCESS);

    nixl_blob_t md;
    std::string name;
    b.getLocalMD(md);
    CHECK(a.loadRemoteMD(md, name) == NIXL_SUCCESS);
    // pieces that cross the boundaries between allocations
    nixl_xfer_dlist_t l(VRAM_SEG), r(VRAM_SEG);
    std::vector<uint8_t> expect(win_len, 0);
    for (int i = 0; i < 12; ++i) {
        const size_t off = size_t(i) * 250000 + 64, len = 200000 + 16 * i;
        l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.p) + off, len, 0));
        r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(win) + off, len, 1));
        std::memcpy(expect.data() + off, src.p + off, len);
    }
    nixlXferReqH *req = nullptr;
    CHECK(a.createXferReq(NIXL_WRITE, l, r, bn, req) == NIXL_SUCCESS);
    CHECK(a.postXferReq(req) >= 0);
    CHECK_EQ(waitDone(a, req), NIXL_SUCCESS);
    CHECK(std::memcmp(win, expect.data(), win_len) == 0);
    CHECK_EQ(a.releaseXferReq(req), NIXL_SUCCESS);
    CHECK_EQ(a.invalidateRemoteMD(bn), NIXL_SUCCESS);
    CHECK_EQ(b.deregisterMem(rb), NIXL_SUCCESS);
    CHECK_EQ(a.deregisterMem(ra), NIXL_SUCCESS);
    for (int d = 0; d < 2; ++d) {
        cudaSetDevice(d);
        cudaDeviceSynchronize();
    }
    fake_cuda::freeVmm(vm);
}

TEST_CASE(device_memory_crosses_the_tcp_backend_through_its_staging_buffers) {
    // The TCP backend built against the stand-in runtime: device memory on either end is staged through a pinned buffer
    // (4 MiB pieces), host memory is not.  9 MiB and a bit, so that the staging loop runs more than twice per message set.
    const std::string an = "fg_tcp_a" + std::to_string(++g_serial), bn = "fg_tcp_b" + std::to_string(g_serial);
    nixlAgent a(an, nixlAgentConfig(false)), b(bn, nixlAgentConfig(false));
    nixlBackendH *ha = nullptr, *hb = nullptr;
    const nixl_b_params_t params = {{"address", "127.0.0.1"}, {"rails", "2"}, {"chunk_bytes", "6291456"}};
    CHECK(a.createBackend("TCP", params, ha) == NIXL_SUCCESS && b.createBackend("TCP", params, hb) == NIXL_SUCCESS);
    constexpr size_t kBytes = (9 << 20) + 12345;
    DevBuf src(0, kBytes), dst(1, kBytes, 0);
    src.randomize(4242);
    std::vector<uint8_t> host(kBytes, 0);
    nixl_reg_dlist_t ra(VRAM_SEG), rb(VRAM_SEG), rh(DRAM_SEG);
    ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.p), kBytes, 0, ""));
    rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.p), kBytes, 1, ""));
    rh.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(host.data()), kBytes, 0, ""));
    CHECK(a.registerMem(ra) == NIXL_SUCCESS && b.registerMem(rb) == NIXL_SUCCESS && b.registerMem(rh) == NIXL_SUCCESS);
    // a descriptor that names the wrong GPU, and host memory passed off as device memory, are refused at registration
    nixl_reg_dlist_t wrong(VRAM_SEG), fake(VRAM_SEG);
    wrong.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.p), 4096, 1, ""));
    fake.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(host.data()), 4096, 0, ""));
    CHECK(a.registerMem(wrong) != NIXL_SUCCESS);
    CHECK(a.registerMem(fake) != NIXL_SUCCESS);
    nixl_blob_t md;
    std::string name;
    b.getLocalMD(md);
    CHECK_EQ(a.loadRemoteMD(md, name), NIXL_SUCCESS);

    auto run = [&](nixl_xfer_op_t op, nixl_mem_t remote_mem, uintptr_t remote, int remote_dev) {
        nixl_xfer_dlist_t l(VRAM_SEG), r(remote_mem);
        // three pieces, the middle one larger than a staging buffer
        const size_t cuts[4] = {0, 1000003, (6 << 20) + 77, kBytes};
        for (int i = 0; i < 3; ++i) {
            l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.p) + cuts[i], cuts[i + 1] - cuts[i], 0));
            r.addDesc(nixlBasicDesc(remote + cuts[i], cuts[i + 1] - cuts[i], remote_dev));
        }
        nixl_opt_args_t args;
        args.notif = "staged";
        nixlXferReqH *req = nullptr;
        CHECK_EQ(a.createXferReq(op, l, r, bn, req, &args), NIXL_SUCCESS);
        CHECK(a.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(a, req), NIXL_SUCCESS);
        CHECK_EQ(a.releaseXferReq(req), NIXL_SUCCESS);
    };
    run(NIXL_WRITE, VRAM_SEG, reinterpret_cast<uintptr_t>(dst.p), 1); // device -> device
    CHECK(std::memcmp(src.p, dst.p, kBytes) == 0);
    run(NIXL_WRITE, DRAM_SEG, reinterpret_cast<uintptr_t>(host.data()), 0); // device -> host
    CHECK(std::memcmp(src.p, host.data(), kBytes) == 0);
    for (size_t i = 0; i < kBytes; i += 997) dst.p[i] = static_cast<uint8_t>(dst.p[i] + 3);
    std::vector<uint8_t> expect(dst.p, dst.p + kBytes);
    run(NIXL_READ, VRAM_SEG, reinterpret_cast<uintptr_t>(dst.p), 1); // device <- device
    CHECK(std::memcmp(src.p, expect.data(), kBytes) == 0);
    for (size_t i = 0; i < kBytes; i += 991) host[i] = static_cast<uint8_t>(host[i] + 5);
    run(NIXL_READ, DRAM_SEG, reinterpret_cast<uintptr_t>(host.data()), 0); // device <- host
    CHECK(std::memcmp(src.p, host.data(), kBytes) == 0);
    int notifs = 0;
    const auto end = clk::now() + std::chrono::seconds(5);
    while (notifs < 4 && clk::now() < end) {
        nixl_notifs_t n;
        b.getNotifs(n);
        notifs += static_cast<int>(n[an].size());
    }
    CHECK_EQ(notifs, 4);
    CHECK_EQ(a.invalidateRemoteMD(bn), NIXL_SUCCESS);
    CHECK(a.deregisterMem(ra) == NIXL_SUCCESS && b.deregisterMem(rb) == NIXL_SUCCESS && b.deregisterMem(rh) == NIXL_SUCCESS);
}

TEST_CASE(random_requests_against_a_model_under_every_path_choice) {
    // Requests drawn at random (1 to 300 pieces from one byte to 3 MiB, touching or apart, in any order on either side,
    // WRITE and READ, some posted twice, several in flight) under engine settings that push them down different
    // paths: everything through the copy kernel, long runs through the copy engines, small requests through the doorbell
    // proxy, merging on and off, one stream and four.  After each wave both buffers must equal the model.
    struct Setting {
        const char *name;
        nixl_b_params_t params;
    };
    const Setting settings[] = {
        {"kernel only", {{"proxy", "false"}, {"ce_threshold", "0"}}},
        {"copy engines from 256 KiB", {{"proxy", "false"}, {"ce_threshold", "262144"}}},
        {"proxy and copy engines", {{"ce_threshold", "1048576"}, {"num_streams", "4"}}},
        {"no merging", {{"coalesce", "false"}, {"ce_threshold", "524288"}, {"num_streams", "2"}}},
    };
    constexpr size_t kBytes = 24 << 20;
    std::mt19937_64 rng(20240611);
    for (const Setting &st : settings) {
        Pair p(st.params, kBytes);
        std::vector<uint8_t> model_src(p.src.p, p.src.p + kBytes), model_dst(kBytes, 0);
        for (int wave = 0; wave < 40; ++wave) {
            // a wave: up to three requests in flight over disjoint thirds of the buffers
            const int in_flight = 1 + static_cast<int>(rng() % 3);
            std::vector<nixlXferReqH *> reqs;
            for (int r = 0; r < in_flight; ++r) {
                const size_t lane = kBytes / 3, base = lane * static_cast<size_t>(r);
                const nixl_xfer_op_t op = rng() % 3 == 0 ? NIXL_READ : NIXL_WRITE;
                const int shape = static_cast<int>(rng() % 4);
                int n = shape == 0 ? 1 : shape == 1 ? 2 + static_cast<int>(rng() % 30) : shape == 2 ? 33 + static_cast<int>(rng() % 268) : 1 + static_cast<int>(rng() % 6);
                std::vector<size_t> len(static_cast<size_t>(n));
                size_t total = 0;
                for (auto &l : len) {
                    l = shape == 3 ? 200000 + rng() % 2900000 : shape == 0 ? 1 + rng() % 5000000 : 1 + rng() % (rng() % 5 == 0 ? 150000 : 6000);
                    total += l;
                }
                while (total > lane) { // shrink until the wave fits its lane
                    total = 0;
                    for (auto &l : len) {
                        l = std::max<size_t>(1, l / 2);
                        total += l;
                    }
                }
                auto place = [&](bool touching) {
                    std::vector<size_t> order(len.size()), off(len.size());
                    for (size_t i = 0; i < order.size(); ++i) order[i] = i;
                    if (rng() % 2) std::shuffle(order.begin(), order.end(), rng);
                    size_t slack = lane - total, at = base;
                    for (size_t k = 0; k < order.size(); ++k) {
                        const size_t gap = touching || slack == 0 ? 0 : rng() % (slack / (order.size() - k) + 1);
                        at += gap;
                        slack -= gap;
                        off[order[k]] = at;
                        at += len[order[k]];
                    }
                    return off;
                };
                const std::vector<size_t> lo = place(rng() % 2), ro = place(rng() % 2);
                std::vector<std::pair<size_t, size_t>> cuts;
                for (size_t i = 0; i < len.size(); ++i) cuts.emplace_back(lo[i], len[i]);
                for (size_t i = 0; i < len.size(); ++i) {
                    if (op == NIXL_WRITE) std::memcpy(model_dst.data() + ro[i], model_src.data() + lo[i], len[i]);
                    else std::memcpy(model_src.data() + lo[i], model_dst.data() + ro[i], len[i]);
                }
                nixlXferReqH *req = p.request(op, cuts, ro);
                CHECK(p.a.postXferReq(req) >= 0);
                reqs.push_back(req);
            }
            for (nixlXferReqH *req : reqs) CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
            if (rng() % 2) { // the same requests once more: nothing may change
                for (nixlXferReqH *req : reqs) CHECK(p.a.postXferReq(req) >= 0);
                for (nixlXferReqH *req : reqs) CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
            }
            for (nixlXferReqH *req : reqs) CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
            if (std::memcmp(p.src.p, model_src.data(), kBytes) != 0 || std::memcmp(p.dst.p, model_dst.data(), kBytes) != 0)
                throw harness::Failure(std::string("buffers differ from the model under '") + st.name + "', wave " + std::to_string(wave));
            // fresh bytes for the next wave
            for (size_t i = 0; i < kBytes; i += 4093) {
                p.src.p[i] = model_src[i] = static_cast<uint8_t>(rng());
                p.dst.p[i] = model_dst[i] = static_cast<uint8_t>(rng());
            }
        }
    }
}

TEST_CASE(device_memory_to_files_and_back_through_the_gds_engine_against_a_model) {
    // The GDS engine built against the stand-in runtime: pieces of device memory go to places in two files and come back,
    // through the engine's pairs of pinned staging buffers (8 MiB each, so the 20 MiB piece cycles them) and its worker
    // threads.  Pieces are drawn at random; a model says what the files and the buffer must hold after every request.
    char tmpl[] = "/tmp/nixl_fake_gds_XXXXXX";
    CHECK(::mkdtemp(tmpl) != nullptr);
    const std::string dir = tmpl;
    nixlAgent a("fg_gds", nixlAgentConfig(false));
    nixlBackendH *h = nullptr;
    CHECK_EQ(a.createBackend("GDS", {{"thread_count", "3"}}, h), NIXL_SUCCESS);
    constexpr size_t kBytes = 48 << 20, kFile = 32 << 20;
    DevBuf buf(1, kBytes);
    buf.randomize(77);
    nixl_reg_dlist_t rv(VRAM_SEG), rf(FILE_SEG);
    rv.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf.p), kBytes, 1, ""));
    int fds[2];
    std::vector<std::vector<uint8_t>> model_file(2, std::vector<uint8_t>(kFile, 0));
    for (int f = 0; f < 2; ++f) {
        fds[f] = ::open((dir + "/f" + std::to_string(f)).c_str(), O_RDWR | O_CREAT, 0644);
        CHECK(fds[f] >= 0 && ::ftruncate(fds[f], kFile) == 0);
        rf.addDesc(nixlBlobDesc(0, kFile, static_cast<uint64_t>(fds[f]), ""));
    }
    CHECK(a.registerMem(rv) == NIXL_SUCCESS && a.registerMem(rf) == NIXL_SUCCESS);
    std::vector<uint8_t> model_buf(buf.p, buf.p + kBytes);
    std::mt19937_64 rng(5);
    for (int round = 0; round < 14; ++round) {
        const nixl_xfer_op_t op = round % 3 == 2 ? NIXL_READ : NIXL_WRITE;
        const int n = round == 0 ? 1 : 1 + static_cast<int>(rng() % 12);
        nixl_xfer_dlist_t l(VRAM_SEG), r(FILE_SEG);
        size_t at_buf = rng() % 4096, at_file[2] = {rng() % 4096, rng() % 4096};
        for (int i = 0; i < n; ++i) {
            const int f = static_cast<int>(rng() % 2);
            size_t len = round == 0 ? (20u << 20) + 123 : 1 + rng() % (rng() % 4 == 0 ? 3000000 : 40000);
            len = std::min({len, kBytes - at_buf, kFile - at_file[f]});
            if (len == 0) break;
            l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf.p) + at_buf, len, 1));
            r.addDesc(nixlBasicDesc(at_file[f], len, static_cast<uint64_t>(fds[f])));
            if (op == NIXL_WRITE) std::memcpy(model_file[static_cast<size_t>(f)].data() + at_file[f], model_buf.data() + at_buf, len);
            else std::memcpy(model_buf.data() + at_buf, model_file[static_cast<size_t>(f)].data() + at_file[f], len);
            at_buf += len + rng() % 5000;
            at_file[f] += len + rng() % 5000;
            if (at_buf >= kBytes) break;
        }
        if (l.descCount() == 0) continue;
        nixlXferReqH *req = nullptr;
        CHECK_EQ(a.createXferReq(op, l, r, "fg_gds", req), NIXL_SUCCESS);
        CHECK(a.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(a, req, 60.0), NIXL_SUCCESS);
        CHECK_EQ(a.releaseXferReq(req), NIXL_SUCCESS);
        CHECK(std::memcmp(buf.p, model_buf.data(), kBytes) == 0);
        for (int f = 0; f < 2; ++f) {
            std::vector<uint8_t> on_disk(kFile);
            CHECK_EQ(::pread(fds[f], on_disk.data(), kFile, 0), static_cast<ssize_t>(kFile));
            CHECK(on_disk == model_file[static_cast<size_t>(f)]);
        }
        // new bytes in the buffer for the next round
        for (size_t i = 0; i < kBytes; i += 1021) buf.p[i] = model_buf[i] = static_cast<uint8_t>(rng());
    }
    CHECK(a.deregisterMem(rf) == NIXL_SUCCESS && a.deregisterMem(rv) == NIXL_SUCCESS);
    for (int f = 0; f < 2; ++f) {
        ::close(fds[f]);
        ::unlink((dir + "/f" + std::to_string(f)).c_str());
    }
    ::rmdir(dir.c_str());
}

TEST_CASE(launch_failures_are_reported_and_leave_the_engine_usable) {
    using fake_cuda::LaunchKind;
    // a copy-kernel launch fails: the post says so, the request can be posted again and released
    {
        Pair p({{"proxy", "false"}}, 1 << 20);
        nixl_opt_args_t args;
        args.notif = "never";
        nixlXferReqH *req = p.request(NIXL_WRITE, {{0, 300000}}, {0}, &args);
        fake_cuda::failLaunches(LaunchKind::Copy, 1);
        CHECK_EQ(p.a.postXferReq(req), NIXL_ERR_BACKEND);
        CHECK_EQ(p.a.getXferStatus(req), NIXL_ERR_BACKEND);
        nixl_notifs_t got;
        p.b.getNotifs(got);
        CHECK(got[p.an].empty()); // the slot claimed for the notification was voided, nothing was delivered
        CHECK(p.a.postXferReq(req) >= 0); // the next launch works
        CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
        CHECK(std::memcmp(p.src.p, p.dst.p, 300000) == 0);
        for (int i = 0; i < 2000 && got[p.an].empty(); ++i) p.b.getNotifs(got);
        CHECK_EQ(got[p.an].size(), size_t(1)); // one notification, from the post that worked
        CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
    }
    // the one-thread kernel behind the copy engines fails
    {
        Pair p({{"ce_threshold", "65536"}}, 1 << 20);
        nixlXferReqH *req = p.request(NIXL_WRITE, {{0, 1 << 19}}, {0});
        fake_cuda::failLaunches(LaunchKind::Signal, 1);
        CHECK_EQ(p.a.postXferReq(req), NIXL_ERR_BACKEND);
        CHECK(p.a.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
        CHECK(std::memcmp(p.src.p, p.dst.p, 1 << 19) == 0);
        CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
    }
    // the doorbell proxy cannot be started: the request that rang it reports the failure, later small requests take
    // the launch path
    {
        Pair p({}, 1 << 20);
        nixlXferReqH *req = p.request(NIXL_WRITE, {{0, 4096}}, {0});
        fake_cuda::failLaunches(LaunchKind::Proxy, 1);
        const nixl_status_t first = p.a.postXferReq(req);
        CHECK(first == NIXL_ERR_BACKEND || (first == NIXL_IN_PROG && waitDone(p.a, req) == NIXL_ERR_BACKEND));
        for (int i = 0; i < 20; ++i) {
            p.src.p[i] ^= 0x42;
            CHECK(p.a.postXferReq(req) >= 0);
            CHECK_EQ(waitDone(p.a, req), NIXL_SUCCESS);
            CHECK(std::memcmp(p.src.p, p.dst.p, 4096) == 0);
        }
        CHECK_EQ(p.a.releaseXferReq(req), NIXL_SUCCESS);
    }
}

TEST_CASE(a_target_that_went_away_is_reported_and_its_metadata_dropped) {
    auto p = std::make_unique<Pair>(nixl_b_params_t{}, 1 << 16);
    nixlXferReqH *req = p->request(NIXL_WRITE, {{0, 4096}}, {0});
    CHECK(p->a.postXferReq(req) >= 0);
    CHECK_EQ(waitDone(p->a, req), NIXL_SUCCESS);
    // Only the target agent goes; its buffer stays allocated (the Pair owns it) so nothing dangles.
    // A Pair cannot drop one agent, so the check uses a second target created and destroyed here.
    {
        auto other = std::make_unique<nixlAgent>("fg_gone", nixlAgentConfig(false));
        nixlBackendH *h = nullptr;
        CHECK_EQ(other->createBackend("NVLINK", {}, h), NIXL_SUCCESS);
        DevBuf there(1, 1 << 16, 0);
        nixl_reg_dlist_t reg(VRAM_SEG);
        reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(there.p), there.bytes, 1, ""));
        CHECK_EQ(other->registerMem(reg), NIXL_SUCCESS);
        nixl_blob_t md;
        std::string name;
        other->getLocalMD(md);
        CHECK_EQ(p->a.loadRemoteMD(md, name), NIXL_SUCCESS);
        nixl_xfer_dlist_t l(VRAM_SEG), r(VRAM_SEG);
        l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(p->src.p), 4096, 0));
        r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(there.p), 4096, 1));
        nixlXferReqH *to_other = nullptr;
        CHECK_EQ(p->a.createXferReq(NIXL_WRITE, l, r, "fg_gone", to_other), NIXL_SUCCESS);
        CHECK(p->a.postXferReq(to_other) >= 0);
        CHECK_EQ(waitDone(p->a, to_other), NIXL_SUCCESS);
        other->deregisterMem(reg);
        other.reset();
        CHECK_EQ(p->a.postXferReq(to_other), NIXL_ERR_REMOTE_DISCONNECT);
        CHECK_EQ(p->a.checkRemoteMD("fg_gone", nixl_xfer_dlist_t(VRAM_SEG)), NIXL_ERR_NOT_FOUND);
        p->a.releaseXferReq(to_other);
    }
    CHECK_EQ(p->a.releaseXferReq(req), NIXL_SUCCESS);
}

int main(int argc, char **argv) {
    nixlPluginManager::getInstance().addPluginDirectory(FAKE_GPU_PLUGIN_DIR); // in front of the regular plug-in directory
    return harness::runAll(argc, argv);
}

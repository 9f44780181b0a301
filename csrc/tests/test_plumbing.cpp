// CPU plumbing: two agents in one process move 64 x 1 MiB DRAM descriptors (WRITE then
// READ) with a completion notification, metadata round-trips through loadRemoteMD, and the
// same buffers go to a file and back through the POSIX backend.
// Mirrors the scenarios of the reference's test/gtest/test_transfer.cpp and
// test/unit/plugins/posix/nixl_posix_test.cpp.
#include <chrono>
#include <cstring>
#include <fcntl.h>
#include <random>
#include <thread>
#include <unistd.h>

#include <filesystem>
#include <fstream>
#include <sys/stat.h>

#include "harness.h"
#include "utils/hw_info.h"
#include "utils/topology.h"
#include "utils/misc.h"
#include "nixl.h"

namespace {
constexpr size_t kDescs = 64, kLen = 1 << 20;

std::vector<uint8_t> seeded(size_t n, uint64_t seed) {
    std::mt19937_64 g(seed);
    std::vector<uint8_t> v(n);
    for (size_t i = 0; i < n; i += 8) {
        const uint64_t r = g();
        std::memcpy(&v[i], &r, std::min<size_t>(8, n - i));
    }
    return v;
}

nixl_status_t waitDone(nixlAgent &a, nixlXferReqH *req) {
    nixl_status_t st;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(30);
    while ((st = a.getXferStatus(req)) == NIXL_IN_PROG) {
        if (std::chrono::steady_clock::now() > deadline) return NIXL_ERR_UNKNOWN;
        std::this_thread::yield();
    }
    return st;
}

nixl_xfer_dlist_t slices(nixl_mem_t mem, const void *base, uint64_t dev) {
    nixl_xfer_dlist_t l(mem);
    for (size_t i = 0; i < kDescs; ++i) l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(base) + i * kLen, kLen, dev));
    return l;
}
} // namespace

TEST_CASE(dram_write_read_notif) {
    nixlAgentConfig cfg(false);
    nixlAgent A("alpha", cfg), B("beta", cfg);
    nixlBackendH *ba = nullptr, *bb = nullptr;
    nixl_b_params_t params;
    nixl_mem_list_t mems;
    CHECK_EQ(A.getPluginParams("NVLINK", mems, params), NIXL_SUCCESS);
    CHECK(mems.size() == 2);
    CHECK_EQ(A.createBackend("NVLINK", params, ba), NIXL_SUCCESS);
    CHECK_EQ(B.createBackend("UCX", params, bb), NIXL_SUCCESS); // alias of the NVLink backend

    std::vector<uint8_t> src = seeded(kDescs * kLen, 0), dst(kDescs * kLen, 0);
    nixl_reg_dlist_t ra(DRAM_SEG), rb(DRAM_SEG);
    ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
    rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
    CHECK_EQ(A.registerMem(ra), NIXL_SUCCESS);
    CHECK_EQ(B.registerMem(rb), NIXL_SUCCESS);

    nixl_blob_t mdA, mdB;
    CHECK_EQ(A.getLocalMD(mdA), NIXL_SUCCESS);
    CHECK_EQ(B.getLocalMD(mdB), NIXL_SUCCESS);
    std::string name;
    CHECK_EQ(A.loadRemoteMD(mdB, name), NIXL_SUCCESS);
    CHECK(name == "beta");
    CHECK_EQ(B.loadRemoteMD(mdA, name), NIXL_SUCCESS);
    CHECK(name == "alpha");
    CHECK_EQ(A.loadRemoteMD(mdA, name), NIXL_ERR_INVALID_PARAM); // own metadata
    CHECK_EQ(A.checkRemoteMD("beta", slices(DRAM_SEG, dst.data(), 0)), NIXL_SUCCESS);
    CHECK_EQ(A.checkRemoteMD("gamma", nixl_xfer_dlist_t(DRAM_SEG)), NIXL_ERR_NOT_FOUND);

    // WRITE alpha -> beta with a notification.
    nixl_opt_args_t opt;
    opt.notif = "write-done";
    nixlXferReqH *req = nullptr;
    CHECK_EQ(A.createXferReq(NIXL_WRITE, slices(DRAM_SEG, src.data(), 0), slices(DRAM_SEG, dst.data(), 0), "beta", req, &opt),
             NIXL_SUCCESS);
    nixl_status_t st = A.postXferReq(req);
    CHECK(st == NIXL_SUCCESS || st == NIXL_IN_PROG);
    CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
    CHECK(src == dst);
    nixl_notifs_t notifs;
    for (int i = 0; i < 1000 && notifs.empty(); ++i) CHECK_EQ(B.getNotifs(notifs), NIXL_SUCCESS);
    CHECK(notifs.count("alpha") == 1 && notifs["alpha"].size() == 1 && notifs["alpha"][0] == "write-done");
    CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);

    // READ: alpha pulls beta's (modified) buffer back.
    for (auto &b : dst) b ^= 0x5a;
    CHECK_EQ(A.createXferReq(NIXL_READ, slices(DRAM_SEG, src.data(), 0), slices(DRAM_SEG, dst.data(), 0), "beta", req),
             NIXL_SUCCESS);
    st = A.postXferReq(req);
    CHECK(st >= 0);
    CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
    CHECK(src == dst);
    // Requests are re-postable once complete.
    st = A.postXferReq(req);
    CHECK(st >= 0);
    CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
    CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);

    // Stand-alone notification.
    CHECK_EQ(B.genNotif("alpha", "hello"), NIXL_SUCCESS);
    notifs.clear();
    for (int i = 0; i < 1000 && notifs.empty(); ++i) A.getNotifs(notifs);
    CHECK(notifs["beta"].size() == 1 && notifs["beta"][0] == "hello");

    // After invalidation the remote is unknown.
    CHECK_EQ(A.invalidateRemoteMD("beta"), NIXL_SUCCESS);
    CHECK_EQ(A.createXferReq(NIXL_WRITE, slices(DRAM_SEG, src.data(), 0), slices(DRAM_SEG, dst.data(), 0), "beta", req),
             NIXL_ERR_NOT_FOUND);
    CHECK_EQ(A.deregisterMem(ra), NIXL_SUCCESS);
    CHECK_EQ(B.deregisterMem(rb), NIXL_SUCCESS);
}

TEST_CASE(prepared_lists_and_merge) {
    nixlAgentConfig cfg(false);
    nixlAgent A("p1", cfg), B("p2", cfg);
    nixlBackendH *ba = nullptr, *bb = nullptr;
    CHECK_EQ(A.createBackend("NVLINK", {}, ba), NIXL_SUCCESS);
    CHECK_EQ(B.createBackend("NVLINK", {}, bb), NIXL_SUCCESS);
    std::vector<uint8_t> src = seeded(kDescs * 4096, 3), dst(kDescs * 4096, 0);
    nixl_reg_dlist_t ra(DRAM_SEG), rb(DRAM_SEG);
    ra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
    rb.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
    CHECK_EQ(A.registerMem(ra), NIXL_SUCCESS);
    CHECK_EQ(B.registerMem(rb), NIXL_SUCCESS);
    nixl_blob_t md;
    std::string name;
    CHECK_EQ(B.getLocalMD(md), NIXL_SUCCESS);
    CHECK_EQ(A.loadRemoteMD(md, name), NIXL_SUCCESS);

    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    for (size_t i = 0; i < kDescs; ++i) {
        l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()) + i * 4096, 4096, 0));
        r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.data()) + i * 4096, 4096, 0));
    }
    nixlDlistH *lh = nullptr, *rh = nullptr;
    CHECK_EQ(A.prepXferDlist(NIXL_INIT_AGENT, l, lh), NIXL_SUCCESS);
    CHECK_EQ(A.prepXferDlist("p2", r, rh), NIXL_SUCCESS);
    // Reverse order on the remote side: block i lands in slot 63-i.
    std::vector<int> li, ri;
    for (int i = 0; i < (int)kDescs; ++i) {
        li.push_back(i);
        ri.push_back((int)kDescs - 1 - i);
    }
    nixlXferReqH *req = nullptr;
    CHECK_EQ(A.makeXferReq(NIXL_WRITE, lh, li, rh, ri, req), NIXL_SUCCESS);
    CHECK(A.postXferReq(req) >= 0);
    CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
    for (size_t i = 0; i < kDescs; ++i)
        CHECK(std::memcmp(src.data() + i * 4096, dst.data() + (kDescs - 1 - i) * 4096, 4096) == 0);
    CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);
    // In-order indices merge into one descriptor; mismatched counts are rejected.
    CHECK_EQ(A.makeXferReq(NIXL_WRITE, lh, li, rh, li, req), NIXL_SUCCESS);
    CHECK(A.postXferReq(req) >= 0);
    CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
    CHECK(src == dst);
    CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);
    std::vector<int> short_idx = {0, 1};
    CHECK_EQ(A.makeXferReq(NIXL_WRITE, lh, li, rh, short_idx, req), NIXL_ERR_INVALID_PARAM);
    CHECK_EQ(A.makeXferReq(NIXL_WRITE, rh, li, lh, li, req), NIXL_ERR_INVALID_PARAM); // sides swapped
    CHECK_EQ(A.releasedDlistH(lh), NIXL_SUCCESS);
    CHECK_EQ(A.releasedDlistH(rh), NIXL_SUCCESS);
}

TEST_CASE(posix_file_roundtrip) {
    nixlAgentConfig cfg(false);
    nixlAgent A("filer", cfg);
    nixlBackendH *posix = nullptr;
    CHECK_EQ(A.createBackend("POSIX", {}, posix), NIXL_SUCCESS);
    std::vector<uint8_t> src = seeded(kDescs * kLen, 0), back(kDescs * kLen, 0);
    char path[] = "/tmp/nixl_b200_plumbing_XXXXXX";
    const int fd = ::mkstemp(path);
    CHECK(fd >= 0);

    nixl_reg_dlist_t rm(DRAM_SEG), rf(FILE_SEG);
    rm.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
    rm.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(back.data()), back.size(), 0, ""));
    rf.addDesc(nixlBlobDesc(0, 0, fd, "")); // whole file, fd mode
    CHECK_EQ(A.registerMem(rm), NIXL_SUCCESS);
    CHECK_EQ(A.registerMem(rf), NIXL_SUCCESS);

    nixl_xfer_dlist_t file(FILE_SEG);
    for (size_t i = 0; i < kDescs; ++i) file.addDesc(nixlBasicDesc(i * kLen, kLen, fd));
    nixlXferReqH *req = nullptr;
    CHECK_EQ(A.createXferReq(NIXL_WRITE, slices(DRAM_SEG, src.data(), 0), file, "filer", req), NIXL_SUCCESS);
    CHECK(A.postXferReq(req) >= 0);
    CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
    CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);
    CHECK_EQ(A.createXferReq(NIXL_READ, slices(DRAM_SEG, back.data(), 0), file, "filer", req), NIXL_SUCCESS);
    CHECK(A.postXferReq(req) >= 0);
    CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
    CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);
    CHECK(src == back);

    // queryMem: the file exists and has the expected size; a bogus name does not.
    nixl_reg_dlist_t q(FILE_SEG);
    q.addDesc(nixlBlobDesc(0, 0, 0, path));
    q.addDesc(nixlBlobDesc(0, 0, 0, "/nonexistent/nixl_b200"));
    std::vector<nixl_query_resp_t> resp;
    nixl_opt_args_t opt;
    opt.backends.push_back(posix);
    CHECK_EQ(A.queryMem(q, resp, &opt), NIXL_SUCCESS);
    CHECK(resp.size() == 2 && resp[0].has_value() && !resp[1].has_value());
    CHECK(resp[0]->at("size") == std::to_string(kDescs * kLen));

    // Path mode: the backend opens the file itself; devId is just a unique key.
    CHECK_EQ(A.deregisterMem(rf), NIXL_SUCCESS);
    nixl_reg_dlist_t rp(FILE_SEG);
    rp.addDesc(nixlBlobDesc(0, 0, 777, std::string("ro:") + path));
    CHECK_EQ(A.registerMem(rp), NIXL_SUCCESS);
    std::fill(back.begin(), back.end(), 0);
    nixl_xfer_dlist_t pfile(FILE_SEG);
    for (size_t i = 0; i < kDescs; ++i) pfile.addDesc(nixlBasicDesc(i * kLen, kLen, 777));
    CHECK_EQ(A.createXferReq(NIXL_READ, slices(DRAM_SEG, back.data(), 0), pfile, "filer", req), NIXL_SUCCESS);
    CHECK(A.postXferReq(req) >= 0);
    CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
    CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);
    CHECK(src == back);
    ::close(fd);
    ::unlink(path);
}

TEST_CASE(posix_every_queue_kind_moves_more_operations_than_its_depth) {
    // 300 descriptors through a kernel queue of 32 entries: submit has to reap while it fills.
    constexpr size_t kOps = 300, kOpLen = 4096;
    const char *kinds[] = {"use_aio", "use_uring", "use_posix_aio", "threads"};
    for (const char *kind : kinds) {
        nixlAgentConfig cfg(false);
        const std::string me = std::string("filer_") + kind;
        nixlAgent A(me, cfg);
        nixl_b_params_t params = {{"kernel_queue_size", "32"}, {"ios_pool_size", "4"}};
        if (std::string(kind) != "threads") params[kind] = "true";
        nixlBackendH *posix = nullptr;
        CHECK_EQ(A.createBackend("POSIX", params, posix), NIXL_SUCCESS);
        std::vector<uint8_t> src = seeded(kOps * kOpLen, 7), back(kOps * kOpLen, 0);
        char path[] = "/tmp/nixl_b200_queues_XXXXXX";
        const int fd = ::mkstemp(path);
        CHECK(fd >= 0);
        nixl_reg_dlist_t rm(DRAM_SEG), rf(FILE_SEG);
        rm.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
        rm.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(back.data()), back.size(), 0, ""));
        rf.addDesc(nixlBlobDesc(0, 0, fd, ""));
        CHECK_EQ(A.registerMem(rm), NIXL_SUCCESS);
        CHECK_EQ(A.registerMem(rf), NIXL_SUCCESS);
        nixl_xfer_dlist_t file(FILE_SEG), out(DRAM_SEG), in(DRAM_SEG);
        for (size_t i = 0; i < kOps; ++i) {
            // File offsets in reverse order, so that a queue which mixed up its slots would show.
            file.addDesc(nixlBasicDesc((kOps - 1 - i) * kOpLen, kOpLen, fd));
            out.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()) + i * kOpLen, kOpLen, 0));
            in.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(back.data()) + i * kOpLen, kOpLen, 0));
        }
        nixlXferReqH *req = nullptr;
        CHECK_EQ(A.createXferReq(NIXL_WRITE, out, file, me, req), NIXL_SUCCESS);
        CHECK(A.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
        CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);
        CHECK_EQ(A.createXferReq(NIXL_READ, in, file, me, req), NIXL_SUCCESS);
        CHECK(A.postXferReq(req) >= 0);
        CHECK_EQ(waitDone(A, req), NIXL_SUCCESS);
        CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);
        CHECK(src == back);
        // The file holds the blocks in reverse order.
        std::vector<uint8_t> first(kOpLen);
        CHECK(::pread(fd, first.data(), kOpLen, 0) == static_cast<ssize_t>(kOpLen));
        CHECK(std::equal(first.begin(), first.end(), src.begin() + (kOps - 1) * kOpLen));
        // Reading past the end of the file fails the request instead of hanging it.
        nixl_xfer_dlist_t beyond(FILE_SEG), one(DRAM_SEG);
        beyond.addDesc(nixlBasicDesc(kOps * kOpLen + (1 << 20), kOpLen, fd));
        one.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(back.data()), kOpLen, 0));
        CHECK_EQ(A.createXferReq(NIXL_READ, one, beyond, me, req), NIXL_SUCCESS);
        const nixl_status_t posted = A.postXferReq(req);
        CHECK(posted < 0 || waitDone(A, req) < 0);
        CHECK_EQ(A.releaseXferReq(req), NIXL_SUCCESS);
        ::close(fd);
        ::unlink(path);
    }
}

TEST_CASE(hw_info_counts_devices_from_a_sysfs_tree) {
    // A fake /sys/bus/pci/devices: two B200s, one NVSwitch, one ConnectX, one EFA, one unrelated NIC.
    char tmpl[] = "/tmp/nixl_hwinfo_XXXXXX";
    CHECK(::mkdtemp(tmpl) != nullptr);
    const std::string root = tmpl;
    auto add = [&](const std::string &name, const char *vendor, const char *cls, const char *device) {
        const std::string d = root + "/" + name;
        CHECK(::mkdir(d.c_str(), 0755) == 0);
        std::ofstream(d + "/vendor") << vendor << "\n";
        std::ofstream(d + "/class") << cls << "\n";
        std::ofstream(d + "/device") << device << "\n";
    };
    add("0000:1b:00.0", "0x10de", "0x030200", "0x2901");
    add("0000:43:00.0", "0x10de", "0x030200", "0x2901");
    add("0000:05:00.0", "0x10de", "0x068000", "0x22a3");
    add("0000:0c:00.0", "0x15b3", "0x020700", "0x1021");
    add("0000:0d:00.0", "0x1d0f", "0x020000", "0xefa2");
    add("0000:0e:00.0", "0x8086", "0x020000", "0x1572");
    const nixl::hwInfo hw = nixl::hwInfo::scan(root);
    CHECK_EQ(hw.numNvidiaGpus, 2u);
    CHECK_EQ(hw.numNvSwitches, 1u);
    CHECK_EQ(hw.numIbDevices, 1u);
    CHECK_EQ(hw.numEfaDevices, 1u);
    CHECK_EQ(hw.numAmdGpus, 0u);
    CHECK(hw.toString().find("nvidia_gpus=2") != std::string::npos);
    const nixl::hwInfo none = nixl::hwInfo::scan(root + "/does_not_exist");
    CHECK_EQ(none.numNvidiaGpus, 0u);
    std::filesystem::remove_all(root);
}

TEST_CASE(topology_orders_network_interfaces_by_their_place_in_the_pci_tree) {
    // A node in the shape of an 8-GPU NVLink box, two of its four PCIe switches shown: each switch carries GPUs and the
    // NICs meant for them; the two sockets are NUMA nodes 0 and 1; a management NIC hangs off the chipset.
    //   pci0000:15 (numa 0) - 15:01.0 - 16:00.0 +- 17:00.0 - 1b:00.0  GPU 0
    //                                           +- 17:01.0 - 1c:00.0  NIC ib0
    //                                           +- 17:02.0 - 1d:00.0  GPU 1
    //   pci0000:00 (numa 0) - 00:1f.0 - 02:00.0                       NIC eno1 (management)
    //   pci0000:97 (numa 1) - 97:01.0 - 98:00.0 +- 99:00.0 - 9b:00.0  GPU 2
    //                                           +- 99:01.0 - 9c:00.0  NIC ib1 (two ports: ib1, ib1b)
    char tmpl[] = "/tmp/nixl_topo_XXXXXX";
    CHECK(::mkdtemp(tmpl) != nullptr);
    const std::string base = tmpl, bus = base + "/bus";
    CHECK(::mkdir(bus.c_str(), 0755) == 0);
    auto mkdirs = [](const std::string &path) {
        for (size_t i = 1; i <= path.size(); ++i)
            if (i == path.size() || path[i] == '/') ::mkdir(path.substr(0, i).c_str(), 0755);
    };
    auto add = [&](const std::string &chain, const char *vendor, const char *cls, int numa, std::vector<std::string> ifs = {}) {
        const std::string dir = base + "/devices/" + chain;
        mkdirs(dir);
        std::ofstream(dir + "/vendor") << vendor << "\n";
        std::ofstream(dir + "/class") << cls << "\n";
        std::ofstream(dir + "/device") << "0x2901\n";
        std::ofstream(dir + "/numa_node") << numa << "\n";
        for (const auto &i : ifs) mkdirs(dir + "/net/" + i);
        const std::string bdf = chain.substr(chain.rfind('/') + 1);
        CHECK(::symlink(dir.c_str(), (bus + "/" + bdf).c_str()) == 0);
    };
    const std::string sw0 = "pci0000:15/0000:15:01.0/0000:16:00.0/", sw1 = "pci0000:97/0000:97:01.0/0000:98:00.0/";
    add(sw0 + "0000:17:00.0/0000:1b:00.0", "0x10de", "0x030200", 0);
    add(sw0 + "0000:17:01.0/0000:1c:00.0", "0x15b3", "0x020700", 0, {"ib0"});
    add(sw0 + "0000:17:02.0/0000:1d:00.0", "0x10de", "0x030200", 0);
    add("pci0000:00/0000:00:1f.0/0000:02:00.0", "0x8086", "0x020000", 0, {"eno1"});
    add(sw1 + "0000:99:00.0/0000:9b:00.0", "0x10de", "0x030200", 1);
    add(sw1 + "0000:99:01.0/0000:9c:00.0", "0x15b3", "0x020700", 1, {"ib1", "ib1b"});
    add("pci0000:00/0000:00:14.0", "0x8086", "0x0c0330", 0); // a USB controller: neither GPU nor NIC

    const nixl::pciTopology t = nixl::pciTopology::scan(bus);
    CHECK_EQ(t.gpus().size(), size_t(3));
    CHECK_EQ(t.nics().size(), size_t(3));
    CHECK(t.gpus()[0].bdf == "0000:1b:00.0" && t.gpus()[2].bdf == "0000:9b:00.0" && t.gpus()[2].numaNode == 1);
    CHECK(t.gpus()[0].chain.size() == 5 && t.gpus()[0].chain.front() == "pci0000:15" && t.gpus()[0].chain.back() == "0000:1b:00.0");
    // under one switch: up to the switch and down again
    const nixl::pciDevice &ib0 = *t.nicsNearGpu(0).front();
    CHECK(ib0.bdf == "0000:1c:00.0");
    CHECK_EQ(nixl::pciTopology::distance(t.gpus()[0], ib0), 4);
    CHECK_EQ(nixl::pciTopology::distance(t.gpus()[1], ib0), 4);
    // another root complex on the same socket costs 100 more, another socket 100 more again
    CHECK((t.interfacesNearGpu(0) == std::vector<std::string>{"ib0", "eno1", "ib1", "ib1b"}));
    CHECK((t.interfacesNearGpu(2) == std::vector<std::string>{"ib1", "ib1b", "eno1", "ib0"}));
    CHECK(nixl::pciTopology::distance(t.gpus()[0], *t.nicsNearGpu(0)[1]) > 100 && nixl::pciTopology::distance(t.gpus()[0], *t.nicsNearGpu(0)[1]) < 200);
    CHECK(nixl::pciTopology::distance(t.gpus()[0], *t.nicsNearGpu(0)[2]) > 200);
    // no such GPU: bus order
    CHECK((t.interfacesNearGpu(99) == std::vector<std::string>{"eno1", "ib0", "ib1", "ib1b"}));
    CHECK(t.toString().find("gpu2 0000:9b:00.0 numa 1: 0000:9c:00.0(ib1,ib1b;d=4)") != std::string::npos);
    CHECK(nixl::pciTopology::scan(base + "/absent").gpus().empty());
    std::filesystem::remove_all(base);
}

TEST_CASE(topology_of_an_eight_gpu_box_gives_every_gpu_its_own_nic_first) {
    // The shape of an HGX B200 node with eight fabric NICs (two sockets, two root complexes each, one PCIe switch per
    // root complex with two GPUs and their two NICs behind separate downstream ports of it): every GPU's nearest NIC is
    // the one behind the neighbouring port, then the other NIC of its switch, then the same socket, then the other.
    char tmpl[] = "/tmp/nixl_topo8_XXXXXX";
    CHECK(::mkdtemp(tmpl) != nullptr);
    const std::string base = tmpl, bus = base + "/bus";
    CHECK(::mkdir(bus.c_str(), 0755) == 0);
    auto mkdirs = [](const std::string &path) {
        for (size_t i = 1; i <= path.size(); ++i)
            if (i == path.size() || path[i] == '/') ::mkdir(path.substr(0, i).c_str(), 0755);
    };
    auto add = [&](const std::string &chain, const char *vendor, const char *cls, int numa, const std::string &netif) {
        const std::string dir = base + "/devices/" + chain;
        mkdirs(dir);
        std::ofstream(dir + "/vendor") << vendor << "\n";
        std::ofstream(dir + "/class") << cls << "\n";
        std::ofstream(dir + "/device") << "0x2901\n";
        std::ofstream(dir + "/numa_node") << numa << "\n";
        if (!netif.empty()) mkdirs(dir + "/net/" + netif);
        CHECK(::symlink(dir.c_str(), (bus + "/" + chain.substr(chain.rfind('/') + 1)).c_str()) == 0);
    };
    char buf[256];
    // root complexes 0x10, 0x30 on socket 0 and 0x90, 0xb0 on socket 1; bus numbers grow with the GPU number
    const int roots[4] = {0x10, 0x30, 0x90, 0xb0};
    for (int sw = 0; sw < 4; ++sw) {
        const int r = roots[sw], numa = sw / 2;
        for (int k = 0; k < 2; ++k) { // two GPU + NIC pairs per switch; a pair shares a second-level bridge
            const int gpu = sw * 2 + k;
            std::snprintf(buf, sizeof(buf), "pci0000:%02x/0000:%02x:01.0/0000:%02x:00.0/0000:%02x:0%d.0/0000:%02x:00.0/0000:%02x:00.0", r, r, r + 1, r + 2, k,
                          r + 3 + 4 * k, r + 4 + 4 * k);
            add(buf, "0x10de", "0x030200", numa, "");
            std::snprintf(buf, sizeof(buf), "pci0000:%02x/0000:%02x:01.0/0000:%02x:00.0/0000:%02x:0%d.0/0000:%02x:00.0/0000:%02x:01.0", r, r, r + 1, r + 2, k,
                          r + 3 + 4 * k, r + 4 + 4 * k);
            add(buf, "0x1d0f", "0x020000", numa, "rdmap" + std::to_string(gpu));
        }
    }
    const nixl::pciTopology t = nixl::pciTopology::scan(bus);
    CHECK_EQ(t.gpus().size(), size_t(8));
    CHECK_EQ(t.nics().size(), size_t(8));
    for (size_t g = 0; g < 8; ++g) {
        const std::vector<std::string> order = t.interfacesNearGpu(g);
        CHECK_EQ(order.size(), size_t(8));
        CHECK(order[0] == "rdmap" + std::to_string(g));           // its own
        CHECK(order[1] == "rdmap" + std::to_string(g ^ 1));       // the other pair of its switch
        const size_t socket_first = (g / 4) * 4;
        for (size_t k = 2; k < 4; ++k) CHECK(order[k] == "rdmap" + std::to_string(socket_first + (((g % 4) / 2) ^ 1) * 2 + (k - 2))); // same socket, other root
        for (size_t k = 4; k < 8; ++k) CHECK(order[k][5] - '0' >= 0 && (static_cast<size_t>(order[k][5] - '0') / 4) != g / 4);            // the other socket last
        CHECK_EQ(nixl::pciTopology::distance(t.gpus()[g], *t.nicsNearGpu(g)[0]), 2);
        CHECK(nixl::pciTopology::distance(t.gpus()[g], *t.nicsNearGpu(g)[1]) < 100);
        CHECK(nixl::pciTopology::distance(t.gpus()[g], *t.nicsNearGpu(g)[2]) > 100 && nixl::pciTopology::distance(t.gpus()[g], *t.nicsNearGpu(g)[2]) < 200);
        CHECK(nixl::pciTopology::distance(t.gpus()[g], *t.nicsNearGpu(g)[7]) > 200);
    }
    std::filesystem::remove_all(base);
}

TEST_CASE(clocks_durations_identifiers_and_strings) {
    using namespace nixl_util;
    // the cycle-counter clock follows the steady clock
    const uint64_t f0 = FastClock::ns(), s0 = nowNs();
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
    const uint64_t f1 = FastClock::ns(), s1 = nowNs();
    CHECK(f1 > f0);
    const double ratio = static_cast<double>(f1 - f0) / static_cast<double>(s1 - s0);
    CHECK(ratio > 0.95 && ratio < 1.05);
    CHECK(nowUs() >= s1 / 1000 && nowMs() >= static_cast<int64_t>(s1 / 1000000));

    std::chrono::nanoseconds d{};
    CHECK(parseDuration("1.5s", d) && d == std::chrono::milliseconds(1500));
    CHECK(parseDuration("250ms", d) && d == std::chrono::milliseconds(250));
    CHECK(parseDuration("40us", d) && d == std::chrono::microseconds(40));
    CHECK(parseDuration("40", d) && d == std::chrono::microseconds(40)); // bare numbers are microseconds
    CHECK(parseDuration("7ns", d) && d == std::chrono::nanoseconds(7));
    CHECK(parseDuration("2min", d) && d == std::chrono::seconds(120));
    CHECK(!parseDuration("", d) && !parseDuration("fast", d) && !parseDuration("3 parsecs", d) && !parseDuration("-1s", d));
    CHECK(formatDuration(std::chrono::milliseconds(2500)) == "2.5s");
    CHECK(formatDuration(std::chrono::microseconds(120000)) == "120ms");
    CHECK(formatDuration(std::chrono::nanoseconds(35000)) == "35us");
    CHECK(formatDuration(std::chrono::nanoseconds(800)) == "800ns");

    CHECK(!hostName().empty());
    const std::string u = uuidV4(), v = uuidV4();
    CHECK(u != v && u.size() == 36 && u[8] == '-' && u[13] == '-' && u[18] == '-' && u[23] == '-');
    CHECK(u[14] == '4' && (u[19] == '8' || u[19] == '9' || u[19] == 'a' || u[19] == 'b'));
    CHECK(random64() != random64());

    CHECK((split("a,b,,c", ',') == std::vector<std::string>{"a", "b", "c"}));
    CHECK((split("a,b,,c", ',', true) == std::vector<std::string>{"a", "b", "", "c"}));
    CHECK(split("", ',').empty());
    CHECK(trim("  x y \t\n") == "x y" && trim(" \t ").empty());
}

TEST_MAIN()

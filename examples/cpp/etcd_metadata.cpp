// Two agents find each other through etcd instead of passing metadata blobs by hand.
//
//   NIXL_ETCD_ENDPOINTS=http://127.0.0.1:2379 NIXL_PLUGIN_DIR=nixl_b200/lib/plugins /tmp/etcd_metadata
//
// built like two_agents.cpp.  The steps are those of the reference's examples/cpp/nixl_etcd_example.cpp: publish the
// full metadata, fetch the peer's, move data; then publish only some registrations under a label of their own
// ("partial metadata"), fetch that label; finally withdraw the metadata and see the peer forget it (through the watch on
// the key, or the poll that stands in for it).  The endpoint is etcd's v3 JSON gateway (every etcd since 3.2 serves it).
// NIXL_ETCD_NAMESPACE changes the key prefix (default /nixl/agents).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#include "nixl.h"

namespace {
bool waitFor(const char *what, const std::function<bool()> &ready, int seconds = 15) {
    const auto end = std::chrono::steady_clock::now() + std::chrono::seconds(seconds);
    while (!ready()) {
        if (std::chrono::steady_clock::now() > end) {
            std::fprintf(stderr, "timed out waiting for %s\n", what);
            return false;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(10));
    }
    return true;
}
} // namespace

int main() {
    if (!std::getenv("NIXL_ETCD_ENDPOINTS")) {
        std::fprintf(stderr, "set NIXL_ETCD_ENDPOINTS (e.g. http://127.0.0.1:2379)\n");
        return 1;
    }
    nixlAgentConfig cfg(false);
    nixlAgent prefill("prefill", cfg), decode("decode", cfg);
    nixlBackendH *bp = nullptr, *bd = nullptr;
    if (prefill.createBackend("NVLINK", {}, bp) != NIXL_SUCCESS || decode.createBackend("NVLINK", {}, bd) != NIXL_SUCCESS) {
        std::fprintf(stderr, "backend not available (is NIXL_PLUGIN_DIR set?)\n");
        return 1;
    }
    std::vector<char> kv(1 << 20, 'k'), scratch(1 << 16, 's'), landing(1 << 20, 0), extra(1 << 16, 0);
    nixl_reg_dlist_t reg_kv(DRAM_SEG), reg_scratch(DRAM_SEG), reg_landing(DRAM_SEG), reg_extra(DRAM_SEG);
    reg_kv.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(kv.data()), kv.size(), 0, ""));
    reg_scratch.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(scratch.data()), scratch.size(), 0, ""));
    reg_landing.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(landing.data()), landing.size(), 0, ""));
    reg_extra.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(extra.data()), extra.size(), 0, ""));
    if (prefill.registerMem(reg_kv) != NIXL_SUCCESS || prefill.registerMem(reg_scratch) != NIXL_SUCCESS ||
        decode.registerMem(reg_landing) != NIXL_SUCCESS)
        return 2;

    // 1. full metadata through the store: <namespace>/<agent>/metadata
    if (prefill.sendLocalMD() != NIXL_SUCCESS || decode.sendLocalMD() != NIXL_SUCCESS) return 3;
    if (prefill.fetchRemoteMD("decode") != NIXL_SUCCESS || decode.fetchRemoteMD("prefill") != NIXL_SUCCESS) return 3;
    nixl_xfer_dlist_t none(DRAM_SEG);
    if (!waitFor("the peers' metadata", [&] {
            return prefill.checkRemoteMD("decode", none) == NIXL_SUCCESS && decode.checkRemoteMD("prefill", none) == NIXL_SUCCESS;
        }))
        return 3;
    std::printf("both agents know each other through the store\n");

    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(kv.data()), kv.size(), 0));
    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(landing.data()), landing.size(), 0));
    nixlXferReqH *req = nullptr;
    if (prefill.createXferReq(NIXL_WRITE, l, r, "decode", req) != NIXL_SUCCESS) return 4;
    nixl_status_t st = prefill.postXferReq(req);
    while (st == NIXL_IN_PROG) st = prefill.getXferStatus(req);
    if (st != NIXL_SUCCESS || std::memcmp(kv.data(), landing.data(), kv.size()) != 0) return 4;
    prefill.releaseXferReq(req);
    std::printf("moved %zu bytes\n", kv.size());

    // 2. partial metadata: decode registers one more buffer and publishes just that, under a label of its own
    if (decode.registerMem(reg_extra) != NIXL_SUCCESS) return 5;
    nixl_opt_args_t label;
    label.metadataLabel = "extra_buffers";
    if (decode.sendLocalPartialMD(reg_extra, &label) != NIXL_SUCCESS) return 5;
    if (prefill.fetchRemoteMD("decode", &label) != NIXL_SUCCESS) return 5;
    nixl_xfer_dlist_t want(DRAM_SEG);
    want.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(extra.data()), extra.size(), 0));
    if (!waitFor("the partial metadata", [&] { return prefill.checkRemoteMD("decode", want) == NIXL_SUCCESS; })) return 5;
    nixl_xfer_dlist_t l2(DRAM_SEG);
    l2.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(scratch.data()), scratch.size(), 0));
    if (prefill.createXferReq(NIXL_WRITE, l2, want, "decode", req) != NIXL_SUCCESS) return 5;
    st = prefill.postXferReq(req);
    while (st == NIXL_IN_PROG) st = prefill.getXferStatus(req);
    if (st != NIXL_SUCCESS || std::memcmp(scratch.data(), extra.data(), extra.size()) != 0) return 5;
    prefill.releaseXferReq(req);
    std::printf("reached a buffer that was published on its own under label '%s'\n", label.metadataLabel.c_str());

    // 3. decode withdraws: its keys go away and prefill, which watches what it fetched, forgets it
    if (decode.invalidateLocalMD() != NIXL_SUCCESS) return 6;
    if (!waitFor("the invalidation", [&] { return prefill.checkRemoteMD("decode", none) != NIXL_SUCCESS; })) return 6;
    std::printf("decode withdrew its metadata and prefill dropped it\n");

    prefill.deregisterMem(reg_kv);
    prefill.deregisterMem(reg_scratch);
    decode.deregisterMem(reg_landing);
    decode.deregisterMem(reg_extra);
    return 0;
}

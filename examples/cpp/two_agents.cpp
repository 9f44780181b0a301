// Two agents in one process move a buffer with the C++ API and signal completion with a notification.
//
//   g++ -std=c++20 -I csrc/include examples/cpp/two_agents.cpp -L nixl_b200/lib -lnixl \
//       -Wl,-rpath,$PWD/nixl_b200/lib -o /tmp/two_agents && NIXL_PLUGIN_DIR=nixl_b200/lib/plugins /tmp/two_agents
//
// The same calls work between processes once the metadata blob travels by any side channel
// (or through sendLocalMD / fetchRemoteMD with a listener, a TCPStore or etcd).
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "nixl.h"

int main(int argc, char **argv) {
    // "two_agents TCP" runs the same calls over the socket backend, the one that also reaches another host.
    const std::string backend = argc > 1 ? argv[1] : "NVLINK";
    nixlAgentConfig cfg(false);
    nixlAgent prefill("prefill", cfg), decode("decode", cfg);
    nixlBackendH *bp = nullptr, *bd = nullptr;
    if (prefill.createBackend(backend, {}, bp) != NIXL_SUCCESS || decode.createBackend(backend, {}, bd) != NIXL_SUCCESS) {
        std::fprintf(stderr, "backend not available (is NIXL_PLUGIN_DIR set?)\n");
        return 1;
    }
    std::vector<char> src(1 << 20, 'k'), dst(1 << 20, 0);
    nixl_reg_dlist_t rs(DRAM_SEG), rd(DRAM_SEG);
    rs.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0, ""));
    rd.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0, ""));
    if (prefill.registerMem(rs) != NIXL_SUCCESS || decode.registerMem(rd) != NIXL_SUCCESS) return 2;

    nixl_blob_t md;
    std::string who;
    decode.getLocalMD(md);                    // what the other side needs to reach `decode`
    if (prefill.loadRemoteMD(md, who) != NIXL_SUCCESS) return 3;

    nixl_xfer_dlist_t l(DRAM_SEG), r(DRAM_SEG);
    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src.data()), src.size(), 0));
    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst.data()), dst.size(), 0));
    nixl_opt_args_t opt;
    opt.notif = "kv-ready";                   // delivered to `decode` after the data
    nixlXferReqH *req = nullptr;
    if (prefill.createXferReq(NIXL_WRITE, l, r, who, req, &opt) != NIXL_SUCCESS) return 4;
    nixl_status_t st = prefill.postXferReq(req);
    while (st == NIXL_IN_PROG) st = prefill.getXferStatus(req);
    if (st != NIXL_SUCCESS) return 5;

    nixl_notifs_t notifs;
    while (notifs.empty()) decode.getNotifs(notifs);
    nixlBackendH *used = nullptr;
    prefill.queryXferBackend(req, used);
    std::printf("backend %s: moved %zu bytes to %s, %s says \"%s\", data %s\n", backend.c_str(), src.size(), who.c_str(), notifs.begin()->first.c_str(),
                notifs.begin()->second.front().c_str(), std::memcmp(src.data(), dst.data(), src.size()) == 0 ? "identical" : "DIFFERENT");
    prefill.releaseXferReq(req);
    prefill.deregisterMem(rs);
    decode.deregisterMem(rd);
    return 0;
}

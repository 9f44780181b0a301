// nixlbench: native sweep driver for the C++ agent API (two agents in one process).
//
// Role parity with the reference's benchmark/nixlbench (block-size and batch sweeps
// src/main.cpp:107,:220; pipelined transfer loop worker/nixl/nixl_worker.cpp:1708-1831;
// statistics utils.cpp:1336: GB/s, average latency, prepare / post / transfer times with p99).
// Scope here: initiator and target agents live in this process; memory is VRAM on two GPUs
// (or one), or DRAM; the backend is chosen by name.  Multi-process sweeps are driven by
// benchmarks/nixlbench.py.
//
//   nixlbench [--backend NVLINK] [--op WRITE|READ] [--mem VRAM|DRAM] [--src-dev 0] [--dst-dev 1]
//             [--min 4096] [--max 1073741824] [--batch 1] [--batch-max N] [--iters 1000] [--warmup 100]
//             [--depth 1] [--num-threads 1] [--enable-pt] [--copy-path vector|bulk] [--param key=value]... [--check]
//             [--prepared] [--recreate] [--reregister] [--scatter] [--config file]
//             [--file path [--num-files N] [--direct]]      storage mode (POSIX, GDS, GDS_MT backends)
//             [--backend OBJ|AZURE_BLOB --param bucket=... [--obj-prefix name]]   object stores: one object per block
//             [--scheme pairwise|onetomany|manytoone|tp --num-initiator-dev N --num-target-dev M]
//
// --role target --listen-port P  /  --role initiator --peer-ip A --peer-port P: the pairwise sweep between two
// processes, which may sit on two hosts (then with --backend TCP): the target registers its buffer and listens for
// metadata on port P; the initiator fetches the target's metadata there, sends its own, learns the buffer's address
// from a notification, runs the sweep and says when it is through.  --check reads what it wrote back over the backend.
// With --etcd-endpoints URL on both sides (the reference's way to rendezvous) neither needs the other's address: both
// publish their metadata in that etcd and fetch the other's by name.
//
// --scheme onetomany: one initiator (--src-dev) posts the same request to M targets at once; manytoone: N
// initiators post to one target (--dst-dev) at once, which is the pattern that shows what a receiver's ingress
// sustains; tp: N initiators x M targets, every initiator sends 1/M of each block to every target (tensor-parallel
// resharding).  One agent per endpoint, all in this process (VRAM: one endpoint per GPU; DRAM: host buffers); the
// figure is the sum over all flows.
//
// --num-threads T: T worker threads share the batch (thread t owns descriptors t, t + T, ...), each with its own
// requests and pipeline (the reference's worker threads, worker/nixl/nixl_worker.cpp:125,:1834); --enable-pt gives
// the agents a progress thread.
//
// --prepared builds requests with prepXferDlist + makeXferReq (the reference's prepared_xfer),
// --recreate creates and releases the request on every iteration (recreate_xfer), --reregister
// registers and deregisters the source buffer on every iteration (reregister_mem), --config reads
// "option=value" lines (config_file).  In storage mode the target side is a set of files owned by
// the same agent: WRITE stores memory into the files, READ loads it back (filepath / num_files /
// storage_enable_direct of the reference).
#include <algorithm>
#include <barrier>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <fstream>
#include <unistd.h>

#include <cuda_runtime.h>

#include "nixl.h"

namespace {
using clk = std::chrono::steady_clock;
double us(clk::time_point a, clk::time_point b) { return std::chrono::duration<double, std::micro>(b - a).count(); }

struct Args {
    std::string backend = "NVLINK", op = "WRITE", mem = "VRAM", copy_path = "vector";
    int src_dev = 0, dst_dev = -1, batch = 1, iters = 1000, warmup = 100, depth = 1;
    size_t min = 4096, max = size_t(1) << 30, total = size_t(8) << 30;
    bool check = false, prepared = false, recreate = false, reregister = false, direct = false;
    bool scatter = false; // target blocks of a batch in reverse order: no descriptor continues its predecessor
    std::string scheme = "pairwise"; // pairwise | onetomany | manytoone | tp (benchmark/nixlbench/src/utils/utils.h:122-125 of the reference)
    int num_initiator_dev = 1, num_target_dev = 1;
    int batch_max = 0, num_files = 1;
    int num_threads = 1;    // worker threads of the pairwise scheme, each with its share of the batch
    bool enable_pt = false; // agents with a progress thread
    std::string file; // storage mode when set
    std::string obj_prefix = "nixlbench";
    nixl_b_params_t extra; // --param key=value, passed to the backend
    // two processes (on one host or two): "target" owns the destination buffer and listens, "initiator" finds it there
    std::string etcd; // two processes find each other through this etcd instead of a listener's address
    std::string role, peer_ip = "127.0.0.1";
    int peer_port = 0, listen_port = 0;
};

// One option (with its value, if it takes one).  False for an unknown option.
bool setOption(Args &a, const std::string &k, const std::string &v) {
    if (k == "--backend") a.backend = v;
    else if (k == "--op") a.op = v;
    else if (k == "--mem") a.mem = v;
    else if (k == "--copy-path") a.copy_path = v;
    else if (k == "--scheme") a.scheme = v;
    else if (k == "--num-initiator-dev") a.num_initiator_dev = std::max(1, std::atoi(v.c_str()));
    else if (k == "--num-target-dev") a.num_target_dev = std::max(1, std::atoi(v.c_str()));
    else if (k == "--src-dev") a.src_dev = std::atoi(v.c_str());
    else if (k == "--dst-dev") a.dst_dev = std::atoi(v.c_str());
    else if (k == "--batch") a.batch = std::max(1, std::atoi(v.c_str()));
    else if (k == "--batch-max") a.batch_max = std::atoi(v.c_str());
    else if (k == "--iters") a.iters = std::atoi(v.c_str());
    else if (k == "--warmup") a.warmup = std::atoi(v.c_str());
    else if (k == "--depth") a.depth = std::max(1, std::atoi(v.c_str()));
    else if (k == "--num-threads") a.num_threads = std::max(1, std::atoi(v.c_str()));
    else if (k == "--min") a.min = std::strtoull(v.c_str(), nullptr, 0);
    else if (k == "--max") a.max = std::strtoull(v.c_str(), nullptr, 0);
    else if (k == "--total") a.total = std::strtoull(v.c_str(), nullptr, 0);
    else if (k == "--etcd-endpoints") a.etcd = v;
    else if (k == "--role") a.role = v;
    else if (k == "--peer-ip") a.peer_ip = v;
    else if (k == "--peer-port") a.peer_port = std::atoi(v.c_str());
    else if (k == "--listen-port") a.listen_port = std::atoi(v.c_str());
    else if (k == "--file") a.file = v;
    else if (k == "--obj-prefix") a.obj_prefix = v;
    else if (k == "--num-files") a.num_files = std::max(1, std::atoi(v.c_str()));
    else if (k == "--param") {
        const size_t eq = v.find('=');
        if (eq != std::string::npos) a.extra[v.substr(0, eq)] = v.substr(eq + 1);
    } else return false;
    return true;
}
bool setFlag(Args &a, const std::string &k) {
    if (k == "--check") a.check = true;
    else if (k == "--enable-pt") a.enable_pt = true;
    else if (k == "--prepared") a.prepared = true;
    else if (k == "--recreate") a.recreate = true;
    else if (k == "--reregister") a.reregister = true;
    else if (k == "--direct") a.direct = true;
    else if (k == "--scatter") a.scatter = true;
    else return false;
    return true;
}
struct Spelling;
std::string canonicalName(const std::string &k);
bool loadConfig(Args &a, const std::string &path) {
    std::ifstream f(path);
    if (!f) return false;
    std::string line;
    while (std::getline(f, line)) {
        const size_t hash = line.find('#');
        if (hash != std::string::npos) line.erase(hash);
        while (!line.empty() && std::isspace(static_cast<unsigned char>(line.back()))) line.pop_back();
        size_t b = 0;
        while (b < line.size() && std::isspace(static_cast<unsigned char>(line[b]))) ++b;
        line.erase(0, b);
        if (line.empty()) continue;
        const size_t eq = line.find('=');
        std::string k = "--" + (eq == std::string::npos ? line : line.substr(0, eq));
        k = canonicalName(k); // underscores, and the reference's long names
        const std::string v = eq == std::string::npos ? "" : line.substr(eq + 1);
        if (eq == std::string::npos || v == "true" || v == "1") {
            if (setFlag(a, k)) continue;
        }
        if (v == "false" || v == "0") {
            Args probe;
            if (setFlag(probe, k)) continue; // a flag explicitly switched off
        }
        if (!setOption(a, k, v)) {
            std::fprintf(stderr, "%s: unknown option %s\n", path.c_str(), line.c_str());
            return false;
        }
    }
    return true;
}

// Accepts the spellings of the reference's nixlbench (benchmark/nixlbench/src/utils/utils.cpp:
// gflags names with underscores, `--name=value`) next to this tool's own short ones.
struct Spelling {
    enum Kind { OPTION, IGNORED, POSIX_API, PARAM } kind = OPTION;
    std::string name;  // this tool's option
    std::string param; // backend parameter for PARAM
};
Spelling canonical(std::string k) {
    for (char &c : k)
        if (c == '_') c = '-';
    static const std::map<std::string, std::string> same = {
        {"--start-block-size", "--min"},     {"--max-block-size", "--max"},       {"--start-batch-size", "--batch"},
        {"--max-batch-size", "--batch-max"}, {"--num-iter", "--iters"},           {"--warmup-iter", "--warmup"},
        {"--op-type", "--op"},               {"--initiator-seg-type", "--mem"},   {"--check-consistency", "--check"},
        {"--total-buffer-size", "--total"},  {"--pipeline-depth", "--depth"},     {"--recreate-xfer", "--recreate"},
        {"--reregister-mem", "--reregister"}, {"--prepared-xfer", "--prepared"},  {"--config-file", "--config"},
        {"--filepath", "--file"},            {"--storage-enable-direct", "--direct"},
    };
    static const std::map<std::string, std::string> params = {
        {"--posix-ios-pool-size", "ios_pool_size"}, {"--posix-kernel-queue-size", "kernel_queue_size"},
        {"--gds-mt-num-threads", "thread_count"},   {"--hf3fs-iopool-size", "iopool_size"},
        {"--obj-bucket-name", "bucket"},            {"--azure-blob-container-name", "container_name"},
        {"--obj-access-key", "access_key"},         {"--obj-secret-key", "secret_key"},
        {"--obj-session-token", "session_token"},   {"--obj-scheme", "scheme"},
        {"--obj-region", "region"},                 {"--obj-use-virtual-addressing", "use_virtual_addressing"},
        {"--obj-endpoint-override", "endpoint_override"}, {"--obj-req-checksum", "req_checksum"},
        {"--obj-ca-bundle", "ca_bundle"},           {"--obj-crt-min-limit", "crtMinLimit"},
        {"--azure-blob-account-url", "account_url"}, {"--azure-blob-connection-string", "connection_string"},
    };
    // One process drives both agents here: there is no runtime to rendezvous through, no second
    // worker type and one initiator / target device each.
    static const char *ignored[] = {"--runtime-type", "--worker-type", "--mode",
                                    "--progress-threads", "--device-list", "--target-seg-type",
                                    "--large-blk-iter-ftr", "--benchmark-group"};
    Spelling sp;
    sp.name = k;
    if (auto it = same.find(k); it != same.end()) sp.name = it->second;
    else if (auto pit = params.find(k); pit != params.end()) {
        sp.kind = Spelling::PARAM;
        sp.param = pit->second;
    } else if (k == "--posix-api-type") sp.kind = Spelling::POSIX_API;
    else
        for (const char *name : ignored)
            if (k == name) sp.kind = Spelling::IGNORED;
    return sp;
}

std::string canonicalName(const std::string &k) { return canonical(k).name; }

double pct(std::vector<double> &v, double q) {
    if (v.empty()) return 0;
    std::sort(v.begin(), v.end());
    return v[std::min(v.size() - 1, static_cast<size_t>(q * v.size()))];
}
// One-to-many / many-to-one / tp: a flow per (initiator, target) pair, all posted together every iteration.
//   onetomany  one initiator (--src-dev), M targets: the same request goes to every target
//   manytoone  N initiators, one target (--dst-dev): what a receiver's ingress sustains
//   tp         N initiators x M targets (tensor-parallel resharding): every initiator sends 1/M of each block to
//              every target, so a flow's descriptors are block / M bytes
// One agent per endpoint, all in this process.  VRAM: one endpoint per GPU.  DRAM: endpoints are host buffers.
int runScheme(const Args &a, int ndev) {
    const bool vram = a.mem == "VRAM";
    const int n_ini = a.scheme == "onetomany" ? 1 : a.num_initiator_dev;
    const int n_tgt = a.scheme == "manytoone" ? 1 : a.num_target_dev;
    if (vram && n_ini + n_tgt > ndev) {
        std::fprintf(stderr, "--scheme %s needs %d GPUs (found %d)\n", a.scheme.c_str(), n_ini + n_tgt, ndev);
        return 2;
    }
    // Devices: the "one" side keeps the device the options name, the others take the remaining ordinals in order.
    std::vector<int> ini_dev, tgt_dev;
    {
        std::vector<bool> used(std::max(ndev, 1), false);
        auto take = [&](int want) {
            if (!vram) return 0;
            if (want >= 0 && want < ndev && !used[want]) {
                used[want] = true;
                return want;
            }
            for (int d = 0; d < ndev; ++d)
                if (!used[d]) {
                    used[d] = true;
                    return d;
                }
            return 0;
        };
        if (a.scheme == "manytoone") tgt_dev.push_back(take(a.dst_dev >= 0 ? a.dst_dev : 0));
        for (int i = 0; i < n_ini; ++i) ini_dev.push_back(take(i == 0 ? a.src_dev : -1));
        while (static_cast<int>(tgt_dev.size()) < n_tgt) tgt_dev.push_back(take(tgt_dev.empty() ? a.dst_dev : -1));
    }
    const int split = a.scheme == "tp" ? n_tgt : 1; // a block is cut into this many pieces, one per target
    const size_t buf_bytes = std::min(a.total, std::max<size_t>(a.max * std::max(a.batch, a.batch_max), a.max));
    nixlAgentConfig cfg(a.enable_pt);
    nixl_b_params_t params;
    params["copy_path"] = a.copy_path;
    for (auto &kv : a.extra) params[kv.first] = kv.second;
    const nixl_mem_t mt = vram ? VRAM_SEG : DRAM_SEG;
    struct Side {
        int dev = 0;
        char *buf = nullptr; // initiator: one source region; target: one landing region per initiator
        size_t bytes = 0;
        std::string name;
        std::unique_ptr<nixlAgent> agent;
    };
    auto make = [&](int dev, const std::string &name, size_t bytes, int fill, Side &s) {
        s.dev = dev;
        s.bytes = bytes;
        s.name = name;
        if (vram) {
            cudaSetDevice(dev);
            if (cudaMalloc(reinterpret_cast<void **>(&s.buf), bytes) != cudaSuccess) return false;
            cudaMemset(s.buf, fill, bytes);
            cudaDeviceSynchronize();
        } else {
            void *p = nullptr;
            if (posix_memalign(&p, 4096, bytes) != 0) return false;
            s.buf = static_cast<char *>(p);
            std::memset(s.buf, fill, bytes);
        }
        s.agent = std::make_unique<nixlAgent>(name, cfg);
        nixlBackendH *b = nullptr;
        if (s.agent->createBackend(a.backend, params, b) != NIXL_SUCCESS) return false;
        nixl_reg_dlist_t reg(mt);
        reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(s.buf), bytes, vram ? dev : 0, ""));
        return s.agent->registerMem(reg) == NIXL_SUCCESS;
    };
    const nixl_xfer_op_t op = a.op == "READ" ? NIXL_READ : NIXL_WRITE;
    // WRITE: initiators hold the pattern, targets start at zero; READ: the other way round.
    std::vector<Side> inis(n_ini), tgts(n_tgt);
    for (int i = 0; i < n_ini; ++i)
        if (!make(ini_dev[i], "ini" + std::to_string(i), buf_bytes, op == NIXL_WRITE ? 0x5a : 0, inis[i])) return 3;
    for (int j = 0; j < n_tgt; ++j)
        if (!make(tgt_dev[j], "tgt" + std::to_string(j), buf_bytes * n_ini, op == NIXL_WRITE ? 0 : 0x5a, tgts[j])) return 3;
    for (auto &ini : inis)
        for (auto &tgt : tgts) {
            nixl_blob_t md;
            std::string name;
            tgt.agent->getLocalMD(md);
            if (ini.agent->loadRemoteMD(md, name) != NIXL_SUCCESS) return 6;
        }
    const int flows = n_ini * n_tgt;
    std::printf("# scheme %s: %d initiator(s) x %d target(s), %d flow(s), %s\n", a.scheme.c_str(), n_ini, n_tgt, flows, a.mem.c_str());
    std::printf("%-12s %6s %10s %12s %10s %10s\n", "block", "batch", "GB/s", "GB/s_per_flow", "p50_us", "p99_us");
    for (int batch = a.batch; batch <= std::max(a.batch, a.batch_max); batch *= 2)
    for (size_t block = a.min; block <= a.max && block * batch <= buf_bytes; block *= 2) {
        const size_t piece = block / split; // bytes per descriptor of one flow
        if (piece == 0) continue;
        const size_t per_flow = piece * batch;
        int iters = a.iters, warm = a.warmup;
        if (per_flow * n_tgt > (size_t(64) << 20)) {
            iters = std::max<int>(10, static_cast<int>((size_t(64) << 30) / (per_flow * n_tgt) / 16));
            warm = 3;
        }
        std::vector<nixlXferReqH *> reqs(flows, nullptr);
        for (int i = 0; i < n_ini; ++i)
            for (int j = 0; j < n_tgt; ++j) {
                nixl_xfer_dlist_t l(mt), r(mt);
                char *land = tgts[j].buf + static_cast<size_t>(i) * buf_bytes; // initiator i's region at target j
                for (int k = 0; k < batch; ++k) {
                    // tp: target j receives piece j of every block and packs the pieces densely
                    const size_t loff = static_cast<size_t>(k) * block + (split > 1 ? static_cast<size_t>(j) * piece : 0);
                    const size_t roff = (a.scatter ? static_cast<size_t>(batch - 1 - k) : static_cast<size_t>(k)) * piece;
                    l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(inis[i].buf) + loff, piece, vram ? inis[i].dev : 0));
                    r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(land) + roff, piece, vram ? tgts[j].dev : 0));
                }
                if (inis[i].agent->createXferReq(op, l, r, tgts[j].name, reqs[i * n_tgt + j]) != NIXL_SUCCESS) return 7;
            }
        std::vector<double> step;
        clk::time_point t_begin = clk::now();
        for (int it = 0; it < warm + iters; ++it) {
            if (it == warm) t_begin = clk::now();
            const auto t0 = clk::now();
            std::vector<bool> busy(flows, false);
            for (int f = 0; f < flows; ++f) {
                const nixl_status_t st = inis[f / n_tgt].agent->postXferReq(reqs[f]);
                if (st < 0) return 9;
                busy[f] = st != NIXL_SUCCESS;
            }
            for (bool any = true; any;) {
                any = false;
                for (int f = 0; f < flows; ++f) {
                    if (!busy[f]) continue;
                    const nixl_status_t st = inis[f / n_tgt].agent->getXferStatus(reqs[f]);
                    if (st < 0) return 8;
                    busy[f] = st != NIXL_SUCCESS;
                    any |= busy[f];
                }
            }
            if (it >= warm) step.push_back(us(t0, clk::now()));
        }
        const double wall = us(t_begin, clk::now());
        const double gbs = double(per_flow) * flows * iters / wall / 1e3;
        std::printf("%-12zu %6d %10.2f %12.2f %10.2f %10.2f\n", block, batch, gbs, gbs / flows, pct(step, 0.5), pct(step, 0.99));
        std::fflush(stdout);
        for (int f = 0; f < flows; ++f) inis[f / n_tgt].agent->releaseXferReq(reqs[f]);
        if (a.check) { // every landing region (WRITE) or source region (READ) must hold the pattern where flows wrote
            std::vector<unsigned char> h(std::min<size_t>(per_flow, 1 << 20));
            auto fetch = [&](const Side &s, const char *from) {
                if (vram) {
                    cudaSetDevice(s.dev);
                    cudaDeviceSynchronize();
                    cudaMemcpy(h.data(), from, h.size(), cudaMemcpyDeviceToHost);
                } else {
                    std::memcpy(h.data(), from, h.size());
                }
            };
            for (int i = 0; i < n_ini; ++i)
                for (int j = 0; j < n_tgt; ++j) {
                    if (op == NIXL_WRITE) fetch(tgts[j], tgts[j].buf + static_cast<size_t>(i) * buf_bytes);
                    else if (split == 1 && j == 0) fetch(inis[i], inis[i].buf);
                    else continue;
                    for (unsigned char c : h)
                        if (c != 0x5a) {
                            std::fprintf(stderr, "consistency check failed at block %zu, initiator %d, target %d\n", block, i, j);
                            return 10;
                        }
                }
        }
    }
    return 0;
}
} // namespace


// ---------------------------------------------------------------- two-process mode: the target side
namespace {
int freePort() {
    const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    socklen_t len = sizeof(sa);
    int port = 0;
    if (fd >= 0 && ::bind(fd, reinterpret_cast<sockaddr *>(&sa), sizeof(sa)) == 0 && ::getsockname(fd, reinterpret_cast<sockaddr *>(&sa), &len) == 0)
        port = ntohs(sa.sin_port);
    if (fd >= 0) ::close(fd);
    return port;
}

// Waits for a notification of `from` that starts with `prefix`; the rest of it in `rest`.
bool waitNotif(nixlAgent &agent, const std::string &from, const std::string &prefix, std::string &rest, int seconds) {
    const auto end = clk::now() + std::chrono::seconds(seconds);
    while (clk::now() < end) {
        nixl_notifs_t n;
        agent.getNotifs(n);
        for (const auto &m : n[from])
            if (m.compare(0, prefix.size(), prefix) == 0) {
                rest = m.substr(prefix.size());
                return true;
            }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    return false;
}

int runTarget(const Args &a, bool vram, size_t buf_bytes) {
    if (a.listen_port <= 0 && a.etcd.empty()) {
        std::fprintf(stderr, "--role target needs --listen-port (or --etcd-endpoints)\n");
        return 2;
    }
    const int dev = std::max(0, a.dst_dev);
    void *dst = nullptr;
    if (vram) {
        cudaSetDevice(dev);
        if (cudaMalloc(&dst, buf_bytes) != cudaSuccess) return 3;
        cudaMemset(dst, 0, buf_bytes);
        cudaDeviceSynchronize();
    } else {
        if (posix_memalign(&dst, 4096, buf_bytes) != 0) return 3;
        std::memset(dst, 0, buf_bytes);
    }
    nixlAgentConfig cfg(a.enable_pt, a.listen_port > 0, static_cast<uint16_t>(std::max(0, a.listen_port)));
    nixlAgent tgt("target", cfg);
    nixlBackendH *bt = nullptr;
    nixl_b_params_t params;
    for (auto &kv : a.extra) params[kv.first] = kv.second;
    if (tgt.createBackend(a.backend, params, bt) != NIXL_SUCCESS) {
        std::fprintf(stderr, "cannot create backend %s\n", a.backend.c_str());
        return 4;
    }
    nixl_reg_dlist_t rd(vram ? VRAM_SEG : DRAM_SEG);
    rd.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst), buf_bytes, vram ? dev : 0, ""));
    if (tgt.registerMem(rd) != NIXL_SUCCESS) return 5;
    if (!a.etcd.empty()) { // publish ourselves and ask for the initiator, both through the store
        if (tgt.sendLocalMD() != NIXL_SUCCESS || tgt.fetchRemoteMD("initiator") != NIXL_SUCCESS) return 6;
        std::printf("target: %zu bytes registered, published through %s\n", buf_bytes, a.etcd.c_str());
    } else {
        std::printf("target: %zu bytes registered, listening on port %d\n", buf_bytes, a.listen_port);
    }
    std::fflush(stdout);
    // the initiator's metadata arrives through the listener
    const nixl_xfer_dlist_t none(vram ? VRAM_SEG : DRAM_SEG);
    const auto end = clk::now() + std::chrono::seconds(600);
    while (tgt.checkRemoteMD("initiator", none) != NIXL_SUCCESS) {
        if (clk::now() > end) return 6;
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
    const std::string where = "ADDR " + std::to_string(reinterpret_cast<uintptr_t>(dst)) + " " + std::to_string(buf_bytes) + " " + std::to_string(vram ? dev : 0);
    if (tgt.genNotif("initiator", where) != NIXL_SUCCESS) return 6;
    std::string rest;
    if (!waitNotif(tgt, "initiator", "DONE", rest, 24 * 3600)) return 7;
    std::printf("target: the initiator is through\n");
    tgt.deregisterMem(rd);
    return 0;
}
} // namespace

int main(int argc, char **argv) {
    Args a;
    for (int i = 1; i < argc; ++i) {
        std::string k = argv[i], v;
        bool has_value = false;
        if (const size_t eq = k.find('='); eq != std::string::npos && k.rfind("--", 0) == 0) { // --name=value
            v = k.substr(eq + 1);
            k.erase(eq);
            has_value = true;
        }
        const Spelling sp = canonical(k);
        if (sp.kind == Spelling::IGNORED) {
            std::fprintf(stderr, "note: %s has no effect in this single-process tool\n", k.c_str());
            if (!has_value && i + 1 < argc && std::strncmp(argv[i + 1], "--", 2) != 0) ++i;
            continue;
        }
        k = sp.name;
        if (has_value && (v == "true" || v == "1") && setFlag(a, k)) continue;
        if (has_value && (v == "false" || v == "0")) {
            Args probe;
            if (setFlag(probe, k)) continue;
        }
        if (!has_value && setFlag(a, k)) continue;
        if (!has_value) {
            if (i + 1 >= argc) {
                std::fprintf(stderr, "option %s needs a value\n", k.c_str());
                return 2;
            }
            v = argv[++i];
        }
        if (k == "--config") {
            if (!loadConfig(a, v)) return 2;
            continue;
        }
        if (sp.kind == Spelling::POSIX_API) {
            const std::string api = v;
            if (api == "AIO" || api == "aio") a.extra["use_aio"] = "true";
            else if (api == "URING" || api == "uring") a.extra["use_uring"] = "true";
            else if (api == "POSIXAIO" || api == "posixaio") a.extra["use_posix_aio"] = "true";
            continue;
        }
        if (sp.kind == Spelling::PARAM) {
            a.extra[sp.param] = v;
            continue;
        }
        if (!setOption(a, k, v)) {
            std::fprintf(stderr, "unknown option %s\n", k.c_str());
            return 2;
        }
    }
    if (!a.etcd.empty() && a.role.empty()) {
        std::fprintf(stderr, "note: --etcd_endpoints has no effect without --role (both ends live in this process)\n");
        a.etcd.clear();
    }
    if (!a.etcd.empty()) ::setenv("NIXL_ETCD_ENDPOINTS", a.etcd.c_str(), 1); // the agents read it when they are created
    const bool vram = a.mem == "VRAM";
    // Object stores (OBJ: S3 or a directory; AZURE_BLOB): every block of a batch is an object of its own, named
    // "<prefix>-<i>" (--obj-prefix, default "nixlbench"); WRITE puts it, READ gets it.
    const bool objects = a.backend == "OBJ" || a.backend == "AZURE_BLOB";
    const bool storage = !a.file.empty() || objects;
    int ndev = 0;
    if (vram && (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)) {
        std::fprintf(stderr, "no GPU\n");
        return 2;
    }
    if (a.scheme != "pairwise") {
        if (a.scheme != "onetomany" && a.scheme != "manytoone" && a.scheme != "tp") {
            std::fprintf(stderr, "unknown --scheme %s (pairwise, onetomany, manytoone, tp)\n", a.scheme.c_str());
            return 2;
        }
        return runScheme(a, ndev);
    }
    if (a.dst_dev < 0) a.dst_dev = ndev > 1 ? 1 : 0;
    if (a.batch_max < a.batch) a.batch_max = a.batch;
    if (storage && a.backend == "NVLINK") a.backend = vram ? "GDS" : "POSIX";
    const size_t buf_bytes = std::min(a.total, std::max<size_t>(a.max * a.batch_max, a.max));
    if (!a.role.empty() && a.role != "initiator" && a.role != "target") {
        std::fprintf(stderr, "unknown --role %s (initiator, target)\n", a.role.c_str());
        return 2;
    }
    const bool remote_target = a.role == "initiator";
    if ((remote_target || a.role == "target") && storage) {
        std::fprintf(stderr, "--role and --file do not go together\n");
        return 2;
    }
    if (a.role == "target") return runTarget(a, vram, buf_bytes);
    if (remote_target && a.peer_port <= 0 && a.etcd.empty()) {
        std::fprintf(stderr, "--role initiator needs --peer-port (and --peer-ip unless the target is on this host), or --etcd-endpoints\n");
        return 2;
    }
    void *src = nullptr, *dst = nullptr;
    auto allocate = [&](void *&p, int dev, int fill) {
        if (vram) {
            cudaSetDevice(dev);
            if (cudaMalloc(&p, buf_bytes) != cudaSuccess) return false;
            cudaMemset(p, fill, buf_bytes);
            cudaDeviceSynchronize();
        } else {
            if (posix_memalign(&p, 4096, buf_bytes) != 0) return false; // page-aligned: usable with O_DIRECT
            std::memset(p, fill, buf_bytes);
        }
        return true;
    };
    if (!allocate(src, a.src_dev, 0x5a)) return 3;
    if (!storage && !remote_target && !allocate(dst, a.dst_dev, 0)) return 3;
    if (vram) cudaSetDevice(a.src_dev);

    // "--enable-pt": the backend's progress thread completes requests; several worker threads need the agent's lock.
    const nixl_thread_sync_t sync = a.num_threads > 1 ? nixl_thread_sync_t::NIXL_THREAD_SYNC_RW : nixl_thread_sync_t::NIXL_THREAD_SYNC_NONE;
    nixlAgentConfig cfg(a.enable_pt, false, 0, sync);
    // with a target in another process the initiator's metadata travels through the agents' listeners
    const bool by_listener = remote_target && a.etcd.empty();
    nixlAgentConfig ini_cfg(a.enable_pt, by_listener, static_cast<uint16_t>(by_listener ? (a.listen_port > 0 ? a.listen_port : freePort()) : 0), sync);
    nixlAgent ini("initiator", ini_cfg), tgt(remote_target ? "unused" : "target", cfg);
    nixlBackendH *bi = nullptr, *bt = nullptr;
    nixl_b_params_t params;
    if (a.backend == "NVLINK" || a.backend == "UCX") params["copy_path"] = a.copy_path;
    for (auto &kv : a.extra) params[kv.first] = kv.second;
    if (ini.createBackend(a.backend, params, bi) != NIXL_SUCCESS || (!storage && !remote_target && tgt.createBackend(a.backend, params, bt) != NIXL_SUCCESS)) {
        std::fprintf(stderr, "cannot create backend %s\n", a.backend.c_str());
        return 4;
    }
    const nixl_mem_t mt = vram ? VRAM_SEG : DRAM_SEG;
    const nixl_mem_t rmt = objects ? OBJ_SEG : storage ? FILE_SEG : mt;
    const std::string remote_name = storage ? "initiator" : "target";
    nixl_reg_dlist_t rs(mt), rd(rmt);
    rs.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src), buf_bytes, vram ? a.src_dev : 0, ""));
    std::vector<int> fds;
    const size_t file_bytes = (buf_bytes + a.num_files - 1) / a.num_files;
    if (objects) {
        if (vram) {
            std::fprintf(stderr, "object stores take host memory: --mem DRAM\n");
            return 2;
        }
        // One registration per object, long enough for the largest block; devId is the object's number.
        for (int i = 0; i < a.batch_max; ++i) rd.addDesc(nixlBlobDesc(0, a.max, static_cast<uint64_t>(i), a.obj_prefix + "-" + std::to_string(i)));
        if (ini.registerMem(rs) != NIXL_SUCCESS || ini.registerMem(rd) != NIXL_SUCCESS) return 5;
    } else if (storage) {
        // The buffer is striped over num_files files of file_bytes each; devId of a FILE descriptor is its fd.
        for (int f = 0; f < a.num_files; ++f) {
            const std::string path = a.num_files == 1 ? a.file : a.file + "." + std::to_string(f);
            const int fd = ::open(path.c_str(), O_RDWR | O_CREAT | (a.direct ? O_DIRECT : 0), 0644);
            if (fd < 0 || ::ftruncate(fd, static_cast<off_t>(file_bytes)) != 0) {
                std::fprintf(stderr, "cannot prepare %s\n", path.c_str());
                return 5;
            }
            fds.push_back(fd);
            rd.addDesc(nixlBlobDesc(0, file_bytes, static_cast<uint64_t>(fd), ""));
        }
        if (ini.registerMem(rs) != NIXL_SUCCESS || ini.registerMem(rd) != NIXL_SUCCESS) return 5;
    } else if (remote_target) {
        if (ini.registerMem(rs) != NIXL_SUCCESS) return 5;
        nixl_opt_args_t where;
        where.ipAddr = a.peer_ip;
        where.port = a.peer_port;
        const nixl_opt_args_t *how = a.etcd.empty() ? &where : nullptr; // no address: through the central store
        if (ini.fetchRemoteMD("target", how) != NIXL_SUCCESS || ini.sendLocalMD(how) != NIXL_SUCCESS) return 6;
        const nixl_xfer_dlist_t none(mt);
        const auto end = clk::now() + std::chrono::seconds(60);
        while (ini.checkRemoteMD("target", none) != NIXL_SUCCESS) {
            if (clk::now() > end) {
                std::fprintf(stderr, "no metadata from the target (%s)\n", a.etcd.empty() ? (a.peer_ip + ":" + std::to_string(a.peer_port)).c_str() : a.etcd.c_str());
                return 6;
            }
            std::this_thread::sleep_for(std::chrono::milliseconds(2));
        }
        std::string rest;
        if (!waitNotif(ini, "target", "ADDR ", rest, 60)) return 6;
        unsigned long long addr = 0, len = 0;
        int their_dev = 0;
        if (std::sscanf(rest.c_str(), "%llu %llu %d", &addr, &len, &their_dev) != 3 || len < buf_bytes) {
            std::fprintf(stderr, "the target's buffer (%llu bytes) is smaller than this sweep needs (%zu): start both with the same sizes\n", len, buf_bytes);
            ini.genNotif("target", "DONE");
            return 6;
        }
        dst = reinterpret_cast<void *>(static_cast<uintptr_t>(addr)); // an address of the other process: never touched here
        a.dst_dev = their_dev;
    } else {
        rd.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst), buf_bytes, vram ? a.dst_dev : 0, ""));
        if (ini.registerMem(rs) != NIXL_SUCCESS || tgt.registerMem(rd) != NIXL_SUCCESS) return 5;
        nixl_blob_t md;
        std::string name;
        tgt.getLocalMD(md);
        if (ini.loadRemoteMD(md, name) != NIXL_SUCCESS) return 6;
    }
    const nixl_xfer_op_t op = a.op == "READ" ? NIXL_READ : NIXL_WRITE;

    std::printf("%-12s %6s %10s %10s %10s %10s %10s %10s\n", "block", "batch", "GB/s", "avg_us", "p50_us", "p99_us", "prep_us", "post_us");
    for (int batch = a.batch; batch <= a.batch_max; batch *= 2)
    for (size_t block = a.min; block <= a.max && block * batch <= buf_bytes; block *= 2) {
        int iters = a.iters, warm = a.warmup;
        const size_t per = block * batch;
        if (objects && op == NIXL_READ) { // what is to be read has to be there: put the batch once, untimed
            nixl_xfer_dlist_t l(mt), r(rmt);
            for (int i = 0; i < batch; ++i) {
                l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src) + static_cast<size_t>(i) * block, block, 0));
                r.addDesc(nixlBasicDesc(0, block, static_cast<uint64_t>(i)));
            }
            nixlXferReqH *put = nullptr;
            if (ini.createXferReq(NIXL_WRITE, l, r, remote_name, put) != NIXL_SUCCESS) return 7;
            nixl_status_t st = ini.postXferReq(put);
            while (st == NIXL_IN_PROG) st = ini.getXferStatus(put);
            ini.releaseXferReq(put);
            if (st != NIXL_SUCCESS) {
                std::fprintf(stderr, "cannot put the objects to read (status %d)\n", static_cast<int>(st));
                return 7;
            }
        }
        if (per > (size_t(64) << 20)) {
            iters = std::max<int>(10, static_cast<int>((size_t(64) << 30) / per / 16));
            warm = 3;
        }
        if (storage) {
            iters = std::min(iters, 200);
            warm = std::min(warm, 5);
        }
        // Worker threads ("--num-threads"): thread t owns the descriptors t, t + T, ... of the batch and runs the whole
        // pipelined loop on them with requests of its own; the rate counts all threads' bytes over the slowest thread's time.
        const int nthreads = std::max(1, std::min(a.num_threads, batch));
        if (a.reregister && nthreads > 1) {
            std::fprintf(stderr, "--reregister works with one thread\n");
            return 2;
        }
        struct WorkerStats {
            std::vector<double> prep, post, xfer;
            double wall = 0;
            int rc = 0;
        };
        std::vector<WorkerStats> stats(nthreads);
        std::barrier start_line(nthreads);
        auto worker = [&](int tid) -> int {
        // A worker that gives up before the common start leaves the start line, so that the others do not wait for it.
        auto early = [&](int rc) {
            start_line.arrive_and_drop();
            return rc;
        };
        std::vector<double> &prep = stats[tid].prep, &post = stats[tid].post, &xfer = stats[tid].xfer;
        std::vector<nixlXferReqH *> slots(a.depth, nullptr);
        nixl_xfer_dlist_t l(mt), r(rmt);
        int mine = 0;
        for (int i = tid; i < batch; i += nthreads, ++mine) {
            const size_t off = static_cast<size_t>(i) * block;
            l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src) + off, block, vram ? a.src_dev : 0));
            if (objects) {
                r.addDesc(nixlBasicDesc(0, block, static_cast<uint64_t>(i)));
            } else if (storage) {
                const size_t f = std::min<size_t>(off / file_bytes, fds.size() - 1);
                size_t foff = off - f * file_bytes;
                if (foff + block > file_bytes) foff = 0; // a block never straddles two files
                r.addDesc(nixlBasicDesc(foff, block, static_cast<uint64_t>(fds[f])));
            } else {
                const size_t roff = a.scatter ? static_cast<size_t>(batch - 1 - i) * block : off;
                r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst) + roff, block, vram ? a.dst_dev : 0));
            }
        }
        if (vram) cudaSetDevice(a.src_dev);
        nixlDlistH *side_l = nullptr, *side_r = nullptr;
        std::vector<int> all_idx(mine);
        for (int i = 0; i < mine; ++i) all_idx[i] = i;
        if (a.prepared) {
            const auto t0 = clk::now();
            if (ini.prepXferDlist(NIXL_INIT_AGENT, l, side_l) != NIXL_SUCCESS || ini.prepXferDlist(remote_name, r, side_r) != NIXL_SUCCESS) return early(7);
            prep.push_back(us(t0, clk::now()));
        }
        auto create = [&](nixlXferReqH *&h) {
            const auto t0 = clk::now();
            const nixl_status_t st = a.prepared ? ini.makeXferReq(op, side_l, all_idx, side_r, all_idx, h) : ini.createXferReq(op, l, r, remote_name, h);
            prep.push_back(us(t0, clk::now()));
            return st == NIXL_SUCCESS;
        };
        for (auto &s : slots)
            if (!create(s)) return early(7);
        std::vector<clk::time_point> started(a.depth);
        std::vector<bool> busy(a.depth, false);
        start_line.arrive_and_wait();
        clk::time_point t_begin = clk::now();
        int posted = 0, done = 0;
        const int total = warm + iters;
        int failed = 0;
        auto finished = [&](int s, clk::time_point now) {
            busy[s] = false;
            if (done >= warm) xfer.push_back(us(started[s], now));
            ++done;
            if (done == warm) t_begin = clk::now();
            if (a.recreate && posted < total) {
                ini.releaseXferReq(slots[s]);
                slots[s] = nullptr;
                if (!create(slots[s])) failed = 7;
            }
        };
        while (done < total && !failed) {
            for (int s = 0; s < a.depth && !failed; ++s) {
                if (busy[s]) {
                    const nixl_status_t st = ini.getXferStatus(slots[s]);
                    if (st == NIXL_SUCCESS) finished(s, clk::now());
                    else if (st < 0) {
                        std::fprintf(stderr, "transfer failed: %d\n", st);
                        failed = 8;
                    }
                }
                if (!busy[s] && posted < total && !failed) {
                    if (a.reregister && a.depth == 1) {
                        // Every iteration pays for taking the buffer out of the backend and putting it back.
                        ini.releaseXferReq(slots[s]);
                        slots[s] = nullptr;
                        if (ini.deregisterMem(rs) != NIXL_SUCCESS || ini.registerMem(rs) != NIXL_SUCCESS) return 5;
                        if (a.prepared) {
                            ini.releasedDlistH(side_l);
                            if (ini.prepXferDlist(NIXL_INIT_AGENT, l, side_l) != NIXL_SUCCESS) return 7;
                        }
                        if (!create(slots[s])) return 7;
                    }
                    started[s] = clk::now();
                    const nixl_status_t st = ini.postXferReq(slots[s]);
                    const auto t1 = clk::now();
                    if (st < 0) {
                        failed = 9;
                        break;
                    }
                    if (posted >= warm) post.push_back(us(started[s], t1));
                    ++posted;
                    if (st == NIXL_SUCCESS) finished(s, t1);
                    else busy[s] = true;
                }
            }
        }
        stats[tid].wall = us(t_begin, clk::now());
        for (auto s : slots)
            if (s) ini.releaseXferReq(s);
        if (side_l) ini.releasedDlistH(side_l);
        if (side_r) ini.releasedDlistH(side_r);
        return failed;
        };
        {
            std::vector<std::thread> pool;
            for (int t = 1; t < nthreads; ++t) pool.emplace_back([&, t] { stats[t].rc = worker(t); });
            stats[0].rc = worker(0);
            for (auto &t : pool) t.join();
        }
        std::vector<double> prep, post, xfer;
        double wall = 0;
        for (auto &w : stats) {
            if (w.rc) return w.rc;
            prep.insert(prep.end(), w.prep.begin(), w.prep.end());
            post.insert(post.end(), w.post.begin(), w.post.end());
            xfer.insert(xfer.end(), w.xfer.begin(), w.xfer.end());
            wall = std::max(wall, w.wall);
        }
        double sum = 0;
        for (double v : xfer) sum += v;
        double psum = 0;
        for (double v : post) psum += v;
        double prsum = 0;
        for (double v : prep) prsum += v;
        std::printf("%-12zu %6d %10.2f %10.2f %10.2f %10.2f %10.2f %10.2f\n", block, batch, double(per) * iters / wall / 1e3,
                    sum / std::max<size_t>(1, xfer.size()), pct(xfer, 0.5), pct(xfer, 0.99), prsum / std::max<size_t>(1, prep.size()),
                    psum / std::max<size_t>(1, post.size()));
        std::fflush(stdout);
        if (a.check) {
            // WRITE: the destination (memory or file) must hold the source pattern; READ from memory: the source side
            // was overwritten with the target's zeros.
            std::vector<unsigned char> h(std::min<size_t>(block, 1 << 20));
            unsigned char want = 0x5a;
            if (objects) {
                // Get the start of object 0 back into the start of the source: the pattern if the store holds what was put.
                nixl_xfer_dlist_t l(mt), r(rmt);
                l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src), h.size(), 0));
                r.addDesc(nixlBasicDesc(0, h.size(), 0));
                nixlXferReqH *back = nullptr;
                if (ini.createXferReq(NIXL_READ, l, r, remote_name, back) != NIXL_SUCCESS) return 10;
                nixl_status_t st = ini.postXferReq(back);
                while (st == NIXL_IN_PROG) st = ini.getXferStatus(back);
                ini.releaseXferReq(back);
                if (st != NIXL_SUCCESS) return 10;
                std::memcpy(h.data(), src, h.size());
            } else if (storage) {
                if (op != NIXL_WRITE) continue; // a READ returns what an earlier WRITE stored: nothing fixed to compare with
                if (::pread(fds[0], h.data(), h.size(), 0) != static_cast<ssize_t>(h.size())) return 10;
            } else if (remote_target && op == NIXL_WRITE) {
                // Read the start of what was written back into the start of the source: it holds the same pattern if
                // the WRITE arrived, the target's zeros if it did not.
                nixl_xfer_dlist_t l(mt), r(mt);
                l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src), h.size(), vram ? a.src_dev : 0));
                r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst), h.size(), vram ? a.dst_dev : 0));
                nixlXferReqH *back = nullptr;
                if (ini.createXferReq(NIXL_READ, l, r, remote_name, back) != NIXL_SUCCESS) return 10;
                nixl_status_t st = ini.postXferReq(back);
                while (st == NIXL_IN_PROG) st = ini.getXferStatus(back);
                ini.releaseXferReq(back);
                if (st != NIXL_SUCCESS) return 10;
                if (vram) cudaMemcpy(h.data(), src, h.size(), cudaMemcpyDeviceToHost);
                else std::memcpy(h.data(), src, h.size());
            } else if (remote_target) {
                if (vram) cudaMemcpy(h.data(), src, h.size(), cudaMemcpyDeviceToHost);
                else std::memcpy(h.data(), src, h.size());
                want = 0x00;
            } else if (vram) {
                cudaSetDevice(op == NIXL_WRITE ? a.dst_dev : a.src_dev);
                cudaMemcpy(h.data(), op == NIXL_WRITE ? dst : src, h.size(), cudaMemcpyDeviceToHost);
                cudaSetDevice(a.src_dev);
                want = op == NIXL_WRITE ? 0x5a : 0x00;
            } else {
                std::memcpy(h.data(), op == NIXL_WRITE ? dst : src, h.size());
                want = op == NIXL_WRITE ? 0x5a : 0x00;
            }
            for (unsigned char c : h)
                if (c != want) {
                    std::fprintf(stderr, "consistency check failed at block %zu\n", block);
                    return 10;
                }
        }
    }
    for (int fd : fds) ::close(fd);
    if (remote_target) ini.genNotif("target", "DONE");
    return 0;
}

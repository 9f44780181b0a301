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
//             [--min 4096] [--max 1073741824] [--batch 1] [--iters 1000] [--warmup 100]
//             [--depth 1] [--copy-path vector|bulk] [--param key=value]... [--check]
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "nixl.h"

namespace {
using clk = std::chrono::steady_clock;
double us(clk::time_point a, clk::time_point b) { return std::chrono::duration<double, std::micro>(b - a).count(); }

struct Args {
    std::string backend = "NVLINK", op = "WRITE", mem = "VRAM", copy_path = "vector";
    int src_dev = 0, dst_dev = -1, batch = 1, iters = 1000, warmup = 100, depth = 1;
    size_t min = 4096, max = size_t(1) << 30, total = size_t(8) << 30;
    bool check = false;
    nixl_b_params_t extra; // --param key=value, passed to the backend
};

double pct(std::vector<double> &v, double q) {
    if (v.empty()) return 0;
    std::sort(v.begin(), v.end());
    return v[std::min(v.size() - 1, static_cast<size_t>(q * v.size()))];
}
} // namespace

int main(int argc, char **argv) {
    Args a;
    for (int i = 1; i < argc; ++i) {
        const std::string k = argv[i];
        auto val = [&]() -> const char * { return i + 1 < argc ? argv[++i] : ""; };
        if (k == "--backend") a.backend = val();
        else if (k == "--op") a.op = val();
        else if (k == "--mem") a.mem = val();
        else if (k == "--copy-path") a.copy_path = val();
        else if (k == "--src-dev") a.src_dev = std::atoi(val());
        else if (k == "--dst-dev") a.dst_dev = std::atoi(val());
        else if (k == "--batch") a.batch = std::atoi(val());
        else if (k == "--iters") a.iters = std::atoi(val());
        else if (k == "--warmup") a.warmup = std::atoi(val());
        else if (k == "--depth") a.depth = std::max(1, std::atoi(val()));
        else if (k == "--min") a.min = std::strtoull(val(), nullptr, 0);
        else if (k == "--max") a.max = std::strtoull(val(), nullptr, 0);
        else if (k == "--total") a.total = std::strtoull(val(), nullptr, 0);
        else if (k == "--check") a.check = true;
        else if (k == "--param") {
            const std::string kv = val();
            const size_t eq = kv.find('=');
            if (eq != std::string::npos) a.extra[kv.substr(0, eq)] = kv.substr(eq + 1);
        }
        else {
            std::fprintf(stderr, "unknown option %s\n", k.c_str());
            return 2;
        }
    }
    const bool vram = a.mem == "VRAM";
    int ndev = 0;
    if (vram && (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)) {
        std::fprintf(stderr, "no GPU\n");
        return 2;
    }
    if (a.dst_dev < 0) a.dst_dev = ndev > 1 ? 1 : 0;
    const size_t buf_bytes = std::min(a.total, std::max<size_t>(a.max * a.batch, a.max));
    void *src = nullptr, *dst = nullptr;
    if (vram) {
        cudaSetDevice(a.src_dev);
        if (cudaMalloc(&src, buf_bytes) != cudaSuccess) return 3;
        cudaMemset(src, 0x5a, buf_bytes);
        cudaSetDevice(a.dst_dev);
        if (cudaMalloc(&dst, buf_bytes) != cudaSuccess) return 3;
        cudaMemset(dst, 0, buf_bytes);
        cudaSetDevice(a.src_dev);
        cudaDeviceSynchronize();
    } else {
        src = std::malloc(buf_bytes);
        dst = std::malloc(buf_bytes);
        std::memset(src, 0x5a, buf_bytes);
        std::memset(dst, 0, buf_bytes);
    }
    nixlAgentConfig cfg(false);
    nixlAgent ini("initiator", cfg), tgt("target", cfg);
    nixlBackendH *bi = nullptr, *bt = nullptr;
    nixl_b_params_t params = {{"copy_path", a.copy_path}};
    for (auto &kv : a.extra) params[kv.first] = kv.second;
    if (ini.createBackend(a.backend, params, bi) != NIXL_SUCCESS || tgt.createBackend(a.backend, params, bt) != NIXL_SUCCESS) {
        std::fprintf(stderr, "cannot create backend %s\n", a.backend.c_str());
        return 4;
    }
    const nixl_mem_t mt = vram ? VRAM_SEG : DRAM_SEG;
    nixl_reg_dlist_t rs(mt), rd(mt);
    rs.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(src), buf_bytes, vram ? a.src_dev : 0, ""));
    rd.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(dst), buf_bytes, vram ? a.dst_dev : 0, ""));
    if (ini.registerMem(rs) != NIXL_SUCCESS || tgt.registerMem(rd) != NIXL_SUCCESS) return 5;
    nixl_blob_t md;
    std::string name;
    tgt.getLocalMD(md);
    if (ini.loadRemoteMD(md, name) != NIXL_SUCCESS) return 6;
    const nixl_xfer_op_t op = a.op == "READ" ? NIXL_READ : NIXL_WRITE;

    std::printf("%-12s %6s %10s %10s %10s %10s %10s %10s\n", "block", "batch", "GB/s", "avg_us", "p50_us", "p99_us", "prep_us", "post_us");
    for (size_t block = a.min; block <= a.max && block * a.batch <= buf_bytes; block *= 2) {
        int iters = a.iters, warm = a.warmup;
        const size_t per = block * a.batch;
        if (per > (size_t(64) << 20)) {
            iters = std::max<int>(10, static_cast<int>((size_t(64) << 30) / per / 16));
            warm = 3;
        }
        std::vector<double> prep, post, xfer;
        std::vector<nixlXferReqH *> slots(a.depth, nullptr);
        nixl_xfer_dlist_t l(mt), r(mt);
        for (int i = 0; i < a.batch; ++i) {
            l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(src) + i * block, block, vram ? a.src_dev : 0));
            r.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(dst) + i * block, block, vram ? a.dst_dev : 0));
        }
        for (auto &s : slots) {
            const auto t0 = clk::now();
            if (ini.createXferReq(op, l, r, "target", s) != NIXL_SUCCESS) return 7;
            prep.push_back(us(t0, clk::now()));
        }
        std::vector<clk::time_point> started(a.depth);
        std::vector<bool> busy(a.depth, false);
        clk::time_point t_begin;
        int posted = 0, done = 0;
        const int total = warm + iters;
        while (done < total) {
            for (int s = 0; s < a.depth; ++s) {
                if (busy[s]) {
                    const nixl_status_t st = ini.getXferStatus(slots[s]);
                    if (st == NIXL_SUCCESS) {
                        busy[s] = false;
                        if (done >= warm) xfer.push_back(us(started[s], clk::now()));
                        ++done;
                        if (done == warm) t_begin = clk::now();
                    } else if (st < 0) {
                        std::fprintf(stderr, "transfer failed: %d\n", st);
                        return 8;
                    }
                }
                if (!busy[s] && posted < total) {
                    if (posted == warm && warm == 0) t_begin = clk::now();
                    started[s] = clk::now();
                    const nixl_status_t st = ini.postXferReq(slots[s]);
                    const auto t1 = clk::now();
                    if (st < 0) return 9;
                    if (posted >= warm) post.push_back(us(started[s], t1));
                    ++posted;
                    if (st == NIXL_SUCCESS) {
                        if (done >= warm) xfer.push_back(us(started[s], t1));
                        ++done;
                        if (done == warm) t_begin = clk::now();
                    } else busy[s] = true;
                }
            }
        }
        const double wall = us(t_begin, clk::now());
        double sum = 0;
        for (double v : xfer) sum += v;
        double psum = 0;
        for (double v : post) psum += v;
        double prsum = 0;
        for (double v : prep) prsum += v;
        std::printf("%-12zu %6d %10.2f %10.2f %10.2f %10.2f %10.2f %10.2f\n", block, a.batch, double(per) * iters / wall / 1e3,
                    sum / std::max<size_t>(1, xfer.size()), pct(xfer, 0.5), pct(xfer, 0.99), prsum / prep.size(), psum / std::max<size_t>(1, post.size()));
        std::fflush(stdout);
        for (auto s : slots) ini.releaseXferReq(s);
        if (a.check) {
            std::vector<unsigned char> h(std::min<size_t>(per, 1 << 20));
            if (vram) {
                cudaSetDevice(op == NIXL_WRITE ? a.dst_dev : a.src_dev);
                cudaMemcpy(h.data(), op == NIXL_WRITE ? dst : src, h.size(), cudaMemcpyDeviceToHost);
                cudaSetDevice(a.src_dev);
            } else std::memcpy(h.data(), op == NIXL_WRITE ? dst : src, h.size());
            const unsigned char want = op == NIXL_WRITE ? 0x5a : 0x00;
            for (unsigned char c : h)
                if (c != want) {
                    std::fprintf(stderr, "consistency check failed at block %zu\n", block);
                    return 10;
                }
        }
    }
    return 0;
}

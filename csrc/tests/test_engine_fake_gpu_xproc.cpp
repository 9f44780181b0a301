// The NVLINK backend between two PROCESSES on the stand-in CUDA runtime (tests/fake_cuda): the target's "device memory"
// is a shared-memory object, its IPC handle opens in the initiator's process as a mapping at another address, exactly
// the shape of CUDA IPC.  Covered: the published registration (IPC handle, offset, GPU UUID), the opened-handle cache
// and its release, the choice between copy kernel, copy engines and doorbell proxy for another process's memory, the
// notification ring across processes (the target learns of a WRITE that the initiator never polls), READ, and a
// target that exits.  The whole run is done twice: with cudaMalloc memory (shared by IPC handle) and with memory from
// the virtual-memory calls (five allocations behind one address range, shared as file descriptors over the target's
// descriptor server and mapped again in the initiator).  Every process forks before anything in it starts a thread.
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <random>
#include <thread>

#include "core/plugin_manager.h"
#include "cuda_runtime.h"
#include "nixl.h"

namespace {

using clk = std::chrono::steady_clock;
constexpr size_t kBytes = 8 << 20;

struct Shared {
    std::atomic<int> stage;
    size_t tgtMdLen, iniMdLen;
    char tgtMd[1 << 16], iniMd[1 << 16];
    uintptr_t tgtAddr;
    uint64_t sumAfterWrite, sumAfterCe;
    int notifsSeenBeforePoll;
    int targetFailed;
};

bool waitStage(Shared *sh, int s, int seconds = 30) {
    const auto end = clk::now() + std::chrono::seconds(seconds);
    while (sh->stage.load() < s && clk::now() < end) std::this_thread::sleep_for(std::chrono::microseconds(200));
    return sh->stage.load() >= s;
}

uint64_t sumOf(const uint8_t *p, size_t n) {
    uint64_t s = 0;
    for (size_t i = 0; i < n; ++i) s += p[i] * (1 + (i & 7));
    return s;
}

int failures = 0;
#define EXPECT(cond)                                                              \
    do {                                                                          \
        if (!(cond)) {                                                            \
            std::printf("[FAIL] %s:%d: %s\n", __FILE__, __LINE__, #cond);         \
            ++failures;                                                           \
        }                                                                         \
    } while (0)

// ------------------------------------------------------------------ target (child process)
int target(Shared *sh, bool vmm) {
    nixlPluginManager::getInstance().addPluginDirectory(FAKE_GPU_PLUGIN_DIR);
    nixlAgent agent("xp_target", nixlAgentConfig(false));
    nixlBackendH *h = nullptr;
    if (agent.createBackend("NVLINK", {}, h) != NIXL_SUCCESS) return 10;
    cudaSetDevice(1);
    uint8_t *buf = nullptr, *vm = nullptr;
    if (vmm) {
        // 8 MiB that start in the middle of the first of five 2 MiB allocations and end in the middle of the last
        vm = static_cast<uint8_t *>(fake_cuda::mallocVmm(2 << 20, 5, 1));
        if (!vm) return 11;
        buf = vm + (1 << 20) + 4096;
    } else if (cudaMalloc(reinterpret_cast<void **>(&buf), kBytes) != cudaSuccess) {
        return 11;
    }
    std::memset(buf, 0, kBytes);
    nixl_reg_dlist_t reg(VRAM_SEG);
    reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf), kBytes, 1, ""));
    if (agent.registerMem(reg) != NIXL_SUCCESS) return 12;
    nixl_blob_t md;
    agent.getLocalMD(md);
    if (md.size() > sizeof(sh->tgtMd)) return 13;
    std::memcpy(sh->tgtMd, md.data(), md.size());
    sh->tgtMdLen = md.size();
    sh->tgtAddr = reinterpret_cast<uintptr_t>(buf);
    sh->stage.store(1);
    if (!waitStage(sh, 2)) return 14;
    std::string name;
    if (agent.loadRemoteMD(nixl_blob_t(sh->iniMd, sh->iniMdLen), name) != NIXL_SUCCESS) return 15;
    sh->stage.store(3);

    // the initiator posts a WRITE with a notification and does NOT poll it: the ring must deliver
    int got = 0;
    auto end = clk::now() + std::chrono::seconds(20);
    while (got < 1 && clk::now() < end) {
        nixl_notifs_t n;
        agent.getNotifs(n);
        got += static_cast<int>(n["xp_initiator"].size());
    }
    sh->notifsSeenBeforePoll = got;
    sh->sumAfterWrite = sumOf(buf, kBytes);
    sh->stage.store(4);

    if (!waitStage(sh, 5)) return 16; // the copy-engine request and the proxy requests have completed
    sh->sumAfterCe = sumOf(buf, kBytes);
    for (size_t i = 0; i < kBytes; i += 4097) buf[i] = static_cast<uint8_t>(buf[i] + 1); // what the initiator reads back
    sh->stage.store(6);
    if (!waitStage(sh, 7)) return 17;
    agent.deregisterMem(reg);
    if (vmm) fake_cuda::freeVmm(vm);
    else cudaFree(buf);
    return 0; // the agent goes away with the process: the initiator must notice
}

// ------------------------------------------------------------------ initiator (parent process)
nixl_status_t waitDone(nixlAgent &a, nixlXferReqH *req) {
    nixl_status_t st;
    const auto end = clk::now() + std::chrono::seconds(20);
    while ((st = a.getXferStatus(req)) == NIXL_IN_PROG && clk::now() < end) {}
    return st;
}

void initiator(Shared *sh, pid_t child) {
    nixlPluginManager::getInstance().addPluginDirectory(FAKE_GPU_PLUGIN_DIR);
    nixlAgent agent("xp_initiator", nixlAgentConfig(false));
    nixlBackendH *h = nullptr;
    EXPECT(agent.createBackend("NVLINK", {{"ce_threshold", "1048576"}}, h) == NIXL_SUCCESS);
    cudaSetDevice(0);
    uint8_t *buf = nullptr;
    EXPECT(cudaMalloc(reinterpret_cast<void **>(&buf), kBytes) == cudaSuccess);
    std::mt19937 rng(17);
    for (size_t i = 0; i < kBytes; ++i) buf[i] = static_cast<uint8_t>(rng());
    nixl_reg_dlist_t reg(VRAM_SEG);
    reg.addDesc(nixlBlobDesc(reinterpret_cast<uintptr_t>(buf), kBytes, 0, ""));
    EXPECT(agent.registerMem(reg) == NIXL_SUCCESS);
    EXPECT(waitStage(sh, 1));
    std::string name;
    EXPECT(agent.loadRemoteMD(nixl_blob_t(sh->tgtMd, sh->tgtMdLen), name) == NIXL_SUCCESS);
    EXPECT(name == "xp_target");
    nixl_blob_t md;
    agent.getLocalMD(md);
    EXPECT(md.size() <= sizeof(sh->iniMd));
    std::memcpy(sh->iniMd, md.data(), md.size());
    sh->iniMdLen = md.size();
    sh->stage.store(2);
    EXPECT(waitStage(sh, 3));
    const uintptr_t there = sh->tgtAddr; // an address of the OTHER process: the backend translates it through the opened handle

    // 1. forty scattered pieces through the copy kernel, notification released by the kernel's tail
    std::vector<uint8_t> expect(kBytes, 0);
    nixl_xfer_dlist_t l(VRAM_SEG), r(VRAM_SEG);
    for (int i = 0; i < 40; ++i) {
        const size_t off = size_t(i) * 70000 + 16, roff = size_t(39 - i) * 70000 + 48, len = 30000 + 77 * i;
        l.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf) + off, len, 0));
        r.addDesc(nixlBasicDesc(there + roff, len, 1));
        std::memcpy(expect.data() + roff, buf + off, len);
    }
    nixl_opt_args_t args;
    args.notif = "wrote";
    nixlXferReqH *req = nullptr;
    EXPECT(agent.createXferReq(NIXL_WRITE, l, r, "xp_target", req, &args) == NIXL_SUCCESS);
    EXPECT(agent.postXferReq(req) >= 0);
    EXPECT(waitStage(sh, 4)); // the target has seen the notification; this side has not looked at its request since the post
    EXPECT(sh->notifsSeenBeforePoll == 1);
    EXPECT(sh->sumAfterWrite == sumOf(expect.data(), kBytes));
    EXPECT(waitDone(agent, req) == NIXL_SUCCESS);
    EXPECT(agent.releaseXferReq(req) == NIXL_SUCCESS);

    // 2. a run of 2 MiB (sixteen blocks that continue each other): copy engines; then 300 small requests: doorbell proxy
    nixl_xfer_dlist_t l2(VRAM_SEG), r2(VRAM_SEG);
    for (int i = 0; i < 16; ++i) {
        l2.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf) + (4 << 20) + size_t(i) * 131072, 131072, 0));
        r2.addDesc(nixlBasicDesc(there + (4 << 20) + size_t(i) * 131072, 131072, 1));
    }
    std::memcpy(expect.data() + (4 << 20), buf + (4 << 20), 2 << 20);
    EXPECT(agent.createXferReq(NIXL_WRITE, l2, r2, "xp_target", req) == NIXL_SUCCESS);
    EXPECT(agent.postXferReq(req) >= 0);
    EXPECT(waitDone(agent, req) == NIXL_SUCCESS);
    EXPECT(agent.releaseXferReq(req) == NIXL_SUCCESS);
    nixl_xfer_dlist_t l3(VRAM_SEG), r3(VRAM_SEG);
    l3.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf) + (7 << 20), 8192, 0));
    r3.addDesc(nixlBasicDesc(there + (7 << 20), 8192, 1));
    EXPECT(agent.createXferReq(NIXL_WRITE, l3, r3, "xp_target", req) == NIXL_SUCCESS);
    for (int i = 0; i < 300; ++i) {
        buf[(7 << 20) + (i % 8192)] = static_cast<uint8_t>(i);
        EXPECT(agent.postXferReq(req) >= 0);
        EXPECT(waitDone(agent, req) == NIXL_SUCCESS);
    }
    std::memcpy(expect.data() + (7 << 20), buf + (7 << 20), 8192);
    EXPECT(agent.releaseXferReq(req) == NIXL_SUCCESS);
    sh->stage.store(5);
    EXPECT(waitStage(sh, 6));
    EXPECT(sh->sumAfterCe == sumOf(expect.data(), kBytes));

    // 3. READ what the target changed
    for (size_t i = 0; i < kBytes; i += 4097) expect[i] = static_cast<uint8_t>(expect[i] + 1);
    nixl_xfer_dlist_t l4(VRAM_SEG), r4(VRAM_SEG);
    l4.addDesc(nixlBasicDesc(reinterpret_cast<uintptr_t>(buf), kBytes, 0));
    r4.addDesc(nixlBasicDesc(there, kBytes, 1));
    EXPECT(agent.createXferReq(NIXL_READ, l4, r4, "xp_target", req) == NIXL_SUCCESS);
    EXPECT(agent.postXferReq(req) >= 0);
    EXPECT(waitDone(agent, req) == NIXL_SUCCESS);
    EXPECT(std::memcmp(buf, expect.data(), kBytes) == 0);

    // 4. the target process exits: the next post reports it and the metadata is dropped
    sh->stage.store(7);
    int status = 0;
    EXPECT(::waitpid(child, &status, 0) == child);
    EXPECT(WIFEXITED(status) && WEXITSTATUS(status) == 0);
    EXPECT(agent.postXferReq(req) == NIXL_ERR_REMOTE_DISCONNECT);
    EXPECT(agent.checkRemoteMD("xp_target", nixl_xfer_dlist_t(VRAM_SEG)) == NIXL_ERR_NOT_FOUND);
    agent.releaseXferReq(req);
    agent.deregisterMem(reg);
    cudaFree(buf);
}

} // namespace

int scenario(bool vmm) {
    auto *sh = static_cast<Shared *>(::mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0));
    if (sh == MAP_FAILED) return 99;
    new (&sh->stage) std::atomic<int>(0);
    const pid_t child = ::fork(); // before the stand-in runtime or an agent has started any thread
    if (child == 0) ::_exit(target(sh, vmm));
    initiator(sh, child);
    return failures;
}

int main() {
    // One process per run, so that each run's pair forks from a process that has never started a thread.
    const char *names[2] = {"between_processes_over_ipc_handles", "between_processes_over_exported_allocations"};
    int failed = 0;
    for (int vmm = 0; vmm < 2; ++vmm) {
        std::fflush(stdout);
        const pid_t run = ::fork();
        if (run == 0) {
            const int f = scenario(vmm != 0);
            std::fflush(stdout);
            ::_exit(f ? 1 : 0);
        }
        int status = 0;
        const bool ok = ::waitpid(run, &status, 0) == run && WIFEXITED(status) && WEXITSTATUS(status) == 0;
        std::printf("%s %s\n", ok ? "[ OK ]" : "[FAIL]", names[vmm]);
        failed += !ok;
    }
    std::printf("2 cases, %d failed\n", failed);
    return failed ? 1 : 0;
}

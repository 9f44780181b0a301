// Sharing of device memory that CUDA IPC cannot export: memory created with the virtual memory
// management API (cuMemCreate + cuMemMap), which is what PyTorch's expandable-segments allocator
// and most serving engines' own pools hand out.
//
// Role of the reference's examples/device/ep/csrc/vmm.cpp:101-173 (exportable allocations for
// its EP buffers), generalised to memory the caller already owns: a registered range is walked
// allocation by allocation, each physical allocation is exported as a POSIX file descriptor
// (cuMemExportToShareableHandle), and a small thread of the owning engine hands those
// descriptors to importers over a unix datagram socket (SCM_RIGHTS).  The importer reserves one
// address range for the whole registration and maps every allocation at its offset, so that a
// descriptor's address translates with one addition, exactly as with an IPC mapping.
//
// Allocations must have been created with CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR among their
// requested handle types (PyTorch's expandable segments are); others stay same-process only.
#ifndef NIXL_B200_VMM_SHARE_H
#define NIXL_B200_VMM_SHARE_H

#include <cstdint>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace nixl_nvlink {

struct VmmChunk {
    uint64_t base = 0; // address in the owner's address space
    uint64_t size = 0;
    int fd = -1;       // exported descriptor, valid in the owner's process
};

// Exports every allocation under [addr, addr + len).  False (and nothing kept) when the range is not
// VMM memory or an allocation is not exportable.  The descriptors stay open until closeChunks().
bool vmmExportRange(uintptr_t addr, size_t len, std::vector<VmmChunk> &out);
void vmmCloseChunks(std::vector<VmmChunk> &chunks);

// A mapping of a peer's chunks in this process.
struct VmmMapping {
    uint64_t va = 0;       // start of the reserved range; corresponds to chunks.front().base in the owner
    uint64_t span = 0;
    std::vector<std::pair<uint64_t, uint64_t>> mapped; // (offset, size) of every mapped piece
};

// Maps chunks whose descriptors (valid in THIS process) are in `fds`, readable and writable by
// every GPU of this process that can reach the owning GPU.  The descriptors are closed.
bool vmmMap(const std::vector<VmmChunk> &chunks, const std::vector<int> &fds, int device_count, int owner_local_device, VmmMapping &out);
void vmmUnmap(VmmMapping &m);

// Thread that hands exported descriptors to importers.  Protocol on the abstract datagram socket
// `name`: request = "NIXLFD" + u32 count + count x i32 descriptor numbers (as published by the
// owner); reply (to the sender's address) = the same header with the descriptors attached as
// SCM_RIGHTS, or count = 0 when a number is not one this server exported.
class VmmFdServer {
public:
    ~VmmFdServer();
    bool start(const std::string &name); // idempotent
    void allow(int fd);
    void revoke(int fd);
    const std::string &name() const { return name_; }

private:
    void loop();
    std::string name_;
    int sock_ = -1;
    int wake_[2] = {-1, -1};
    std::thread th_;
    std::mutex mu_;
    std::vector<int> allowed_;
};

// Importer side of that protocol: the descriptors for `numbers`, in order.  Empty on failure.
std::vector<int> vmmFetchFds(const std::string &server_name, const std::vector<int> &numbers, int timeout_ms = 5000);

} // namespace nixl_nvlink

#endif

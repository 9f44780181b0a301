// Notification ring: lets the initiator's GPU tell the target that a transfer is complete.
//
// The datagram path needs the initiator's host in the loop: it has to see the completion word
// of its copy kernel before it can send the notification, so a target learns of a finished WRITE
// only after the initiator polled.  With the ring, the initiator's host fills a slot of a ring in
// the target's shared memory when it posts (names and message, plain CPU stores) and the last CTA
// of the copy kernel stores the slot's sequence word once the data is complete: one 8-byte store
// from the GPU into host memory of the target process.  The target's getNotifs reads the ring.
// (Role of the active-message notification of the reference's UCX backend,
// src/plugins/ucx/ucx_backend.cpp:1386-1427, which the NIC delivers after the data.)
//
// Layout of the shared-memory object (POSIX shm, name published in the connection info):
//   header: magic, slot count, slot size, head (claimed so far), tail (consumed so far)
//   slots[slot count]: { seq, name length, message length, claim number, pid, claim time, payload }
// Claim: a compare-and-swap on head by the initiator's host (refused when head - tail == slots:
// the caller then uses the datagram path).  The slot for claim number i is i % slots and becomes
// deliverable when its seq word equals i + 1.  The target consumes deliverable slots in any
// order (a long transfer does not hold back the notifications of later, shorter ones) and
// advances tail over the consumed prefix.  A slot whose claimant died before its kernel finished
// is skipped once the claim is older than a second and the pid is gone.
#ifndef NIXL_B200_NVLINK_NOTIF_RING_H
#define NIXL_B200_NVLINK_NOTIF_RING_H

#include <atomic>
#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace nixl_nvlink {

constexpr uint32_t kNotifSlots = 1024;
constexpr uint32_t kNotifSlotBytes = 512;
constexpr uint32_t kNotifVoid = 0xffffffffu; // name length of a slot that carries nothing (its post failed)

struct NotifSlot {
    uint64_t seq;      // claim number + 1 once deliverable: written by the initiator's GPU (or, to void the slot, its host)
    uint32_t nameLen;  // kNotifVoid: skip
    uint32_t msgLen;
    uint64_t claim;    // claim number + 1, written last by the claimant's host
    int64_t pid;       // claimant
    uint64_t claimNs;  // CLOCK_MONOTONIC at the claim
    char payload[kNotifSlotBytes - 40]; // agent name, then message
};
static_assert(sizeof(NotifSlot) == kNotifSlotBytes, "slot layout");
constexpr size_t kNotifPayloadMax = sizeof(NotifSlot::payload);

struct NotifRingHeader {
    uint64_t magic;
    uint32_t slots, slotBytes;
    alignas(64) std::atomic<uint64_t> head;
    alignas(64) std::atomic<uint64_t> tail;
    alignas(64) char pad[64];
};

// Target side: creates the shared-memory object and reads it.
class NotifRingOwner {
public:
    NotifRingOwner() = default;
    ~NotifRingOwner();
    NotifRingOwner(const NotifRingOwner &) = delete;
    NotifRingOwner &operator=(const NotifRingOwner &) = delete;

    bool create(const std::string &name); // name starts with '/'
    const std::string &name() const { return name_; }
    bool ok() const { return hdr_ != nullptr; }
    // Appends every deliverable notification as (agent name, message).
    void poll(std::vector<std::pair<std::string, std::string>> &out);
    uint64_t outstanding() const; // claimed and not yet consumed

private:
    std::string name_;
    NotifRingHeader *hdr_ = nullptr;
    NotifSlot *slots_ = nullptr;
    size_t bytes_ = 0;
    std::vector<uint8_t> taken_; // consumed ahead of tail
    uint64_t lastStuckCheckNs_ = 0;
};

// Initiator side: a mapping of a peer's ring.  One per ring name and process (open() caches).
class NotifRingWriter {
public:
    ~NotifRingWriter();
    static std::shared_ptr<NotifRingWriter> open(const std::string &name);

    // Claims a slot and writes `from` and `msg` into it.  On success *word is the host address of
    // the slot's sequence word and *seq the value that makes it deliverable.  False: the ring is
    // full or the payload does not fit; nothing was claimed.
    bool claim(const std::string &from, const std::string &msg, uint64_t **word, uint64_t *seq);
    // Host-side completion of a claimed slot: deliver as it is (`keep`) or as void.
    static void complete(uint64_t *word, uint64_t seq, bool keep);

    void *base() const { return base_; }
    size_t bytes() const { return bytes_; }
    // Device-visible address of the mapping, set by whoever registered it with CUDA (nullptr until then).
    std::atomic<char *> devBase{nullptr};
    std::atomic<bool> registerFailed{false};
    // Called with base() before the mapping goes away, when devBase was set (undoes the CUDA registration).
    static std::atomic<void (*)(void *)> unregisterHook;
    uint64_t *deviceWord(uint64_t *host_word) const {
        char *d = devBase.load(std::memory_order_acquire);
        return d ? reinterpret_cast<uint64_t *>(d + (reinterpret_cast<char *>(host_word) - static_cast<char *>(base_))) : nullptr;
    }

private:
    NotifRingWriter() = default;
    std::string name_;
    void *base_ = nullptr;
    size_t bytes_ = 0;
    NotifRingHeader *hdr_ = nullptr;
    NotifSlot *slots_ = nullptr;
};

} // namespace nixl_nvlink

#endif

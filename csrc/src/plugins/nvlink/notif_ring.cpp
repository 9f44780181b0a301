// Notification ring in POSIX shared memory (contract: notif_ring.h).
#include "plugins/nvlink/notif_ring.h"

#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <map>
#include <mutex>

#include <dirent.h>
#include <fcntl.h>
#include <signal.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace nixl_nvlink {

namespace {
constexpr uint64_t kMagic = 0x4e58524e47303031ull; // "NXRNG001"

uint64_t nowNs() {
    timespec ts{};
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return static_cast<uint64_t>(ts.tv_sec) * 1000000000ull + static_cast<uint64_t>(ts.tv_nsec);
}

size_t ringBytes() { return sizeof(NotifRingHeader) + size_t(kNotifSlots) * kNotifSlotBytes; }

std::mutex g_writersMu;
std::map<std::string, std::weak_ptr<NotifRingWriter>> g_writers;
} // namespace

// ---------------------------------------------------------------- owner

NotifRingOwner::~NotifRingOwner() {
    if (hdr_) ::munmap(hdr_, bytes_);
    if (!name_.empty()) ::shm_unlink(name_.c_str());
}

// Rings whose owner died without unlinking them ("/<prefix>.<pid>.<tag>"): removed by whoever creates the next one.
static void reapStaleRings(const std::string &name) {
    const size_t dot = name.find('.');
    if (name.size() < 2 || name[0] != '/' || dot == std::string::npos) return;
    const std::string prefix = name.substr(1, dot); // "nixl_b200."
    DIR *d = ::opendir("/dev/shm");
    if (!d) return;
    while (dirent *e = ::readdir(d)) {
        const std::string f = e->d_name;
        if (f.compare(0, prefix.size(), prefix) != 0) continue;
        char *end = nullptr;
        const long pid = std::strtol(f.c_str() + prefix.size(), &end, 10);
        if (pid <= 0 || !end || *end != '.') continue;
        if (::kill(static_cast<pid_t>(pid), 0) != 0 && errno == ESRCH) ::shm_unlink(("/" + f).c_str());
    }
    ::closedir(d);
}

bool NotifRingOwner::create(const std::string &name) {
    if (hdr_) return true;
    reapStaleRings(name);
    const int fd = ::shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR | O_CLOEXEC, 0600);
    if (fd < 0) return false;
    bytes_ = ringBytes();
    // posix_fallocate: a shared-memory file system without room answers here, not with SIGBUS at the first store
    if (::ftruncate(fd, static_cast<off_t>(bytes_)) != 0 || ::posix_fallocate(fd, 0, static_cast<off_t>(bytes_)) != 0) {
        ::close(fd);
        ::shm_unlink(name.c_str());
        return false;
    }
    void *p = ::mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) {
        ::shm_unlink(name.c_str());
        return false;
    }
    name_ = name;
    std::memset(p, 0, bytes_);
    hdr_ = new (p) NotifRingHeader();
    hdr_->slots = kNotifSlots;
    hdr_->slotBytes = kNotifSlotBytes;
    hdr_->head.store(0, std::memory_order_relaxed);
    hdr_->tail.store(0, std::memory_order_relaxed);
    slots_ = reinterpret_cast<NotifSlot *>(static_cast<char *>(p) + sizeof(NotifRingHeader));
    taken_.assign(kNotifSlots, 0);
    std::atomic_thread_fence(std::memory_order_release);
    hdr_->magic = kMagic; // last: a writer that maps the object checks it
    return true;
}

uint64_t NotifRingOwner::outstanding() const {
    if (!hdr_) return 0;
    return hdr_->head.load(std::memory_order_acquire) - hdr_->tail.load(std::memory_order_relaxed);
}

void NotifRingOwner::poll(std::vector<std::pair<std::string, std::string>> &out) {
    if (!hdr_) return;
    const uint64_t head = hdr_->head.load(std::memory_order_acquire);
    uint64_t tail = hdr_->tail.load(std::memory_order_relaxed);
    if (head == tail) return;
    for (uint64_t i = tail; i < head; ++i) {
        const uint32_t at = static_cast<uint32_t>(i % kNotifSlots);
        if (taken_[at]) continue;
        NotifSlot &s = slots_[at];
        if (__atomic_load_n(&s.seq, __ATOMIC_ACQUIRE) != i + 1) continue;
        // The payload was written by the claimant's host before it launched the kernel that stored seq.
        if (__atomic_load_n(&s.claim, __ATOMIC_ACQUIRE) == i + 1 && s.nameLen != kNotifVoid &&
            size_t(s.nameLen) + s.msgLen <= kNotifPayloadMax)
            out.emplace_back(std::string(s.payload, s.nameLen), std::string(s.payload + s.nameLen, s.msgLen));
        taken_[at] = 1;
    }
    // A claimant that died before its kernel finished would hold the tail for ever.
    if (tail < head && !taken_[tail % kNotifSlots]) {
        const uint64_t now = nowNs();
        if (now - lastStuckCheckNs_ > 100000000ull) {
            lastStuckCheckNs_ = now;
            NotifSlot &s = slots_[tail % kNotifSlots];
            if (__atomic_load_n(&s.claim, __ATOMIC_ACQUIRE) == tail + 1 && now - s.claimNs > 1000000000ull && s.pid > 0 &&
                ::kill(static_cast<pid_t>(s.pid), 0) != 0 && errno == ESRCH && __atomic_load_n(&s.seq, __ATOMIC_ACQUIRE) != tail + 1)
                taken_[tail % kNotifSlots] = 1;
        }
    }
    while (tail < head && taken_[tail % kNotifSlots]) {
        taken_[tail % kNotifSlots] = 0;
        ++tail;
    }
    hdr_->tail.store(tail, std::memory_order_release);
}

// ---------------------------------------------------------------- writer

std::atomic<void (*)(void *)> NotifRingWriter::unregisterHook{nullptr};

NotifRingWriter::~NotifRingWriter() {
    if (!base_) return;
    auto hook = unregisterHook.load(std::memory_order_acquire);
    if (hook && devBase.load(std::memory_order_acquire)) hook(base_);
    ::munmap(base_, bytes_);
}

std::shared_ptr<NotifRingWriter> NotifRingWriter::open(const std::string &name) {
    std::lock_guard<std::mutex> g(g_writersMu);
    auto it = g_writers.find(name);
    if (it != g_writers.end()) {
        if (auto sp = it->second.lock()) return sp;
        g_writers.erase(it);
    }
    const int fd = ::shm_open(name.c_str(), O_RDWR | O_CLOEXEC, 0);
    if (fd < 0) return nullptr;
    struct stat st{};
    if (::fstat(fd, &st) != 0 || static_cast<size_t>(st.st_size) != ringBytes()) {
        ::close(fd);
        return nullptr;
    }
    void *p = ::mmap(nullptr, ringBytes(), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) return nullptr;
    auto *hdr = static_cast<NotifRingHeader *>(p);
    if (__atomic_load_n(&hdr->magic, __ATOMIC_ACQUIRE) != kMagic || hdr->slots != kNotifSlots || hdr->slotBytes != kNotifSlotBytes) {
        ::munmap(p, ringBytes());
        return nullptr;
    }
    std::shared_ptr<NotifRingWriter> w(new NotifRingWriter());
    w->name_ = name;
    w->base_ = p;
    w->bytes_ = ringBytes();
    w->hdr_ = hdr;
    w->slots_ = reinterpret_cast<NotifSlot *>(static_cast<char *>(p) + sizeof(NotifRingHeader));
    g_writers[name] = w;
    return w;
}

bool NotifRingWriter::claim(const std::string &from, const std::string &msg, uint64_t **word, uint64_t *seq) {
    if (from.size() + msg.size() > kNotifPayloadMax || from.empty()) return false;
    uint64_t head = hdr_->head.load(std::memory_order_relaxed);
    for (;;) {
        if (head - hdr_->tail.load(std::memory_order_acquire) >= kNotifSlots) return false;
        if (hdr_->head.compare_exchange_weak(head, head + 1, std::memory_order_acq_rel, std::memory_order_relaxed)) break;
    }
    NotifSlot &s = slots_[head % kNotifSlots];
    s.nameLen = static_cast<uint32_t>(from.size());
    s.msgLen = static_cast<uint32_t>(msg.size());
    std::memcpy(s.payload, from.data(), from.size());
    std::memcpy(s.payload + from.size(), msg.data(), msg.size());
    s.pid = static_cast<int64_t>(::getpid());
    s.claimNs = nowNs();
    __atomic_store_n(&s.claim, head + 1, __ATOMIC_RELEASE);
    *word = &s.seq;
    *seq = head + 1;
    return true;
}

void NotifRingWriter::complete(uint64_t *word, uint64_t seq, bool keep) {
    auto *s = reinterpret_cast<NotifSlot *>(word); // seq is the slot's first member
    if (!keep) s->nameLen = kNotifVoid;
    __atomic_store_n(&s->seq, seq, __ATOMIC_RELEASE);
}

} // namespace nixl_nvlink

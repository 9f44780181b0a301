// Single-producer / single-consumer ring of fixed-size records in a memory-mapped file.
// The telemetry BUFFER exporter writes it; reader tools (another process) map the same
// file and drain it.  Role parity: the reference's src/utils/common/cyclic_buffer.h.
//
// File layout: Header (64 bytes) followed by `capacity` records of `record_size` bytes.
// `head` counts records ever written, `tail` records ever consumed; both only grow.
#ifndef NIXL_B200_RING_FILE_H
#define NIXL_B200_RING_FILE_H

#include <atomic>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <stdexcept>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

class nixlRingFile {
public:
    struct Header {
        uint32_t magic;       // 'NXRB'
        uint32_t version;     // telemetry format version
        uint32_t record_size;
        uint32_t capacity;
        std::atomic<uint64_t> head;
        std::atomic<uint64_t> tail;
        std::atomic<uint64_t> dropped; // records rejected because the ring was full
        uint8_t pad[24];
    };
    static_assert(sizeof(Header) == 64, "ring header size");
    static constexpr uint32_t kMagic = 0x4E585242u;

    // create=true: (re)initialise the file as an empty ring of `capacity` records.
    // create=false: attach to an existing ring (capacity/record_size read from the header).
    nixlRingFile(const std::string &path, bool create, uint32_t record_size = 0, uint32_t capacity = 0, uint32_t version = 0)
        : path_(path), owner_(create) {
        fd_ = ::open(path.c_str(), create ? (O_RDWR | O_CREAT | O_TRUNC) : O_RDWR, 0644);
        if (fd_ < 0) throw std::runtime_error("cannot open ring file " + path);
        if (create) {
            bytes_ = sizeof(Header) + static_cast<size_t>(record_size) * capacity;
            if (::ftruncate(fd_, static_cast<off_t>(bytes_)) != 0) {
                ::close(fd_);
                throw std::runtime_error("cannot size ring file " + path);
            }
        } else {
            struct stat st;
            if (::fstat(fd_, &st) != 0 || static_cast<size_t>(st.st_size) < sizeof(Header)) {
                ::close(fd_);
                throw std::runtime_error("ring file too small: " + path);
            }
            bytes_ = static_cast<size_t>(st.st_size);
        }
        void *m = ::mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd_, 0);
        if (m == MAP_FAILED) {
            ::close(fd_);
            throw std::runtime_error("cannot map ring file " + path);
        }
        hdr_ = static_cast<Header *>(m);
        if (create) {
            hdr_->magic = kMagic;
            hdr_->version = version;
            hdr_->record_size = record_size;
            hdr_->capacity = capacity;
            hdr_->head.store(0);
            hdr_->tail.store(0);
            hdr_->dropped.store(0);
        } else if (hdr_->magic != kMagic ||
                   sizeof(Header) + static_cast<size_t>(hdr_->record_size) * hdr_->capacity > bytes_) {
            ::munmap(m, bytes_);
            ::close(fd_);
            throw std::runtime_error("not a ring file: " + path);
        }
    }
    ~nixlRingFile() {
        if (hdr_) ::munmap(hdr_, bytes_);
        if (fd_ >= 0) ::close(fd_);
        if (owner_ && unlink_on_close_) ::unlink(path_.c_str());
    }
    nixlRingFile(const nixlRingFile &) = delete;
    nixlRingFile &operator=(const nixlRingFile &) = delete;

    void unlinkOnClose(bool v) { unlink_on_close_ = v; }
    uint32_t version() const { return hdr_->version; }
    uint32_t capacity() const { return hdr_->capacity; }
    uint32_t recordSize() const { return hdr_->record_size; }
    uint64_t dropped() const { return hdr_->dropped.load(std::memory_order_relaxed); }
    size_t size() const {
        return static_cast<size_t>(hdr_->head.load(std::memory_order_acquire) - hdr_->tail.load(std::memory_order_acquire));
    }

    bool push(const void *rec) {
        const uint64_t h = hdr_->head.load(std::memory_order_relaxed);
        if (h - hdr_->tail.load(std::memory_order_acquire) >= hdr_->capacity) {
            hdr_->dropped.fetch_add(1, std::memory_order_relaxed);
            return false;
        }
        std::memcpy(slot(h), rec, hdr_->record_size);
        hdr_->head.store(h + 1, std::memory_order_release);
        return true;
    }
    bool pop(void *rec) {
        const uint64_t t = hdr_->tail.load(std::memory_order_relaxed);
        if (t == hdr_->head.load(std::memory_order_acquire)) return false;
        std::memcpy(rec, slot(t), hdr_->record_size);
        hdr_->tail.store(t + 1, std::memory_order_release);
        return true;
    }

private:
    uint8_t *slot(uint64_t i) const {
        return reinterpret_cast<uint8_t *>(hdr_) + sizeof(Header) + (i % hdr_->capacity) * hdr_->record_size;
    }
    std::string path_;
    bool owner_;
    bool unlink_on_close_ = false;
    int fd_ = -1;
    size_t bytes_ = 0;
    Header *hdr_ = nullptr;
};

#endif

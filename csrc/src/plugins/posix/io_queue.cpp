#include "plugins/posix/io_queue.h"

#include <aio.h>
#include <cerrno>
#include <cstring>
#include <linux/aio_abi.h>
#include <linux/io_uring.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "utils/log.h"

namespace nixl_posix {
namespace {

void complete(IoBatchState *b, int err) {
    if (err) {
        int expected = 0;
        b->error.compare_exchange_strong(expected, err);
    }
    b->remaining.fetch_sub(1, std::memory_order_acq_rel);
}

// Full-length pread/pwrite (the kernel may return short counts).
int doIo(const IoOp &op) {
    char *p = static_cast<char *>(op.buf);
    size_t left = op.len;
    off_t off = op.offset;
    while (left) {
        const ssize_t r = op.is_read ? ::pread(op.fd, p, left, off) : ::pwrite(op.fd, p, left, off);
        if (r < 0) {
            if (errno == EINTR) continue;
            return errno;
        }
        if (r == 0) return EIO; // read past end of file
        p += r;
        off += r;
        left -= static_cast<size_t>(r);
    }
    return 0;
}

// ---------------------------------------------------------------- thread pool

class ThreadQueue final : public IoQueue {
public:
    explicit ThreadQueue(unsigned n) {
        if (n == 0) n = 1;
        for (unsigned i = 0; i < n; ++i) workers_.emplace_back([this] { run(); });
    }
    ~ThreadQueue() override {
        {
            std::lock_guard<std::mutex> g(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        for (auto &t : workers_) t.join();
    }
    const char *name() const override { return "threads"; }
    nixl_status_t enqueue(const IoOp &op, IoBatchState *batch) override {
        staged_.push_back({op, batch});
        return NIXL_SUCCESS;
    }
    nixl_status_t submit() override {
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto &s : staged_) q_.push_back(s);
        }
        staged_.clear();
        cv_.notify_all();
        return NIXL_SUCCESS;
    }
    void poll() override {}

private:
    struct Item { IoOp op; IoBatchState *batch; };
    void run() {
        std::unique_lock<std::mutex> lk(mu_);
        for (;;) {
            cv_.wait(lk, [this] { return stop_ || !q_.empty(); });
            if (q_.empty()) {
                if (stop_) return;
                continue;
            }
            Item it = q_.front();
            q_.pop_front();
            lk.unlock();
            complete(it.batch, doIo(it.op));
            lk.lock();
        }
    }
    std::vector<Item> staged_; // submitter-thread only
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<Item> q_;
    bool stop_ = false;
    std::vector<std::thread> workers_;
};

// ---------------------------------------------------------------- kernel AIO (raw syscalls)

class LinuxAioQueue final : public IoQueue {
public:
    explicit LinuxAioQueue(unsigned depth) : depth_(depth ? depth : 256) {
        if (::syscall(SYS_io_setup, depth_, &ctx_) != 0) {
            ctx_ = 0;
            NIXL_WARN << "POSIX backend: io_setup failed (" << std::strerror(errno) << ")";
        }
    }
    ~LinuxAioQueue() override {
        while (inflight_ > 0) poll();
        if (ctx_) ::syscall(SYS_io_destroy, ctx_);
    }
    bool ok() const { return ctx_ != 0; }
    const char *name() const override { return "linux_aio"; }
    nixl_status_t enqueue(const IoOp &op, IoBatchState *batch) override {
        auto *slot = new Slot{};
        slot->batch = batch;
        slot->op = op;
        std::memset(&slot->cb, 0, sizeof(slot->cb));
        slot->cb.aio_fildes = static_cast<uint32_t>(op.fd);
        slot->cb.aio_lio_opcode = op.is_read ? IOCB_CMD_PREAD : IOCB_CMD_PWRITE;
        slot->cb.aio_buf = reinterpret_cast<uint64_t>(op.buf);
        slot->cb.aio_nbytes = op.len;
        slot->cb.aio_offset = op.offset;
        slot->cb.aio_data = reinterpret_cast<uint64_t>(slot);
        staged_.push_back(slot);
        return NIXL_SUCCESS;
    }
    nixl_status_t submit() override {
        size_t i = 0;
        while (i < staged_.size()) {
            // Respect the kernel queue depth: reap before overfilling.
            while (inflight_ >= depth_) poll();
            constexpr size_t kBatch = 64;
            iocb *ptrs[kBatch];
            size_t n = 0;
            for (; n < kBatch && i + n < staged_.size() && inflight_ + n < depth_; ++n) ptrs[n] = &staged_[i + n]->cb;
            const long r = ::syscall(SYS_io_submit, ctx_, static_cast<long>(n), ptrs);
            if (r < 0) {
                if (errno == EAGAIN) {
                    poll();
                    continue;
                }
                const int err = errno;
                for (; i < staged_.size(); ++i) { // fail what could not be queued
                    complete(staged_[i]->batch, err);
                    delete staged_[i];
                }
                staged_.clear();
                return NIXL_ERR_BACKEND;
            }
            inflight_ += static_cast<size_t>(r);
            i += static_cast<size_t>(r);
        }
        staged_.clear();
        return NIXL_SUCCESS;
    }
    void poll() override {
        if (!inflight_) return;
        io_event ev[64];
        timespec zero{0, 0};
        const long n = ::syscall(SYS_io_getevents, ctx_, 0L, 64L, ev, &zero);
        for (long k = 0; k < n; ++k) {
            auto *slot = reinterpret_cast<Slot *>(ev[k].data);
            int err = 0;
            if (ev[k].res < 0) err = static_cast<int>(-ev[k].res);
            else if (static_cast<size_t>(ev[k].res) != slot->op.len) {
                // Short transfer: finish the remainder synchronously.
                IoOp rest = slot->op;
                rest.buf = static_cast<char *>(rest.buf) + ev[k].res;
                rest.len -= static_cast<size_t>(ev[k].res);
                rest.offset += ev[k].res;
                err = ev[k].res == 0 ? EIO : doIo(rest);
            }
            complete(slot->batch, err);
            delete slot;
            --inflight_;
        }
    }

private:
    struct Slot { iocb cb; IoBatchState *batch; IoOp op; };
    unsigned depth_;
    aio_context_t ctx_ = 0;
    std::vector<Slot *> staged_;
    size_t inflight_ = 0;
};

// ---------------------------------------------------------------- io_uring (raw syscalls, no liburing)

// Submission and completion rings are the kernel's shared-memory rings, mapped with mmap and
// driven by io_uring_setup / io_uring_enter through syscall(2).  The queue is used by one thread
// at a time (the backend serialises post and poll per request), so plain loads and stores with
// acquire / release on the ring heads and tails are enough.
class IoUringQueue final : public IoQueue {
public:
    explicit IoUringQueue(unsigned depth) {
        unsigned entries = 1;
        while (entries < (depth ? depth : 256) && entries < 4096) entries <<= 1;
        io_uring_params p;
        std::memset(&p, 0, sizeof(p));
        fd_ = static_cast<int>(::syscall(SYS_io_uring_setup, entries, &p));
        if (fd_ < 0) {
            NIXL_WARN << "POSIX backend: io_uring_setup failed (" << std::strerror(errno) << ")";
            return;
        }
        sqBytes_ = p.sq_off.array + p.sq_entries * sizeof(uint32_t);
        cqBytes_ = p.cq_off.cqes + p.cq_entries * sizeof(io_uring_cqe);
        const bool single = (p.features & IORING_FEAT_SINGLE_MMAP) != 0;
        if (single) sqBytes_ = cqBytes_ = sqBytes_ > cqBytes_ ? sqBytes_ : cqBytes_;
        sqRing_ = ::mmap(nullptr, sqBytes_, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd_, IORING_OFF_SQ_RING);
        cqRing_ = single ? sqRing_
                         : ::mmap(nullptr, cqBytes_, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd_, IORING_OFF_CQ_RING);
        sqeBytes_ = p.sq_entries * sizeof(io_uring_sqe);
        sqes_ = static_cast<io_uring_sqe *>(
            ::mmap(nullptr, sqeBytes_, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd_, IORING_OFF_SQES));
        if (sqRing_ == MAP_FAILED || cqRing_ == MAP_FAILED || sqes_ == MAP_FAILED) {
            NIXL_WARN << "POSIX backend: mapping the io_uring rings failed (" << std::strerror(errno) << ")";
            if (sqRing_ == MAP_FAILED) sqRing_ = nullptr;
            if (cqRing_ == MAP_FAILED) cqRing_ = nullptr;
            if (sqes_ == MAP_FAILED) sqes_ = nullptr;
            unmapAll(single);
            ::close(fd_);
            fd_ = -1;
            return;
        }
        singleMap_ = single;
        char *sq = static_cast<char *>(sqRing_), *cq = static_cast<char *>(cqRing_);
        sqHead_ = reinterpret_cast<std::atomic<uint32_t> *>(sq + p.sq_off.head);
        sqTail_ = reinterpret_cast<std::atomic<uint32_t> *>(sq + p.sq_off.tail);
        sqMask_ = *reinterpret_cast<uint32_t *>(sq + p.sq_off.ring_mask);
        sqArray_ = reinterpret_cast<uint32_t *>(sq + p.sq_off.array);
        cqHead_ = reinterpret_cast<std::atomic<uint32_t> *>(cq + p.cq_off.head);
        cqTail_ = reinterpret_cast<std::atomic<uint32_t> *>(cq + p.cq_off.tail);
        cqMask_ = *reinterpret_cast<uint32_t *>(cq + p.cq_off.ring_mask);
        cqes_ = reinterpret_cast<io_uring_cqe *>(cq + p.cq_off.cqes);
        sqEntries_ = p.sq_entries;
        cqEntries_ = p.cq_entries;
    }
    ~IoUringQueue() override {
        if (fd_ < 0) return;
        while (inflight_ > 0) reap(true);
        unmapAll(singleMap_);
        ::close(fd_);
    }
    bool ok() const { return fd_ >= 0; }
    const char *name() const override { return "io_uring"; }
    nixl_status_t enqueue(const IoOp &op, IoBatchState *batch) override {
        staged_.push_back(new Slot{batch, op});
        return NIXL_SUCCESS;
    }
    nixl_status_t submit() override {
        size_t i = 0;
        while (i < staged_.size()) {
            // Never have more in flight than the completion ring can hold.
            while (inflight_ >= cqEntries_) reap(true);
            uint32_t tail = sqTail_->load(std::memory_order_relaxed);
            const uint32_t head = sqHead_->load(std::memory_order_acquire);
            unsigned n = 0;
            while (i + n < staged_.size() && tail - head < sqEntries_ && inflight_ + n < cqEntries_) {
                Slot *slot = staged_[i + n];
                const uint32_t idx = tail & sqMask_;
                io_uring_sqe *e = &sqes_[idx];
                std::memset(e, 0, sizeof(*e));
                e->opcode = slot->op.is_read ? IORING_OP_READ : IORING_OP_WRITE;
                e->fd = slot->op.fd;
                e->addr = reinterpret_cast<uint64_t>(slot->op.buf);
                // One submission moves at most 1 GiB; the remainder of a larger (or short)
                // transfer is finished synchronously when its completion is reaped.
                e->len = static_cast<uint32_t>(slot->op.len < (1u << 30) ? slot->op.len : (1u << 30));
                e->off = static_cast<uint64_t>(slot->op.offset);
                e->user_data = reinterpret_cast<uint64_t>(slot);
                sqArray_[idx] = idx;
                ++tail;
                ++n;
            }
            sqTail_->store(tail, std::memory_order_release);
            unsigned left = n;
            while (left) {
                const long r = ::syscall(SYS_io_uring_enter, fd_, left, 0u, 0u, nullptr, 0);
                if (r < 0) {
                    if (errno == EINTR) continue;
                    if (errno == EAGAIN || errno == EBUSY) {
                        reap(true);
                        continue;
                    }
                    const int err = errno;
                    NIXL_ERROR << "POSIX backend: io_uring_enter failed (" << std::strerror(err) << ")";
                    // Entries the kernel did not take stay in the ring; fail them and everything
                    // not yet queued, and stop using this ring position.
                    for (size_t k = i + (n - left); k < staged_.size(); ++k) {
                        complete(staged_[k]->batch, err);
                        delete staged_[k];
                    }
                    sqTail_->store(sqHead_->load(std::memory_order_acquire), std::memory_order_release);
                    inflight_ += n - left;
                    staged_.clear();
                    return NIXL_ERR_BACKEND;
                }
                left -= static_cast<unsigned>(r);
            }
            inflight_ += n;
            i += n;
        }
        staged_.clear();
        return NIXL_SUCCESS;
    }
    void poll() override {
        if (inflight_) reap(false);
    }

private:
    struct Slot { IoBatchState *batch; IoOp op; };

    void unmapAll(bool single) {
        if (sqes_) ::munmap(sqes_, sqeBytes_);
        if (cqRing_ && !single) ::munmap(cqRing_, cqBytes_);
        if (sqRing_) ::munmap(sqRing_, sqBytes_);
        sqes_ = nullptr;
        sqRing_ = cqRing_ = nullptr;
    }

    // Consume what the completion ring holds; when `wait` is set and it is empty, block in the
    // kernel for one completion first.
    void reap(bool wait) {
        uint32_t head = cqHead_->load(std::memory_order_relaxed);
        if (wait && head == cqTail_->load(std::memory_order_acquire)) {
            long r;
            do r = ::syscall(SYS_io_uring_enter, fd_, 0u, 1u, IORING_ENTER_GETEVENTS, nullptr, 0);
            while (r < 0 && errno == EINTR);
        }
        const uint32_t tail = cqTail_->load(std::memory_order_acquire);
        for (; head != tail; ++head) {
            const io_uring_cqe &c = cqes_[head & cqMask_];
            auto *slot = reinterpret_cast<Slot *>(c.user_data);
            int err = 0;
            if (c.res < 0) err = -c.res;
            else if (static_cast<size_t>(c.res) != slot->op.len) {
                IoOp rest = slot->op;
                rest.buf = static_cast<char *>(rest.buf) + c.res;
                rest.len -= static_cast<size_t>(c.res);
                rest.offset += c.res;
                err = c.res == 0 ? EIO : doIo(rest);
            }
            complete(slot->batch, err);
            delete slot;
            --inflight_;
        }
        cqHead_->store(head, std::memory_order_release);
    }

    int fd_ = -1;
    bool singleMap_ = false;
    void *sqRing_ = nullptr, *cqRing_ = nullptr;
    io_uring_sqe *sqes_ = nullptr;
    size_t sqBytes_ = 0, cqBytes_ = 0, sqeBytes_ = 0;
    std::atomic<uint32_t> *sqHead_ = nullptr, *sqTail_ = nullptr, *cqHead_ = nullptr, *cqTail_ = nullptr;
    uint32_t sqMask_ = 0, cqMask_ = 0, sqEntries_ = 0, cqEntries_ = 0;
    uint32_t *sqArray_ = nullptr;
    io_uring_cqe *cqes_ = nullptr;
    std::vector<Slot *> staged_;
    size_t inflight_ = 0;
};

// ---------------------------------------------------------------- POSIX aio (glibc)

class PosixAioQueue final : public IoQueue {
public:
    ~PosixAioQueue() override {
        while (!inflight_.empty()) {
            poll();
            if (!inflight_.empty()) std::this_thread::yield();
        }
    }
    const char *name() const override { return "posix_aio"; }
    nixl_status_t enqueue(const IoOp &op, IoBatchState *batch) override {
        auto *slot = new Slot{};
        std::memset(&slot->cb, 0, sizeof(slot->cb));
        slot->cb.aio_fildes = op.fd;
        slot->cb.aio_buf = op.buf;
        slot->cb.aio_nbytes = op.len;
        slot->cb.aio_offset = op.offset;
        slot->batch = batch;
        slot->op = op;
        staged_.push_back(slot);
        return NIXL_SUCCESS;
    }
    nixl_status_t submit() override {
        for (auto *slot : staged_) {
            const int r = slot->op.is_read ? ::aio_read(&slot->cb) : ::aio_write(&slot->cb);
            if (r != 0) {
                complete(slot->batch, errno);
                delete slot;
            } else inflight_.push_back(slot);
        }
        staged_.clear();
        return NIXL_SUCCESS;
    }
    void poll() override {
        for (size_t i = 0; i < inflight_.size();) {
            Slot *slot = inflight_[i];
            const int e = ::aio_error(&slot->cb);
            if (e == EINPROGRESS) {
                ++i;
                continue;
            }
            int err = e;
            if (e == 0) {
                const ssize_t got = ::aio_return(&slot->cb);
                if (got < 0) err = EIO;
                else if (static_cast<size_t>(got) != slot->op.len) {
                    IoOp rest = slot->op;
                    rest.buf = static_cast<char *>(rest.buf) + got;
                    rest.len -= static_cast<size_t>(got);
                    rest.offset += got;
                    err = got == 0 ? EIO : doIo(rest);
                }
            } else ::aio_return(&slot->cb);
            complete(slot->batch, err);
            delete slot;
            inflight_[i] = inflight_.back();
            inflight_.pop_back();
        }
    }

private:
    struct Slot { aiocb cb; IoBatchState *batch; IoOp op; };
    std::vector<Slot *> staged_, inflight_;
};

} // namespace

std::unique_ptr<IoQueue> makeQueue(QueueKind kind, unsigned pool_size, unsigned kernel_depth) {
    if (kind == QueueKind::LINUX_AIO) {
        auto q = std::make_unique<LinuxAioQueue>(kernel_depth);
        if (q->ok()) return q;
        NIXL_WARN << "POSIX backend: kernel AIO unavailable, using the thread pool";
    } else if (kind == QueueKind::IO_URING) {
        auto q = std::make_unique<IoUringQueue>(kernel_depth);
        if (q->ok()) return q;
        NIXL_WARN << "POSIX backend: io_uring unavailable, using the thread pool";
    } else if (kind == QueueKind::POSIX_AIO) {
        return std::make_unique<PosixAioQueue>();
    }
    return std::make_unique<ThreadQueue>(pool_size);
}

} // namespace nixl_posix

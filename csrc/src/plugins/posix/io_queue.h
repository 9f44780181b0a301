// Asynchronous file I/O queues of the POSIX backend.
//
// Role parity with the reference's src/plugins/posix/io_queue.{h,cpp} and its three
// implementations (linux-aio, io_uring, POSIX aio).  Here:
//   THREADS   - a pool of workers doing pread/pwrite (default; no library needed)
//   LINUX_AIO - kernel AIO through raw io_setup/io_submit/io_getevents system calls
//   IO_URING  - io_uring through raw io_uring_setup/io_uring_enter system calls and mmap'd rings
//   POSIX_AIO - glibc aio_read/aio_write
// A kernel interface that is unavailable at run time (seccomp, old kernel) selects THREADS.
#ifndef NIXL_B200_POSIX_IO_QUEUE_H
#define NIXL_B200_POSIX_IO_QUEUE_H

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <sys/types.h>

#include "nixl_types.h"

namespace nixl_posix {

struct IoOp {
    int fd;
    void *buf;
    size_t len;
    off_t offset;
    bool is_read;
};

// Completion state of one batch, shared between submitter and queue.
struct IoBatchState {
    std::atomic<size_t> remaining{0};
    std::atomic<int> error{0}; // first errno seen, or EIO for short transfers
};

class IoQueue {
public:
    virtual ~IoQueue() = default;
    virtual const char *name() const = 0;
    // Queue one operation belonging to `batch` (whose `remaining` the caller already set).
    virtual nixl_status_t enqueue(const IoOp &op, IoBatchState *batch) = 0;
    // Hand queued operations to the OS.
    virtual nixl_status_t submit() = 0;
    // Reap completions; cheap when nothing finished.
    virtual void poll() = 0;
};

enum class QueueKind { THREADS, LINUX_AIO, IO_URING, POSIX_AIO };

std::unique_ptr<IoQueue> makeQueue(QueueKind kind, unsigned pool_size, unsigned kernel_depth);

} // namespace nixl_posix

#endif

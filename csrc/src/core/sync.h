// Thread-synchronisation policy of an agent.  NONE: the caller promises single-threaded
// use and locking is skipped.  STRICT: every call is exclusive.  RW: read-mostly calls
// (transfer posting, status, preparation) share the lock; calls that change the agent's
// tables take it exclusively.  Parity: the reference's src/core/sync.h:24.
#ifndef NIXL_B200_SYNC_H
#define NIXL_B200_SYNC_H

#include <shared_mutex>
#include "nixl_types.h"

class nixlLock {
public:
    explicit nixlLock(nixl_thread_sync_t mode) : mode_(mode) {}
    void lock() {
        if (mode_ != nixl_thread_sync_t::NIXL_THREAD_SYNC_NONE) mu_.lock();
    }
    void unlock() {
        if (mode_ != nixl_thread_sync_t::NIXL_THREAD_SYNC_NONE) mu_.unlock();
    }
    void lock_shared() {
        if (mode_ == nixl_thread_sync_t::NIXL_THREAD_SYNC_RW) mu_.lock_shared();
        else lock();
    }
    void unlock_shared() {
        if (mode_ == nixl_thread_sync_t::NIXL_THREAD_SYNC_RW) mu_.unlock_shared();
        else unlock();
    }
    nixl_thread_sync_t mode() const { return mode_; }

private:
    nixl_thread_sync_t mode_;
    std::shared_mutex mu_;
};

struct nixlExclusiveGuard {
    explicit nixlExclusiveGuard(nixlLock &l) : l_(l) { l_.lock(); }
    ~nixlExclusiveGuard() { l_.unlock(); }
    nixlLock &l_;
};
struct nixlSharedGuard {
    explicit nixlSharedGuard(nixlLock &l) : l_(l) { l_.lock_shared(); }
    ~nixlSharedGuard() { l_.unlock_shared(); }
    nixlLock &l_;
};

#endif

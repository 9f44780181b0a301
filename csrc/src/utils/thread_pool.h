// Minimal fixed-size thread pool for storage backends (tasks are void()).
#ifndef NIXL_B200_THREAD_POOL_H
#define NIXL_B200_THREAD_POOL_H

#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

class nixlThreadPool {
public:
    explicit nixlThreadPool(unsigned n) {
        if (n == 0) n = 1;
        for (unsigned i = 0; i < n; ++i) workers_.emplace_back([this] { run(); });
    }
    ~nixlThreadPool() {
        {
            std::lock_guard<std::mutex> g(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        for (auto &t : workers_) t.join();
    }
    void submit(std::function<void()> f) {
        {
            std::lock_guard<std::mutex> g(mu_);
            q_.push_back(std::move(f));
        }
        cv_.notify_one();
    }

private:
    void run() {
        std::unique_lock<std::mutex> lk(mu_);
        for (;;) {
            cv_.wait(lk, [this] { return stop_ || !q_.empty(); });
            if (q_.empty()) {
                if (stop_) return;
                continue;
            }
            auto f = std::move(q_.front());
            q_.pop_front();
            lk.unlock();
            f();
            lk.lock();
        }
    }
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<std::function<void()>> q_;
    bool stop_ = false;
    std::vector<std::thread> workers_;
};

#endif

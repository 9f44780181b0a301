#include "utils/log.h"

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <strings.h>

namespace nixl_log {
namespace {
std::atomic<int> g_level{-1};
std::atomic<unsigned long> g_problems{0};
std::mutex g_io;

Level parse(const char *s) {
    if (!s) return WARN;
    static const struct { const char *n; Level l; } tbl[] = {{"TRACE", TRACE}, {"DEBUG", DEBUG}, {"INFO", INFO},
                                                              {"WARN", WARN},   {"WARNING", WARN}, {"ERROR", ERROR},
                                                              {"FATAL", FATAL}, {"OFF", OFF}};
    for (auto &e : tbl)
        if (strcasecmp(s, e.n) == 0) return e.l;
    return WARN;
}
} // namespace

Level threshold() {
    int l = g_level.load(std::memory_order_relaxed);
    if (l < 0) {
        l = parse(std::getenv("NIXL_LOG_LEVEL"));
        g_level.store(l, std::memory_order_relaxed);
    }
    return static_cast<Level>(l);
}

void setThreshold(Level l) { g_level.store(l, std::memory_order_relaxed); }
unsigned long problemCount() { return g_problems.load(); }

void write(Level l, const char *file, int line, const std::string &msg) {
    static const char tag[] = {'T', 'D', 'I', 'W', 'E', 'F'};
    if (l >= WARN) g_problems.fetch_add(1);
    const char *base = std::strrchr(file, '/');
    base = base ? base + 1 : file;
    const auto now = std::chrono::system_clock::now().time_since_epoch();
    const long long us = std::chrono::duration_cast<std::chrono::microseconds>(now).count();
    std::lock_guard<std::mutex> g(g_io);
    std::fprintf(stderr, "%c%lld.%06lld %s:%d] %s\n", tag[l > FATAL ? FATAL : l], us / 1000000, us % 1000000, base, line,
                 msg.c_str());
}
} // namespace nixl_log

// Small process-wide helpers shared by the core and the plug-ins: monotonic time, a cycle-counter
// clock for hot paths, durations as text, host name, random identifiers.
//
// Parity: the reference's src/utils/common/nixl_time.h (microsecond / nanosecond stamps, fast
// clock), nixl_duration.{h,cpp} (duration parsing and printing), hostname.h, uuid_v4.{h,cpp} and
// str_util.h, folded into one header because everything here is a few lines.
#ifndef NIXL_B200_UTILS_MISC_H
#define NIXL_B200_UTILS_MISC_H

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <random>
#include <string>
#include <vector>

#include <unistd.h>

#if defined(__x86_64__)
#include <x86intrin.h>
#endif

namespace nixl_util {

// ---------------------------------------------------------------- time

inline uint64_t nowNs() {
    return static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count());
}
inline uint64_t nowUs() { return nowNs() / 1000; }
inline int64_t nowMs() { return static_cast<int64_t>(nowNs() / 1000000); }

// Cycle counter scaled to nanoseconds: a time stamp without a call into the C library's clock
// code, for paths that take one per request.  Calibrated once against the steady clock (1 ms);
// without a usable counter it is the steady clock.
class FastClock {
public:
    static uint64_t ns() {
        static const FastClock c;
        return c.read();
    }

private:
    double nsPerTick_ = 0;
    uint64_t tick0_ = 0, ns0_ = 0;

    static uint64_t ticks() {
#if defined(__x86_64__)
        return __rdtsc();
#elif defined(__aarch64__)
        uint64_t v;
        asm volatile("mrs %0, cntvct_el0" : "=r"(v));
        return v;
#else
        return 0;
#endif
    }
    FastClock() {
        const uint64_t t0 = ticks(), n0 = nowNs();
        if (t0 == 0 && ticks() == 0) return;
        while (nowNs() - n0 < 1000000) {}
        const uint64_t t1 = ticks(), n1 = nowNs();
        if (t1 > t0) {
            nsPerTick_ = static_cast<double>(n1 - n0) / static_cast<double>(t1 - t0);
            tick0_ = t1;
            ns0_ = n1;
        }
    }
    uint64_t read() const {
        if (nsPerTick_ <= 0) return nowNs();
        return ns0_ + static_cast<uint64_t>(static_cast<double>(ticks() - tick0_) * nsPerTick_);
    }
};

// "1.5s", "250ms", "40us", "7ns", or a bare number of microseconds.  False when the text is none of these.
inline bool parseDuration(const std::string &text, std::chrono::nanoseconds &out) {
    if (text.empty()) return false;
    char *end = nullptr;
    const double v = std::strtod(text.c_str(), &end);
    if (end == text.c_str() || v < 0) return false;
    const std::string unit = end;
    double scale;
    if (unit.empty() || unit == "us") scale = 1e3;
    else if (unit == "ns") scale = 1;
    else if (unit == "ms") scale = 1e6;
    else if (unit == "s") scale = 1e9;
    else if (unit == "m" || unit == "min") scale = 60e9;
    else return false;
    out = std::chrono::nanoseconds(static_cast<int64_t>(v * scale));
    return true;
}

// The largest unit that leaves at least one whole digit: "2.5s", "120ms", "35us", "800ns".
inline std::string formatDuration(std::chrono::nanoseconds d) {
    const double ns = static_cast<double>(d.count());
    char buf[48];
    if (ns >= 1e9) std::snprintf(buf, sizeof(buf), "%.3gs", ns / 1e9);
    else if (ns >= 1e6) std::snprintf(buf, sizeof(buf), "%.3gms", ns / 1e6);
    else if (ns >= 1e3) std::snprintf(buf, sizeof(buf), "%.3gus", ns / 1e3);
    else std::snprintf(buf, sizeof(buf), "%.0fns", ns);
    return buf;
}

// ---------------------------------------------------------------- identity

inline std::string hostName() {
    char buf[256] = {0};
    if (::gethostname(buf, sizeof(buf) - 1) != 0 || buf[0] == 0) return "localhost";
    return buf;
}

// Process-wide generator seeded from the system's entropy source and the pid (a forked child draws other numbers).
inline uint64_t random64() {
    static std::mutex mu;
    static std::mt19937_64 gen{(static_cast<uint64_t>(std::random_device{}()) << 32) ^ std::random_device{}() ^ (static_cast<uint64_t>(::getpid()) << 17)};
    static pid_t owner = ::getpid();
    std::lock_guard<std::mutex> g(mu);
    if (owner != ::getpid()) {
        owner = ::getpid();
        gen.seed((static_cast<uint64_t>(std::random_device{}()) << 32) ^ std::random_device{}() ^ (static_cast<uint64_t>(owner) << 17));
    }
    return gen();
}

// Random (version 4) UUID in the canonical 8-4-4-4-12 form.
inline std::string uuidV4() {
    uint64_t hi = random64(), lo = random64();
    hi = (hi & 0xffffffffffff0fffull) | 0x0000000000004000ull; // version 4
    lo = (lo & 0x3fffffffffffffffull) | 0x8000000000000000ull; // variant 10
    char buf[40];
    std::snprintf(buf, sizeof(buf), "%08x-%04x-%04x-%04x-%012llx", static_cast<unsigned>(hi >> 32), static_cast<unsigned>((hi >> 16) & 0xffff),
                  static_cast<unsigned>(hi & 0xffff), static_cast<unsigned>(lo >> 48), static_cast<unsigned long long>(lo & 0xffffffffffffull));
    return buf;
}

// ---------------------------------------------------------------- strings

inline std::vector<std::string> split(const std::string &text, char sep, bool keep_empty = false) {
    std::vector<std::string> out;
    size_t at = 0;
    for (;;) {
        const size_t next = text.find(sep, at);
        const std::string piece = text.substr(at, next == std::string::npos ? std::string::npos : next - at);
        if (keep_empty || !piece.empty()) out.push_back(piece);
        if (next == std::string::npos) break;
        at = next + 1;
    }
    return out;
}

inline std::string trim(const std::string &text) {
    const size_t a = text.find_first_not_of(" \t\r\n");
    if (a == std::string::npos) return "";
    const size_t b = text.find_last_not_of(" \t\r\n");
    return text.substr(a, b - a + 1);
}

} // namespace nixl_util

#endif

// Tiny test harness: CHECK macros, named cases, exit code = number of failed cases.
#ifndef NIXL_B200_TEST_HARNESS_H
#define NIXL_B200_TEST_HARNESS_H

#include <cstdio>
#include <cstdlib>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

namespace harness {
struct Failure : std::runtime_error { using std::runtime_error::runtime_error; };

struct Case { std::string name; std::function<void()> fn; };
inline std::vector<Case> &cases() { static std::vector<Case> c; return c; }
struct Reg { Reg(const char *n, std::function<void()> f) { cases().push_back({n, std::move(f)}); } };

inline int runAll(int argc, char **argv) {
    const std::string only = argc > 1 ? argv[1] : "";
    int failed = 0, ran = 0;
    for (auto &c : cases()) {
        if (!only.empty() && c.name.find(only) == std::string::npos) continue;
        ++ran;
        try {
            c.fn();
            std::printf("[ OK ] %s\n", c.name.c_str());
        } catch (const std::exception &e) {
            ++failed;
            std::printf("[FAIL] %s: %s\n", c.name.c_str(), e.what());
        }
        std::fflush(stdout);
    }
    std::printf("%d cases, %d failed\n", ran, failed);
    return failed;
}
} // namespace harness

#define TEST_CASE(name) \
    static void name(); \
    static harness::Reg reg_##name(#name, name); \
    static void name()

#define CHECK(cond) \
    do { \
        if (!(cond)) throw harness::Failure(std::string(__FILE__) + ":" + std::to_string(__LINE__) + ": CHECK(" #cond ") failed"); \
    } while (0)

#define CHECK_EQ(a, b) \
    do { \
        auto va_ = (a); \
        auto vb_ = (b); \
        if (!(va_ == vb_)) \
            throw harness::Failure(std::string(__FILE__) + ":" + std::to_string(__LINE__) + ": " #a " == " #b " failed (" + \
                                   std::to_string((long long)va_) + " vs " + std::to_string((long long)vb_) + ")"); \
    } while (0)

#define TEST_MAIN() \
    int main(int argc, char **argv) { return harness::runAll(argc, argv); }

#endif

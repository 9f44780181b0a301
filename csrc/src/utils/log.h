// Minimal leveled logger.  Level comes from NIXL_LOG_LEVEL (TRACE, DEBUG, INFO, WARN,
// ERROR, FATAL; default WARN), matching the knob documented for the reference
// (src/utils/common/nixl_log.cpp:39-75).  Lines go to stderr.
#ifndef NIXL_B200_LOG_H
#define NIXL_B200_LOG_H

#include <sstream>

namespace nixl_log {
enum Level { TRACE = 0, DEBUG = 1, INFO = 2, WARN = 3, ERROR = 4, FATAL = 5, OFF = 6 };
Level threshold();
void setThreshold(Level l);
void write(Level l, const char *file, int line, const std::string &msg);
// Count of WARN+ lines written since start (tests use it to assert "no problems logged").
unsigned long problemCount();

class Line {
public:
    Line(Level l, const char *file, int line) : lvl_(l), file_(file), line_(line) {}
    ~Line() { write(lvl_, file_, line_, ss_.str()); }
    template<class T> Line &operator<<(const T &v) { ss_ << v; return *this; }

private:
    Level lvl_;
    const char *file_;
    int line_;
    std::ostringstream ss_;
};
struct Voidify {
    void operator&(const Line &) {}
};
} // namespace nixl_log

// `cond ? (void)0 : Voidify() & stream` keeps the macro a single expression (no dangling else).
#define NIXL_LOG_AT(lvl) \
    (nixl_log::lvl < nixl_log::threshold()) ? (void)0 : nixl_log::Voidify() & nixl_log::Line(nixl_log::lvl, __FILE__, __LINE__)
#define NIXL_TRACE NIXL_LOG_AT(TRACE)
#define NIXL_DEBUG NIXL_LOG_AT(DEBUG)
#define NIXL_INFO NIXL_LOG_AT(INFO)
#define NIXL_WARN NIXL_LOG_AT(WARN)
#define NIXL_ERROR NIXL_LOG_AT(ERROR)

#endif

// Tracing facade: scoped spans, point marks and key/value attributes emitted by the
// agent's entry points, fanned out to zero or more trace backends.
//
// Behavioural parity with the reference's src/core/tracing (trace.h Kind :42, macros in
// trace_macros.h, plugin ABI trace_plugin.h): backends are chosen per process by
// NIXL_TRACE_BACKENDS (comma list); the NVTX backend is added automatically when an
// NVTX injection library is configured (NVTX_INJECTION64_PATH); with no backend every
// call is a cheap no-op; a correlation-id stack links the spans of one request.
// Backends: built-in "log" and "memory", and plugins libtrace_backend_<name>.so.
#ifndef NIXL_B200_TRACE_H
#define NIXL_B200_TRACE_H

#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

struct nixlAuxPluginHandle;

namespace nixl::trace {

enum class Kind : uint32_t { API = 0, REGISTER, PREPARE, POST, STATUS, NOTIF, METADATA, BACKEND, INTERNAL, KIND_COUNT };
const char *kindName(Kind k);

// A trace backend.  Span begin/end pairs nest per thread.
class Backend {
public:
    virtual ~Backend() = default;
    virtual const char *name() const = 0;
    virtual void spanBegin(const std::string &agent, Kind kind, const char *what, uint64_t correlation) = 0;
    virtual void spanEnd(const std::string &agent, Kind kind, const char *what, uint64_t correlation) = 0;
    virtual void mark(const std::string &agent, Kind kind, const char *what, uint64_t correlation) = 0;
    virtual void attr(const std::string &agent, const char *key, const std::string &value) {}
};

// Plugin ABI for libtrace_backend_<name>.so: exports nixl_trace_plugin_init.
#define NIXL_TRACE_PLUGIN_API_VERSION 1
struct TracePlugin {
    int api_version;
    Backend *(*create_backend)(const char *agent_name);
    void (*destroy_backend)(Backend *);
    const char *(*get_plugin_name)();
};

// One finished span or mark as recorded by the "memory" backend (tests read these).
struct Record {
    std::string agent;
    Kind kind;
    std::string what;
    uint64_t correlation;
    bool isMark;
    uint64_t durationNs;
};
std::vector<Record> memoryBackendDrain();

class Tracer;

class Span {
public:
    Span() = default;
    Span(const Tracer *t, Kind k, const char *what);
    Span(Span &&o) noexcept : t_(o.t_), kind_(o.kind_), what_(o.what_), corr_(o.corr_) { o.t_ = nullptr; }
    Span(const Span &) = delete;
    ~Span();

private:
    const Tracer *t_ = nullptr;
    Kind kind_ = Kind::API;
    const char *what_ = "";
    uint64_t corr_ = 0;
};

// Pushes a correlation id for the current thread; spans opened inside carry it.
class CorrelationScope {
public:
    explicit CorrelationScope(uint64_t id);
    ~CorrelationScope();
    static uint64_t current();
    static uint64_t fresh();
};

class Tracer {
public:
    explicit Tracer(const std::string &agent_name);
    ~Tracer();
    bool enabled() const { return !backends_.empty(); }
    Span span(Kind k, const char *what) const { return enabled() ? Span(this, k, what) : Span(); }
    void mark(Kind k, const char *what) const;
    void attr(const char *key, const std::string &value) const;
    std::vector<std::string> backendNames() const;

private:
    friend class Span;
    struct Slot {
        std::shared_ptr<nixlAuxPluginHandle> lib;
        Backend *impl = nullptr;
        void (*destroy)(Backend *) = nullptr;
    };
    std::string agent_;
    std::vector<Slot> backends_;
};

} // namespace nixl::trace

#define NIXL_TRACE_CAT2(a, b) a##b
#define NIXL_TRACE_CAT(a, b) NIXL_TRACE_CAT2(a, b)
#ifdef NIXL_DISABLE_TRACE
#define NIXL_TRACE_SCOPE(tracer, kind, what) ((void)0)
#define NIXL_TRACE_MARK(tracer, kind, what) ((void)0)
#else
#define NIXL_TRACE_SCOPE(tracer, kind, what) \
    auto NIXL_TRACE_CAT(nixl_span_, __LINE__) = (tracer).span(nixl::trace::Kind::kind, what)
#define NIXL_TRACE_MARK(tracer, kind, what) (tracer).mark(nixl::trace::Kind::kind, what)
#endif

#endif

#include "core/tracing/trace.h"

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <sstream>

#include "core/plugin_manager.h"
#include "utils/config.h"
#include "utils/log.h"
#include "utils/misc.h"

namespace nixl::trace {

const char *kindName(Kind k) {
    static const char *names[] = {"api", "register", "prepare", "post", "status", "notif", "metadata", "backend", "internal"};
    const auto i = static_cast<uint32_t>(k);
    return i < static_cast<uint32_t>(Kind::KIND_COUNT) ? names[i] : "?";
}

namespace {
thread_local std::vector<uint64_t> t_corr;
std::atomic<uint64_t> g_nextCorr{1};

using nixl_util::nowNs;

// Writes one log line per finished span (INFO level).
class LogBackend final : public Backend {
public:
    const char *name() const override { return "log"; }
    void spanBegin(const std::string &, Kind, const char *, uint64_t) override { t_starts.push_back(nowNs()); }
    void spanEnd(const std::string &agent, Kind kind, const char *what, uint64_t corr) override {
        const uint64_t t0 = t_starts.empty() ? nowNs() : t_starts.back();
        if (!t_starts.empty()) t_starts.pop_back();
        NIXL_INFO << "trace " << agent << " " << kindName(kind) << ":" << what << " corr=" << corr << " "
                  << (nowNs() - t0) / 1000.0 << "us";
    }
    void mark(const std::string &agent, Kind kind, const char *what, uint64_t corr) override {
        NIXL_INFO << "trace " << agent << " mark " << kindName(kind) << ":" << what << " corr=" << corr;
    }

private:
    static thread_local std::vector<uint64_t> t_starts;
};
thread_local std::vector<uint64_t> LogBackend::t_starts;

std::mutex g_memMu;
std::vector<Record> g_memRecords;

// Keeps finished spans in memory so tests can assert on them.
class MemoryBackend final : public Backend {
public:
    const char *name() const override { return "memory"; }
    void spanBegin(const std::string &, Kind, const char *, uint64_t) override { t_starts.push_back(nowNs()); }
    void spanEnd(const std::string &agent, Kind kind, const char *what, uint64_t corr) override {
        const uint64_t t0 = t_starts.empty() ? nowNs() : t_starts.back();
        if (!t_starts.empty()) t_starts.pop_back();
        std::lock_guard<std::mutex> g(g_memMu);
        if (g_memRecords.size() < 65536) g_memRecords.push_back({agent, kind, what, corr, false, nowNs() - t0});
    }
    void mark(const std::string &agent, Kind kind, const char *what, uint64_t corr) override {
        std::lock_guard<std::mutex> g(g_memMu);
        if (g_memRecords.size() < 65536) g_memRecords.push_back({agent, kind, what, corr, true, 0});
    }

private:
    static thread_local std::vector<uint64_t> t_starts;
};
thread_local std::vector<uint64_t> MemoryBackend::t_starts;
} // namespace

std::vector<Record> memoryBackendDrain() {
    std::lock_guard<std::mutex> g(g_memMu);
    std::vector<Record> out;
    out.swap(g_memRecords);
    return out;
}

CorrelationScope::CorrelationScope(uint64_t id) { t_corr.push_back(id); }
CorrelationScope::~CorrelationScope() {
    if (!t_corr.empty()) t_corr.pop_back();
}
uint64_t CorrelationScope::current() { return t_corr.empty() ? 0 : t_corr.back(); }
uint64_t CorrelationScope::fresh() { return g_nextCorr.fetch_add(1); }

Tracer::Tracer(const std::string &agent_name) : agent_(agent_name) {
    std::vector<std::string> wanted;
    if (auto spec = nixl::config::getValueOptional<std::string>("NIXL_TRACE_BACKENDS")) {
        std::istringstream in(*spec);
        std::string tok;
        while (std::getline(in, tok, ',')) {
            const size_t b = tok.find_first_not_of(" \t"), e = tok.find_last_not_of(" \t");
            if (b != std::string::npos) wanted.push_back(tok.substr(b, e - b + 1));
        }
    }
    // A profiler that injects NVTX gets ranges without further configuration.
    if (std::getenv("NVTX_INJECTION64_PATH") &&
        std::find(wanted.begin(), wanted.end(), std::string("nvtx")) == wanted.end())
        wanted.push_back("nvtx");

    for (const auto &w : wanted) {
        Slot s;
        if (w == "log") {
            s.impl = new LogBackend();
            s.destroy = [](Backend *b) { delete b; };
        } else if (w == "memory") {
            s.impl = new MemoryBackend();
            s.destroy = [](Backend *b) { delete b; };
        } else {
            s.lib = nixlPluginManager::getInstance().loadAuxPlugin("libtrace_backend_", w, "nixl_trace_plugin_init");
            auto *table = s.lib ? static_cast<TracePlugin *>(s.lib->table) : nullptr;
            if (!table || table->api_version != NIXL_TRACE_PLUGIN_API_VERSION) {
                NIXL_WARN << "trace backend '" << w << "' is not available";
                continue;
            }
            s.impl = table->create_backend(agent_.c_str());
            s.destroy = table->destroy_backend;
            if (!s.impl) continue;
        }
        backends_.push_back(std::move(s));
    }
}

Tracer::~Tracer() {
    for (auto &s : backends_)
        if (s.impl && s.destroy) s.destroy(s.impl);
}

void Tracer::mark(Kind k, const char *what) const {
    const uint64_t c = CorrelationScope::current();
    for (auto &s : backends_) s.impl->mark(agent_, k, what, c);
}

void Tracer::attr(const char *key, const std::string &value) const {
    for (auto &s : backends_) s.impl->attr(agent_, key, value);
}

std::vector<std::string> Tracer::backendNames() const {
    std::vector<std::string> n;
    for (auto &s : backends_) n.push_back(s.impl->name());
    return n;
}

Span::Span(const Tracer *t, Kind k, const char *what) : t_(t), kind_(k), what_(what), corr_(CorrelationScope::current()) {
    for (auto &s : t_->backends_) s.impl->spanBegin(t_->agent_, kind_, what_, corr_);
}

Span::~Span() {
    if (!t_) return;
    for (auto it = t_->backends_.rbegin(); it != t_->backends_.rend(); ++it) it->impl->spanEnd(t_->agent_, kind_, what_, corr_);
}

} // namespace nixl::trace

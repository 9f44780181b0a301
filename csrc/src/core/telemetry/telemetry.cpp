#include "core/telemetry/telemetry.h"

#include <algorithm>
#include <chrono>
#include <fnmatch.h>
#include <map>
#include <sstream>
#include <sys/stat.h>

#include "backend/backend_engine.h"
#include "core/plugin_manager.h"
#include "core/telemetry/ring_file.h"
#include "telemetry/telemetry_plugin.h"
#include "utils/config.h"
#include "utils/log.h"

namespace {
uint64_t nowUs() {
    return static_cast<uint64_t>(
        std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::system_clock::now().time_since_epoch()).count());
}

// ---- built-in sinks ----

// Collect-only sink: events are accepted and discarded.
class NopExporter final : public nixlTelemetryExporter {
public:
    using nixlTelemetryExporter::nixlTelemetryExporter;
    nixl_status_t exportEvent(const nixlTelemetryEvent &) override { return NIXL_SUCCESS; }
};

// Shared-memory ring at $NIXL_TELEMETRY_DIR/<agent>, drained by a reader process.
class BufferExporter final : public nixlTelemetryExporter {
public:
    explicit BufferExporter(const nixlTelemetryExporterInitParams &p) : nixlTelemetryExporter(p) {
        const auto dir = nixl::config::getValueOptional<std::string>(TELEMETRY_DIR_VAR);
        if (!dir || dir->empty()) throw nixlTelemetryBindFailed("BUFFER telemetry exporter needs NIXL_TELEMETRY_DIR");
        ::mkdir(dir->c_str(), 0755);
        try {
            ring_ = std::make_unique<nixlRingFile>(*dir + "/" + p.agentName, true, sizeof(nixlTelemetryEvent),
                                                   static_cast<uint32_t>(p.maxEventsBuffered), TELEMETRY_VERSION);
        } catch (const std::exception &e) {
            throw nixlTelemetryBindFailed(e.what());
        }
        ring_->unlinkOnClose(true);
    }
    nixl_status_t exportEvent(const nixlTelemetryEvent &e) override {
        return ring_->push(&e) ? NIXL_SUCCESS : NIXL_ERR_NOT_ALLOWED;
    }

private:
    std::unique_ptr<nixlRingFile> ring_;
};

std::mutex g_factoryMu;
std::map<std::string, nixlTelemetry::exporter_factory_t> &factories() {
    static auto *m = new std::map<std::string, nixlTelemetry::exporter_factory_t>{
        {"NOP", [](const nixlTelemetryExporterInitParams &p) { return std::make_unique<NopExporter>(p); }},
        {"BUFFER", [](const nixlTelemetryExporterInitParams &p) { return std::make_unique<BufferExporter>(p); }},
    };
    return *m;
}

std::string chooseExporter() {
    if (auto n = nixl::config::getValueOptional<std::string>(TELEMETRY_EXPORTER_VAR); n && !n->empty()) return *n;
    if (nixl::config::lookup(TELEMETRY_DIR_VAR)) return "BUFFER";
    return "NOP";
}

nixl_telemetry_metric_mask_t chooseMetrics() {
    nixl_telemetry_metric_mask_t mask{};
    std::vector<std::string> tokens;
    if (auto spec = nixl::config::getValueOptional<std::string>(TELEMETRY_ENABLED_METRICS_VAR)) {
        std::istringstream in(*spec);
        std::string tok;
        while (std::getline(in, tok, ',')) {
            const size_t b = tok.find_first_not_of(" \t"), e = tok.find_last_not_of(" \t");
            if (b != std::string::npos) tokens.push_back(tok.substr(b, e - b + 1));
        }
    }
    if (tokens.empty()) {
        mask.fill(true);
        return mask;
    }
    for (const auto &tok : tokens) {
        bool hit = false;
        for (size_t i = 0; i < nixl_telemetry_event_type_count; ++i) {
            const std::string name(nixlEnumStrings::telemetryEventTypeStr(static_cast<nixl_telemetry_event_type_t>(i)));
            if (fnmatch(tok.c_str(), name.c_str(), 0) == 0) mask[i] = hit = true;
        }
        if (!hit) NIXL_WARN << TELEMETRY_ENABLED_METRICS_VAR << ": no metric matches '" << tok << "'";
    }
    return mask;
}
} // namespace

bool nixlTelemetryStagingQueue::push(const nixlTelemetryEvent &e) {
    std::lock_guard<std::mutex> g(mu_);
    if (active_.size() >= cap_) {
        ++dropped_;
        return false;
    }
    active_.push_back(e);
    return true;
}

uint64_t nixlTelemetryStagingQueue::drain(std::vector<nixlTelemetryEvent> &out) {
    out.clear();
    out.reserve(cap_);
    std::lock_guard<std::mutex> g(mu_);
    active_.swap(out);
    const uint64_t d = dropped_;
    dropped_ = 0;
    return d;
}

void nixlTelemetry::registerStaticExporter(const std::string &name, exporter_factory_t factory) {
    std::lock_guard<std::mutex> g(g_factoryMu);
    factories()[name] = std::move(factory);
}

std::unique_ptr<nixlTelemetry> nixlTelemetry::create(const std::string &agent_name) {
    try {
        return std::make_unique<nixlTelemetry>(agent_name, chooseExporter());
    } catch (const nixlTelemetryBindFailed &e) {
        NIXL_WARN << e.what() << "; running without a telemetry sink";
    } catch (const std::exception &e) {
        NIXL_WARN << "telemetry disabled: " << e.what();
    }
    return nullptr;
}

nixlTelemetry::nixlTelemetry(const std::string &agent_name, const std::string &exporter_name)
    : agentName_(agent_name), exporterName_(exporter_name),
      maxBuffered_(nixl::config::getValueDefaulted<size_t>(TELEMETRY_BUFFER_SIZE_VAR, 4096)),
      exporter_(nullptr, [](nixlTelemetryExporter *e) { delete e; }), enabled_(chooseMetrics()),
      staging_(maxBuffered_ ? maxBuffered_ : 1),
      interval_(nixl::config::getValueDefaulted<uint64_t>(TELEMETRY_RUN_INTERVAL_VAR, 100)) {
    if (agent_name.empty()) throw std::invalid_argument("telemetry needs a non-empty agent name");
    if (maxBuffered_ == 0) throw std::invalid_argument("telemetry buffer size cannot be 0");
    nixlTelemetryExporterInitParams params{agent_name, maxBuffered_};
    exporter_factory_t factory;
    {
        std::lock_guard<std::mutex> g(g_factoryMu);
        auto it = factories().find(exporter_name);
        if (it != factories().end()) factory = it->second;
    }
    if (factory) {
        exporter_.reset(factory(params).release());
    } else {
        plugin_ = nixlPluginManager::getInstance().loadAuxPlugin("libtelemetry_exporter_", exporter_name,
                                                                 "nixl_telemetry_plugin_init");
        auto *table = plugin_ ? static_cast<nixlTelemetryPlugin *>(plugin_->table) : nullptr;
        if (!table || table->api_version != NIXL_TELEMETRY_PLUGIN_API_VERSION)
            throw nixlTelemetryBindFailed("telemetry exporter '" + exporter_name + "' is not available");
        nixlTelemetryExporter *raw = table->create_exporter(&params);
        if (!raw) throw nixlTelemetryBindFailed("telemetry exporter '" + exporter_name + "' failed to start");
        auto destroy = table->destroy_exporter;
        exporter_ = {raw, [destroy](nixlTelemetryExporter *e) { destroy(e); }};
    }
    worker_ = std::thread([this] { loop(); });
}

nixlTelemetry::~nixlTelemetry() {
    {
        std::lock_guard<std::mutex> g(wakeMu_);
        stop_ = true;
    }
    wake_.notify_all();
    if (worker_.joinable()) worker_.join();
    flushPendingEvents();
    exporter_.reset();
}

void nixlTelemetry::add(nixl_telemetry_event_type_t t, uint64_t v) {
    if (!enabled_[static_cast<size_t>(t)]) return;
    staging_.push(nixlTelemetryEvent(nowUs(), t, v));
}

void nixlTelemetry::addXferStats(uint64_t us, bool is_write, uint64_t bytes) {
    add(nixl_telemetry_event_type_t::AGENT_XFER_TIME, us);
    if (is_write) {
        updateTxBytes(bytes);
        updateTxRequestsNum(1);
    } else {
        updateRxBytes(bytes);
        updateRxRequestsNum(1);
    }
}

void nixlTelemetry::trackBackend(nixlBackendEngine *engine) {
    std::lock_guard<std::mutex> g(backendsMu_);
    backends_.push_back(engine);
}

void nixlTelemetry::untrackBackend(nixlBackendEngine *engine) {
    std::lock_guard<std::mutex> g(backendsMu_);
    backends_.erase(std::remove(backends_.begin(), backends_.end(), engine), backends_.end());
}

void nixlTelemetry::flushPendingEvents() {
    std::lock_guard<std::mutex> g(flushMu_);
    const uint64_t dropped = staging_.drain(scratch_);
    {
        std::lock_guard<std::mutex> b(backendsMu_);
        for (auto *engine : backends_)
            for (auto &e : engine->getTelemetryEvents()) {
                if (!e.timestampUs_) e.timestampUs_ = nowUs();
                if (enabled_[static_cast<size_t>(e.eventType_)]) scratch_.push_back(e);
            }
    }
    if (dropped && enabled_[static_cast<size_t>(nixl_telemetry_event_type_t::AGENT_TELEMETRY_EVENTS_DROPPED)])
        scratch_.emplace_back(nowUs(), nixl_telemetry_event_type_t::AGENT_TELEMETRY_EVENTS_DROPPED, dropped);
    if (scratch_.empty() || !exporter_) return;
    exporter_->beginBatch();
    for (const auto &e : scratch_) exporter_->exportEvent(e);
    exporter_->endBatch();
    scratch_.clear();
}

void nixlTelemetry::loop() {
    std::unique_lock<std::mutex> lk(wakeMu_);
    while (!stop_) {
        wake_.wait_for(lk, interval_, [this] { return stop_; });
        if (stop_) break;
        lk.unlock();
        flushPendingEvents();
        lk.lock();
    }
}

std::vector<uint64_t> nixlTelemetryHistogramBucketsUs() {
    std::vector<uint64_t> b;
    if (auto spec = nixl::config::getValueOptional<std::string>("NIXL_TELEMETRY_HISTOGRAM_BUCKETS_US")) {
        std::istringstream in(*spec);
        std::string tok;
        while (std::getline(in, tok, ',')) {
            auto v = nixl::config::convert<uint64_t>(tok);
            if (v && (b.empty() || *v > b.back())) b.push_back(*v);
        }
    }
    if (b.empty()) b = {10, 100, 1000, 10000, 100000, 1000000, 10000000};
    return b;
}

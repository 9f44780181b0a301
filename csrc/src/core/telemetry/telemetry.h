// Agent-side telemetry: counters and timings are staged in memory by the calling
// threads and flushed by a background thread to an exporter every
// NIXL_TELEMETRY_RUN_INTERVAL milliseconds (default 100).
//
// Behavioural parity with the reference's src/core/telemetry/telemetry.cpp: defaults
// (:79-85), exporter choice (NIXL_TELEMETRY_EXPORTER, else BUFFER when
// NIXL_TELEMETRY_DIR is set, else the collect-only NOP sink), metric allow-list with
// glob patterns (:204), bounded staging with a dropped-events counter.
#ifndef NIXL_B200_TELEMETRY_H
#define NIXL_B200_TELEMETRY_H

#include <array>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "telemetry/telemetry_exporter.h"

class nixlBackendEngine;
struct nixlAuxPluginHandle;

// Double-buffered bounded queue: producers append under a short lock, the flusher swaps
// the whole vector out.  Overflow is counted, not blocked on.
class nixlTelemetryStagingQueue {
public:
    explicit nixlTelemetryStagingQueue(size_t cap) : cap_(cap) { active_.reserve(cap); }
    bool push(const nixlTelemetryEvent &e);
    // Moves all staged events into `out` (cleared first); returns how many were dropped since the last drain.
    uint64_t drain(std::vector<nixlTelemetryEvent> &out);
    size_t capacity() const { return cap_; }

private:
    size_t cap_;
    std::mutex mu_;
    std::vector<nixlTelemetryEvent> active_;
    uint64_t dropped_ = 0;
};

class nixlTelemetry {
public:
    // nullptr when the chosen exporter cannot bind its output.
    static std::unique_ptr<nixlTelemetry> create(const std::string &agent_name);
    nixlTelemetry(const std::string &agent_name, const std::string &exporter_name);
    ~nixlTelemetry();

    void updateTxBytes(uint64_t n) { add(nixl_telemetry_event_type_t::AGENT_TX_BYTES, n); }
    void updateRxBytes(uint64_t n) { add(nixl_telemetry_event_type_t::AGENT_RX_BYTES, n); }
    void updateTxRequestsNum(uint64_t n) { add(nixl_telemetry_event_type_t::AGENT_TX_REQUESTS_NUM, n); }
    void updateRxRequestsNum(uint64_t n) { add(nixl_telemetry_event_type_t::AGENT_RX_REQUESTS_NUM, n); }
    void updateMemoryRegistered(uint64_t n) { add(nixl_telemetry_event_type_t::AGENT_MEMORY_REGISTERED, n); }
    void updateMemoryDeregistered(uint64_t n) { add(nixl_telemetry_event_type_t::AGENT_MEMORY_DEREGISTERED, n); }
    void updateErrorCount(nixl_status_t st) { add(nixlTelemetryEventTypeForStatus(st), 1); }
    void addPostTime(uint64_t us) { add(nixl_telemetry_event_type_t::AGENT_XFER_POST_TIME, us); }
    // Completed transfer: duration plus byte/request counters for the right direction.
    void addXferStats(uint64_t us, bool is_write, uint64_t bytes);

    // Backends whose own event queues are collected at every flush.
    void trackBackend(nixlBackendEngine *engine);
    void untrackBackend(nixlBackendEngine *engine);

    // Run one flush now on the calling thread (tests; also used at shutdown).
    void flushPendingEvents();
    bool isMetricEnabled(nixl_telemetry_event_type_t t) const { return enabled_[static_cast<size_t>(t)]; }
    const std::string &exporterName() const { return exporterName_; }

    // Register an exporter compiled into the application.
    using exporter_factory_t = std::function<std::unique_ptr<nixlTelemetryExporter>(const nixlTelemetryExporterInitParams &)>;
    static void registerStaticExporter(const std::string &name, exporter_factory_t factory);

private:
    void add(nixl_telemetry_event_type_t t, uint64_t v);
    void loop();

    std::string agentName_;
    std::string exporterName_;
    size_t maxBuffered_;
    std::shared_ptr<nixlAuxPluginHandle> plugin_; // keeps a dlopen'ed exporter's code mapped
    std::unique_ptr<nixlTelemetryExporter, std::function<void(nixlTelemetryExporter *)>> exporter_;
    nixl_telemetry_metric_mask_t enabled_{};
    nixlTelemetryStagingQueue staging_;
    std::mutex backendsMu_;
    std::vector<nixlBackendEngine *> backends_;
    std::mutex flushMu_;
    std::vector<nixlTelemetryEvent> scratch_;

    std::chrono::milliseconds interval_;
    std::mutex wakeMu_;
    std::condition_variable wake_;
    bool stop_ = false;
    std::thread worker_;
};

// Default histogram bucket upper bounds in microseconds (10 us ... 10 s), overridable by
// NIXL_TELEMETRY_HISTOGRAM_BUCKETS_US="10,100,...".
std::vector<uint64_t> nixlTelemetryHistogramBucketsUs();

#endif

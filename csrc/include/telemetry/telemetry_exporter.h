// Exporter interface: a sink that receives telemetry events flushed by the agent.
//
// Parity: role of the reference's src/api/cpp/telemetry/telemetry_exporter.h
// (exportEvent + batch hooks, NIXL_TELEMETRY_EXPORTER selects the sink, a sink that
// cannot bind its output throws nixlTelemetryBindFailed and the agent runs without one).
#ifndef NIXL_B200_TELEMETRY_EXPORTER_H
#define NIXL_B200_TELEMETRY_EXPORTER_H

#include <stdexcept>
#include <string>
#include "telemetry/telemetry_event.h"

struct nixlTelemetryExporterInitParams {
    std::string agentName;
    size_t maxEventsBuffered = 4096;
};

class nixlTelemetryBindFailed : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};

class nixlTelemetryExporter {
public:
    explicit nixlTelemetryExporter(const nixlTelemetryExporterInitParams &p) : agentName_(p.agentName) {}
    virtual ~nixlTelemetryExporter() = default;
    // Called once per event, between beginBatch and endBatch of one flush.
    virtual nixl_status_t exportEvent(const nixlTelemetryEvent &event) = 0;
    virtual void beginBatch() {}
    virtual void endBatch() {}
    const std::string &agentName() const { return agentName_; }

private:
    std::string agentName_;
};

#endif

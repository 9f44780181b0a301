// ABI of a telemetry exporter plugin: libtelemetry_exporter_<NAME>.so exports
// nixl_telemetry_plugin_init returning this table (parity: the reference's
// src/api/cpp/telemetry/telemetry_plugin.h).
#ifndef NIXL_B200_TELEMETRY_PLUGIN_H
#define NIXL_B200_TELEMETRY_PLUGIN_H

#include "telemetry/telemetry_exporter.h"

#define NIXL_TELEMETRY_PLUGIN_API_VERSION 1

struct nixlTelemetryPlugin {
    int api_version;
    nixlTelemetryExporter *(*create_exporter)(const nixlTelemetryExporterInitParams *params);
    void (*destroy_exporter)(nixlTelemetryExporter *exporter);
    const char *(*get_plugin_name)();
    const char *(*get_plugin_version)();
};

extern "C" {
__attribute__((visibility("default"))) nixlTelemetryPlugin *nixl_telemetry_plugin_init();
__attribute__((visibility("default"))) void nixl_telemetry_plugin_fini();
}

#endif

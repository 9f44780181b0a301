// Telemetry event record shared by the agent, the backends and exporter plugins.
//
// Parity: the 21 event ids and their snake_case names follow the reference's
// src/core/telemetry/telemetry_event.h:36-58,:119-159 (format version 4), so a
// reader of the reference's shared-memory ring decodes these records unchanged.
#ifndef NIXL_B200_TELEMETRY_EVENT_H
#define NIXL_B200_TELEMETRY_EVENT_H

#include <array>
#include <cstdint>
#include <cstring>
#include <string_view>
#include "nixl_types.h"

constexpr char TELEMETRY_ENABLED_VAR[] = "NIXL_TELEMETRY_ENABLE";
constexpr char TELEMETRY_EXPORTER_VAR[] = "NIXL_TELEMETRY_EXPORTER";
constexpr char TELEMETRY_DIR_VAR[] = "NIXL_TELEMETRY_DIR";
constexpr char TELEMETRY_BUFFER_SIZE_VAR[] = "NIXL_TELEMETRY_BUFFER_SIZE";
constexpr char TELEMETRY_RUN_INTERVAL_VAR[] = "NIXL_TELEMETRY_RUN_INTERVAL";
constexpr char TELEMETRY_ENABLED_METRICS_VAR[] = "NIXL_TELEMETRY_ENABLED_METRICS";
constexpr inline int TELEMETRY_VERSION = 4;

enum class nixl_telemetry_event_type_t : uint32_t {
    AGENT_TX_BYTES = 0,
    AGENT_RX_BYTES = 1,
    AGENT_TX_REQUESTS_NUM = 2,
    AGENT_RX_REQUESTS_NUM = 3,
    AGENT_MEMORY_REGISTERED = 4,
    AGENT_MEMORY_DEREGISTERED = 5,
    AGENT_XFER_TIME = 6,
    AGENT_XFER_POST_TIME = 7,
    AGENT_ERR_NOT_POSTED = 8,
    AGENT_ERR_INVALID_PARAM = 9,
    AGENT_ERR_BACKEND = 10,
    AGENT_ERR_NOT_FOUND = 11,
    AGENT_ERR_MISMATCH = 12,
    AGENT_ERR_NOT_ALLOWED = 13,
    AGENT_ERR_REPOST_ACTIVE = 14,
    AGENT_ERR_UNKNOWN = 15,
    AGENT_ERR_NOT_SUPPORTED = 16,
    AGENT_ERR_REMOTE_DISCONNECT = 17,
    AGENT_ERR_CANCELED = 18,
    AGENT_ERR_NO_TELEMETRY = 19,
    AGENT_TELEMETRY_EVENTS_DROPPED = 20,
};
inline constexpr size_t nixl_telemetry_event_type_count = 21;
using nixl_telemetry_metric_mask_t = std::array<bool, nixl_telemetry_event_type_count>;

// Error status -> its counter event (status -1 maps to id 8, -12 to id 19).
inline nixl_telemetry_event_type_t nixlTelemetryEventTypeForStatus(nixl_status_t s) {
    const int code = -static_cast<int>(s);
    if (code < 1 || code > 12) return nixl_telemetry_event_type_t::AGENT_ERR_UNKNOWN;
    return static_cast<nixl_telemetry_event_type_t>(7 + code);
}

namespace nixlEnumStrings {
inline std::string_view telemetryEventTypeStr(nixl_telemetry_event_type_t t) noexcept {
    static constexpr std::string_view names[nixl_telemetry_event_type_count] = {
        "agent_tx_bytes", "agent_rx_bytes", "agent_tx_requests_num", "agent_rx_requests_num",
        "agent_memory_registered", "agent_memory_deregistered", "agent_xfer_time", "agent_xfer_post_time",
        "agent_err_not_posted", "agent_err_invalid_param", "agent_err_backend", "agent_err_not_found",
        "agent_err_mismatch", "agent_err_not_allowed", "agent_err_repost_active", "agent_err_unknown",
        "agent_err_not_supported", "agent_err_remote_disconnect", "agent_err_canceled", "agent_err_no_telemetry",
        "agent_telemetry_events_dropped"};
    const auto i = static_cast<uint32_t>(t);
    return i < nixl_telemetry_event_type_count ? names[i] : std::string_view("unknown");
}
} // namespace nixlEnumStrings

// Fixed-size record: safe to place in a shared-memory ring.
struct nixlTelemetryEvent {
    uint64_t timestampUs_ = 0;
    nixl_telemetry_event_type_t eventType_ = nixl_telemetry_event_type_t::AGENT_TX_BYTES;
    uint64_t value_ = 0;

    nixlTelemetryEvent() = default;
    nixlTelemetryEvent(nixl_telemetry_event_type_t type, uint64_t value) : eventType_(type), value_(value) {}
    nixlTelemetryEvent(uint64_t ts_us, nixl_telemetry_event_type_t type, uint64_t value)
        : timestampUs_(ts_us), eventType_(type), value_(value) {}
};

#endif

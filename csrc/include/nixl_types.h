// Public enums, aliases and per-call option structs of the transfer library.
//
// API parity: mirrors the contract of the reference's src/api/cpp/nixl_types.h
// (memory types :41, ops :47, status codes :53-68, sync modes :74-79, option
// struct :168-234, per-request telemetry :261-288) so code written against the
// reference compiles unchanged.  Enumerator values are part of the wire/ABI
// contract and must not be renumbered.
#ifndef NIXL_B200_TYPES_H
#define NIXL_B200_TYPES_H

#include <chrono>
#include <cstdint>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

// ---- memory segment kinds (FILE_SEG stays last: it is used as an array bound) ----
enum nixl_mem_t { DRAM_SEG, VRAM_SEG, BLK_SEG, OBJ_SEG, FILE_SEG };

enum nixl_xfer_op_t { NIXL_READ, NIXL_WRITE };

// Positive = still running, zero = done, negative = error.
enum nixl_status_t {
    NIXL_IN_PROG = 1,
    NIXL_SUCCESS = 0,
    NIXL_ERR_NOT_POSTED = -1,
    NIXL_ERR_INVALID_PARAM = -2,
    NIXL_ERR_BACKEND = -3,
    NIXL_ERR_NOT_FOUND = -4,
    NIXL_ERR_MISMATCH = -5,
    NIXL_ERR_NOT_ALLOWED = -6,
    NIXL_ERR_REPOST_ACTIVE = -7,
    NIXL_ERR_UNKNOWN = -8,
    NIXL_ERR_NOT_SUPPORTED = -9,
    NIXL_ERR_REMOTE_DISCONNECT = -10,
    NIXL_ERR_CANCELED = -11,
    NIXL_ERR_NO_TELEMETRY = -12
};

enum class nixl_thread_sync_t {
    NIXL_THREAD_SYNC_NONE,
    NIXL_THREAD_SYNC_STRICT,
    NIXL_THREAD_SYNC_RW,
    NIXL_THREAD_SYNC_DEFAULT = NIXL_THREAD_SYNC_NONE,
};

enum class nixl_cost_t {
    ANALYTICAL_BACKEND = 0,
};

namespace nixlEnumStrings {
std::string memTypeStr(const nixl_mem_t &mem);
std::string xferOpStr(const nixl_xfer_op_t &op);
std::string statusStr(const nixl_status_t &status);
} // namespace nixlEnumStrings

using nixl_backend_t = std::string;
using nixl_telemetry_plugin_t = std::string;
// A blob is a byte string (may hold NULs); never treat it as a C string.
using nixl_blob_t = std::string;
using nixl_mem_list_t = std::vector<nixl_mem_t>;
using nixl_b_params_t = std::unordered_map<std::string, std::string>;
using nixl_notifs_t = std::unordered_map<std::string, std::vector<nixl_blob_t>>;
using nixl_query_resp_t = std::optional<nixl_b_params_t>;

inline constexpr uint16_t default_comm_port = 8888;
extern const std::string default_metadata_label;
extern const std::string default_partial_metadata_label;

class nixlBackendH;
class nixlXferReqH;
class nixlDlistH;

// Optional arguments accepted by most agent calls.  Which fields a call reads
// is documented beside that call in nixl.h.
struct nixlAgentOptionalArgs {
    std::vector<nixlBackendH *> backends; // restrict the call to these backends
    std::optional<nixl_blob_t> notif;     // notification message (preferred form)
    nixl_blob_t notifMsg;                 // legacy pair: message ...
    bool hasNotif = false;                // ... and "is set" flag
    bool skipDescMerge = false;           // makeXferReq: keep descriptors unmerged
    bool includeConnInfo = false;         // partial metadata: add connection info
    std::string ipAddr;                   // metadata exchange peer
    int port = default_comm_port;
    std::string metadataLabel;            // central-store key label
    nixl_blob_t customParam;              // passed through to the backend
};
using nixl_opt_args_t = nixlAgentOptionalArgs;

// Opaque handle to a prepared device-side memory view (see device/nixl_device.cuh).
using nixlMemViewH = void *;

using chrono_point_t = std::chrono::steady_clock::time_point;
using chrono_period_us_t = std::chrono::microseconds;

struct nixlXferTelemetry {
    chrono_point_t startTime;
    chrono_period_us_t postDuration{0};
    chrono_period_us_t xferDuration{0};
    size_t totalBytes = 0;
    size_t descCount = 0;
};
using nixl_xfer_telem_t = nixlXferTelemetry;

// Passing this as the agent name to prepXferDlist selects the local side.
#define NIXL_INIT_AGENT ""
// Placeholder remote-agent name marking a hole in a remote memory view.
extern const std::string nixl_null_agent;

#endif

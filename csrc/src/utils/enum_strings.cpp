// String forms of the public enums, plus the few global constants of nixl_types.h.
#include <iostream>
#include "backend/backend_plugin.h"
#include "nixl_descriptors.h"
#include "nixl_types.h"
#include "utils/log.h"

const std::string default_metadata_label = "metadata";
const std::string default_partial_metadata_label = "partial_metadata";
const std::string nixl_null_agent = "NULL_AGENT";

namespace nixlEnumStrings {
std::string memTypeStr(const nixl_mem_t &mem) {
    switch (mem) {
    case DRAM_SEG: return "DRAM_SEG";
    case VRAM_SEG: return "VRAM_SEG";
    case BLK_SEG: return "BLK_SEG";
    case OBJ_SEG: return "OBJ_SEG";
    case FILE_SEG: return "FILE_SEG";
    }
    return "BAD_SEG";
}
std::string xferOpStr(const nixl_xfer_op_t &op) {
    return op == NIXL_READ ? "READ" : op == NIXL_WRITE ? "WRITE" : "BAD_OP";
}
std::string statusStr(const nixl_status_t &status) {
    switch (status) {
    case NIXL_IN_PROG: return "NIXL_IN_PROG";
    case NIXL_SUCCESS: return "NIXL_SUCCESS";
    case NIXL_ERR_NOT_POSTED: return "NIXL_ERR_NOT_POSTED";
    case NIXL_ERR_INVALID_PARAM: return "NIXL_ERR_INVALID_PARAM";
    case NIXL_ERR_BACKEND: return "NIXL_ERR_BACKEND";
    case NIXL_ERR_NOT_FOUND: return "NIXL_ERR_NOT_FOUND";
    case NIXL_ERR_MISMATCH: return "NIXL_ERR_MISMATCH";
    case NIXL_ERR_NOT_ALLOWED: return "NIXL_ERR_NOT_ALLOWED";
    case NIXL_ERR_REPOST_ACTIVE: return "NIXL_ERR_REPOST_ACTIVE";
    case NIXL_ERR_UNKNOWN: return "NIXL_ERR_UNKNOWN";
    case NIXL_ERR_NOT_SUPPORTED: return "NIXL_ERR_NOT_SUPPORTED";
    case NIXL_ERR_REMOTE_DISCONNECT: return "NIXL_ERR_REMOTE_DISCONNECT";
    case NIXL_ERR_CANCELED: return "NIXL_ERR_CANCELED";
    case NIXL_ERR_NO_TELEMETRY: return "NIXL_ERR_NO_TELEMETRY";
    }
    return "BAD_STATUS";
}
} // namespace nixlEnumStrings

namespace nixl_detail {
void emitLine(const std::string &line) { std::cout << line << std::endl; }
void logPluginFailure(const char *what) { NIXL_ERROR << "backend engine construction failed: " << what; }
} // namespace nixl_detail

void nixlBasicDesc::print(const std::string &suffix) const { NIXL_INFO << "Desc " << to_string() << suffix; }
void nixlBlobDesc::print(const std::string &suffix) const {
    NIXL_INFO << "Desc " << to_string() << " meta[" << metaInfo.size() << "B]" << suffix;
}

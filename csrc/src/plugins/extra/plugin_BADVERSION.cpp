// A plugin that announces an unsupported API version: the plugin manager must refuse it.
#include "backend/backend_plugin.h"

extern "C" NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init() {
    static nixlBackendPlugin table = {NIXL_PLUGIN_API_VERSION + 41, nullptr, nullptr, [] { return "BADVERSION"; }, [] { return "0"; },
                                      [] { return nixl_b_params_t(); }, [] { return nixl_mem_list_t(); }};
    return &table;
}
extern "C" NIXL_PLUGIN_EXPORT void nixl_plugin_fini() {}

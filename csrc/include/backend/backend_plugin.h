// Plugin ABI: a backend lives in lib plugin_<NAME>.so and exports nixl_plugin_init /
// nixl_plugin_fini, or is registered statically with the plugin manager.
//
// Parity: function-table layout and API version follow the reference's
// src/api/cpp/backend/backend_plugin.h:33-57,:119-127.
#ifndef NIXL_B200_BACKEND_PLUGIN_H
#define NIXL_B200_BACKEND_PLUGIN_H

#include <exception>
#include <string>
#include "backend/backend_engine.h"

#define NIXL_PLUGIN_API_VERSION 1
#define NIXL_PLUGIN_EXPORT __attribute__((visibility("default")))

class nixlBackendPlugin {
public:
    int api_version;
    nixlBackendEngine *(*create_engine)(const nixlBackendInitParams *init_params);
    void (*destroy_engine)(nixlBackendEngine *engine);
    const char *(*get_plugin_name)();
    const char *(*get_plugin_version)();
    nixl_b_params_t (*get_backend_options)();
    nixl_mem_list_t (*get_backend_mems)();
};

namespace nixl_detail {
void logPluginFailure(const char *what);
}

// Builds the function table for an engine class with a (const nixlBackendInitParams*) constructor.
template<typename EngineType> class nixlBackendPluginCreator {
public:
    static nixlBackendPlugin *create(int api_version, const char *name, const char *version,
                                     const nixl_b_params_t &params, const nixl_mem_list_t &mems) {
        static const std::string s_name = name, s_version = version;
        static const nixl_b_params_t s_params = params;
        static const nixl_mem_list_t s_mems = mems;
        static nixlBackendPlugin table = {api_version,
                                          &make,
                                          [](nixlBackendEngine *e) { delete e; },
                                          []() { return s_name.c_str(); },
                                          []() { return s_version.c_str(); },
                                          []() { return s_params; },
                                          []() { return s_mems; }};
        return &table;
    }

private:
    static nixlBackendEngine *make(const nixlBackendInitParams *p) {
        try {
            return new EngineType(p);
        } catch (const std::exception &e) {
            nixl_detail::logPluginFailure(e.what());
            return nullptr;
        }
    }
};

typedef nixlBackendPlugin *(*nixlStaticPluginCreatorFunc)();

extern "C" {
NIXL_PLUGIN_EXPORT nixlBackendPlugin *nixl_plugin_init();
NIXL_PLUGIN_EXPORT void nixl_plugin_fini();
}

#endif

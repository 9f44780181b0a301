// Discovery and ownership of plugins: transfer backends (libplugin_<NAME>.so),
// telemetry exporters (libtelemetry_exporter_<NAME>.so) and trace backends
// (libtrace_backend_<name>.so), plus plugins compiled into the library ("static").
//
// Behavioural parity with the reference's src/core/nixl_plugin_manager.cpp: file-name
// prefixes (:33-35), API-version check at load (:95-122), search path = NIXL_PLUGIN_DIR
// then the library's own plugins/ directory (:385-399), static registration (:819-864).
// New here: an alias table so a program asking for the reference's default "UCX" backend
// receives the NVLink backend of this library.
#ifndef NIXL_B200_PLUGIN_MANAGER_H
#define NIXL_B200_PLUGIN_MANAGER_H

#include <map>
#include <set>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "backend/backend_plugin.h"

class nixlTelemetryExporter;
struct nixlTelemetryExporterInitParams;

// One loaded backend plugin.  Keeps the shared object mapped while any engine lives.
class nixlPluginHandle {
public:
    nixlPluginHandle(void *dl, nixlBackendPlugin *table) : dl_(dl), table_(table) {}
    ~nixlPluginHandle();
    nixlBackendEngine *createEngine(const nixlBackendInitParams *p) const { return table_->create_engine(p); }
    void destroyEngine(nixlBackendEngine *e) const { table_->destroy_engine(e); }
    const char *getName() const { return table_->get_plugin_name(); }
    const char *getVersion() const { return table_->get_plugin_version(); }
    nixl_b_params_t getBackendOptions() const { return table_->get_backend_options(); }
    nixl_mem_list_t getBackendMems() const { return table_->get_backend_mems(); }
    bool isStatic() const { return dl_ == nullptr; }

private:
    void *dl_;
    nixlBackendPlugin *table_;
};

// Generic handle for the two auxiliary plugin kinds: holds the dlopen handle and the
// plugin's exported table pointer (interpreted by the telemetry / tracing core).
struct nixlAuxPluginHandle {
    void *dl = nullptr;
    void *table = nullptr;
    std::string name;
    ~nixlAuxPluginHandle();
};

class nixlPluginManager {
public:
    static nixlPluginManager &getInstance();

    // Directories searched for plugin shared objects, first match wins.
    void addPluginDirectory(const std::string &dir);
    std::vector<std::string> getPluginDirectories() const;

    // Load (or return the already loaded) backend plugin.  nullptr if missing or if its
    // api_version differs from NIXL_PLUGIN_API_VERSION.
    std::shared_ptr<const nixlPluginHandle> loadBackendPlugin(const nixl_backend_t &name);
    std::shared_ptr<const nixlPluginHandle> loadPluginFromPath(const std::string &path);
    void unloadBackendPlugin(const nixl_backend_t &name);
    std::shared_ptr<const nixlPluginHandle> getBackendPlugin(const nixl_backend_t &name) const;

    // Every backend name that loadBackendPlugin could satisfy right now.
    std::vector<nixl_backend_t> getAvailableBackendPlugins() const;
    std::vector<nixl_backend_t> getLoadedBackendPluginNames() const;

    // Plugins linked into the library or registered by the application.
    void registerStaticBackend(const nixl_backend_t &name, nixlStaticPluginCreatorFunc creator);
    // "UCX" -> "NVLINK" and the like.  resolveAlias returns its argument when no alias exists.
    void addAlias(const nixl_backend_t &alias, const nixl_backend_t &target);
    nixl_backend_t resolveAlias(const nixl_backend_t &name) const;

    // Auxiliary kinds: returns the dlsym'ed `init_symbol()` result wrapped with its library.
    std::shared_ptr<nixlAuxPluginHandle> loadAuxPlugin(const std::string &file_prefix, const std::string &name,
                                                       const char *init_symbol);
    std::vector<std::string> listAuxPlugins(const std::string &file_prefix) const;

private:
    nixlPluginManager();
    std::string findFile(const std::string &file_name) const;

    mutable std::mutex mu_;
    std::vector<std::string> dirs_;
    std::map<nixl_backend_t, std::shared_ptr<const nixlPluginHandle>> loaded_;
    std::map<nixl_backend_t, nixlStaticPluginCreatorFunc> statics_;
    std::map<nixl_backend_t, nixl_backend_t> aliases_;
    mutable std::set<nixl_backend_t> aliasWarned_; // one WARN per aliased name
};

#endif

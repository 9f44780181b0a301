#include "core/plugin_manager.h"

#include <algorithm>
#include <cstdlib>
#include <dirent.h>
#include <dlfcn.h>
#include <sys/stat.h>

#include "utils/log.h"

namespace {
constexpr const char *kBackendPrefix = "libplugin_";
constexpr const char *kSuffix = ".so";

std::string dirOf(const std::string &path) {
    const size_t slash = path.rfind('/');
    return slash == std::string::npos ? "." : path.substr(0, slash);
}

// Directory holding this library (so the default plugin directory follows the install).
std::string selfDir() {
    Dl_info info;
    if (dladdr(reinterpret_cast<void *>(&selfDir), &info) && info.dli_fname) return dirOf(info.dli_fname);
    return ".";
}

std::vector<std::string> listDir(const std::string &dir, const std::string &prefix) {
    std::vector<std::string> names;
    DIR *d = ::opendir(dir.c_str());
    if (!d) return names;
    while (dirent *e = ::readdir(d)) {
        const std::string f = e->d_name;
        if (f.size() > prefix.size() + 3 && f.compare(0, prefix.size(), prefix) == 0 &&
            f.compare(f.size() - 3, 3, kSuffix) == 0)
            names.push_back(f.substr(prefix.size(), f.size() - prefix.size() - 3));
    }
    ::closedir(d);
    return names;
}
} // namespace

nixlPluginHandle::~nixlPluginHandle() {
    if (!dl_) return;
    if (auto fini = reinterpret_cast<void (*)()>(dlsym(dl_, "nixl_plugin_fini"))) fini();
    dlclose(dl_);
}

nixlAuxPluginHandle::~nixlAuxPluginHandle() {
    if (dl) dlclose(dl);
}

nixlPluginManager &nixlPluginManager::getInstance() {
    static nixlPluginManager *inst = new nixlPluginManager(); // leaked on purpose: engines may outlive static dtors
    return *inst;
}

nixlPluginManager::nixlPluginManager() {
    if (const char *env = std::getenv("NIXL_PLUGIN_DIR")) {
        std::string all = env;
        size_t start = 0;
        while (start <= all.size()) {
            const size_t colon = all.find(':', start);
            const std::string one = all.substr(start, colon == std::string::npos ? std::string::npos : colon - start);
            if (!one.empty()) dirs_.push_back(one);
            if (colon == std::string::npos) break;
            start = colon + 1;
        }
    }
    const std::string here = selfDir();
    dirs_.push_back(here + "/plugins");
    dirs_.push_back(here);
    // Names of the reference's transports without a plug-in of that name in this build.  UCX (and the GPU-initiated
    // GPUNETIO) resolve to the NVLink backend: inside one NVLink domain it is the engine that moves DRAM and VRAM
    // between agents, whatever fabric the caller's configuration was written for.  The transports that only exist to
    // reach other nodes resolve to the TCP backend, the one engine here that does.  A real plug-in of such a name wins.
    for (const char *name : {"UCX", "UCX_MO", "GPUNETIO"}) aliases_[name] = "NVLINK";
    for (const char *name : {"LIBFABRIC", "MOONCAKE", "UCCL"}) aliases_[name] = "TCP";
}

void nixlPluginManager::addPluginDirectory(const std::string &dir) {
    if (dir.empty()) return;
    std::lock_guard<std::mutex> g(mu_);
    if (std::find(dirs_.begin(), dirs_.end(), dir) == dirs_.end()) dirs_.insert(dirs_.begin(), dir);
}

std::vector<std::string> nixlPluginManager::getPluginDirectories() const {
    std::lock_guard<std::mutex> g(mu_);
    return dirs_;
}

std::string nixlPluginManager::findFile(const std::string &file_name) const {
    for (const auto &d : dirs_) {
        const std::string p = d + "/" + file_name;
        struct stat st;
        if (::stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode)) return p;
    }
    return "";
}

void nixlPluginManager::addAlias(const nixl_backend_t &alias, const nixl_backend_t &target) {
    std::lock_guard<std::mutex> g(mu_);
    aliases_[alias] = target;
}

nixl_backend_t nixlPluginManager::resolveAlias(const nixl_backend_t &name) const {
    std::lock_guard<std::mutex> g(mu_);
    // A real plugin of that name always wins over the alias.
    if (loaded_.count(name) || statics_.count(name) || !findFile(kBackendPrefix + name + kSuffix).empty()) return name;
    auto it = aliases_.find(name);
    if (it == aliases_.end()) return name;
    if (aliasWarned_.insert(name).second)
        NIXL_WARN << "backend name '" << name << "' has no plug-in in this build; it resolves to '" << it->second
                  << "' (transfers inside one NVLink domain only)";
    return it->second;
}

void nixlPluginManager::registerStaticBackend(const nixl_backend_t &name, nixlStaticPluginCreatorFunc creator) {
    std::lock_guard<std::mutex> g(mu_);
    statics_[name] = creator;
}

static std::shared_ptr<const nixlPluginHandle> openBackend(const std::string &path) {
    void *dl = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!dl) {
        NIXL_WARN << "cannot load plugin " << path << ": " << dlerror();
        return nullptr;
    }
    auto init = reinterpret_cast<nixlBackendPlugin *(*)()>(dlsym(dl, "nixl_plugin_init"));
    if (!init) {
        NIXL_WARN << path << " exports no nixl_plugin_init";
        dlclose(dl);
        return nullptr;
    }
    nixlBackendPlugin *table = init();
    if (!table) {
        NIXL_WARN << path << ": nixl_plugin_init returned null";
        dlclose(dl);
        return nullptr;
    }
    if (table->api_version != NIXL_PLUGIN_API_VERSION) {
        NIXL_WARN << path << ": plugin API version " << table->api_version << " != " << NIXL_PLUGIN_API_VERSION;
        if (auto fini = reinterpret_cast<void (*)()>(dlsym(dl, "nixl_plugin_fini"))) fini();
        dlclose(dl);
        return nullptr;
    }
    return std::make_shared<const nixlPluginHandle>(dl, table);
}

std::shared_ptr<const nixlPluginHandle> nixlPluginManager::loadPluginFromPath(const std::string &path) {
    auto h = openBackend(path);
    if (!h) return nullptr;
    std::lock_guard<std::mutex> g(mu_);
    auto &slot = loaded_[h->getName()];
    if (!slot) slot = h;
    return slot;
}

std::shared_ptr<const nixlPluginHandle> nixlPluginManager::loadBackendPlugin(const nixl_backend_t &name) {
    std::string path;
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = loaded_.find(name);
        if (it != loaded_.end()) return it->second;
        auto st = statics_.find(name);
        if (st != statics_.end()) {
            nixlBackendPlugin *table = st->second();
            if (!table || table->api_version != NIXL_PLUGIN_API_VERSION) return nullptr;
            auto h = std::make_shared<const nixlPluginHandle>(nullptr, table);
            loaded_[name] = h;
            return h;
        }
        path = findFile(kBackendPrefix + name + kSuffix);
    }
    if (path.empty()) {
        NIXL_INFO << "no plugin file for backend " << name;
        return nullptr;
    }
    auto h = openBackend(path);
    if (!h) return nullptr;
    std::lock_guard<std::mutex> g(mu_);
    auto &slot = loaded_[name];
    if (!slot) slot = h;
    return slot;
}

void nixlPluginManager::unloadBackendPlugin(const nixl_backend_t &name) {
    std::lock_guard<std::mutex> g(mu_);
    loaded_.erase(name);
}

std::shared_ptr<const nixlPluginHandle> nixlPluginManager::getBackendPlugin(const nixl_backend_t &name) const {
    std::lock_guard<std::mutex> g(mu_);
    auto it = loaded_.find(name);
    return it == loaded_.end() ? nullptr : it->second;
}

std::vector<nixl_backend_t> nixlPluginManager::getAvailableBackendPlugins() const {
    std::lock_guard<std::mutex> g(mu_);
    std::vector<nixl_backend_t> out;
    auto add = [&](const std::string &n) {
        if (std::find(out.begin(), out.end(), n) == out.end()) out.push_back(n);
    };
    for (auto &kv : loaded_) add(kv.first);
    for (auto &kv : statics_) add(kv.first);
    for (const auto &d : dirs_)
        for (const auto &n : listDir(d, kBackendPrefix)) add(n);
    std::sort(out.begin(), out.end());
    return out;
}

std::vector<nixl_backend_t> nixlPluginManager::getLoadedBackendPluginNames() const {
    std::lock_guard<std::mutex> g(mu_);
    std::vector<nixl_backend_t> out;
    for (auto &kv : loaded_) out.push_back(kv.first);
    return out;
}

std::shared_ptr<nixlAuxPluginHandle> nixlPluginManager::loadAuxPlugin(const std::string &file_prefix,
                                                                      const std::string &name, const char *init_symbol) {
    std::string path;
    {
        std::lock_guard<std::mutex> g(mu_);
        path = findFile(file_prefix + name + kSuffix);
    }
    if (path.empty()) return nullptr;
    void *dl = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!dl) {
        NIXL_WARN << "cannot load plugin " << path << ": " << dlerror();
        return nullptr;
    }
    auto init = reinterpret_cast<void *(*)()>(dlsym(dl, init_symbol));
    void *table = init ? init() : nullptr;
    if (!table) {
        NIXL_WARN << path << ": missing or failing " << init_symbol;
        dlclose(dl);
        return nullptr;
    }
    auto h = std::make_shared<nixlAuxPluginHandle>();
    h->dl = dl;
    h->table = table;
    h->name = name;
    return h;
}

std::vector<std::string> nixlPluginManager::listAuxPlugins(const std::string &file_prefix) const {
    std::lock_guard<std::mutex> g(mu_);
    std::vector<std::string> out;
    for (const auto &d : dirs_)
        for (const auto &n : listDir(d, file_prefix))
            if (std::find(out.begin(), out.end(), n) == out.end()) out.push_back(n);
    return out;
}

// nixlAgent: the north-bound API implementation.
//
// Behavioural contract (status codes, notification precedence, backend choice, merge
// rule, metadata tags) follows the reference's src/core/nixl_agent.cpp; the relevant
// reference lines are cited beside each rule below.  The structure is this library's own:
// one private nixlAgentData with ordered backend tables, sections that resolve descriptors
// in O(log n), and request handles that remember the generation of the remote metadata
// they were resolved against.
#include <algorithm>
#include <cstring>

#include "core/agent_data.h"
#include "utils/config.h"
#include "utils/log.h"

namespace {

using clock_t_ = std::chrono::steady_clock;

uint64_t usBetween(chrono_point_t a, chrono_point_t b) {
    return static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::microseconds>(b - a).count());
}

// Sync mode NONE is unsafe once a metadata thread can call back into the agent
// (reference: nixl_agent.cpp:151).
nixl_thread_sync_t effectiveSync(const nixlAgentConfig &cfg) {
    const bool md_thread = cfg.useListenThread || nixl::config::lookup("NIXL_ETCD_ENDPOINTS") ||
        nixl::config::lookup("NIXL_TCPSTORE_ENDPOINT");
    if (cfg.syncMode == nixl_thread_sync_t::NIXL_THREAD_SYNC_NONE && md_thread)
        return nixl_thread_sync_t::NIXL_THREAD_SYNC_STRICT;
    return cfg.syncMode;
}

// Backend pairs that must not coexist in one agent (both would claim the same memory
// with incompatible registrations).  Parity: nixl_agent.cpp:44.
const std::pair<const char *, const char *> kExclusive[] = {{"GDS", "GDS_MT"}};

template<class T> bool contains(const std::vector<T> &v, const T &x) { return std::find(v.begin(), v.end(), x) != v.end(); }

} // namespace

// ============================================================ nixlAgentData

nixlAgentData::nixlAgentData(const std::string &agent_name, const nixlAgentConfig &cfg)
    : name(agent_name), config(cfg), lock(effectiveSync(cfg)), tracer(agent_name) {
    if (agent_name.empty()) throw std::invalid_argument("agent needs a non-empty name");
    const bool telem_env = nixl::config::getValueDefaulted<bool>(TELEMETRY_ENABLED_VAR, false);
    if (telem_env || cfg.captureTelemetry) telemetry = nixlTelemetry::create(agent_name);
    // Started last: its threads call back into a fully built object.
    mdManager = std::make_unique<nixlMetadataManager>(*this, cfg);
    mdManager->start();
}

nixlAgentData::~nixlAgentData() {
    if (mdManager) mdManager->stop();
    mdManager.reset();
    // Remote metadata refers to engines, so it goes before them.
    remoteSections.clear();
}

nixlRemoteSection *nixlAgentData::remoteOf(const std::string &agent) const {
    auto it = remoteSections.find(agent);
    return it == remoteSections.end() ? nullptr : it->second.get();
}

nixlRemoteSection &nixlAgentData::selfSection() {
    auto &slot = remoteSections[name];
    if (!slot) slot = std::make_unique<nixlRemoteSection>(name);
    return *slot;
}

bool nixlAgentData::hasBackend(const nixlBackendEngine *e) const {
    return std::find(creationOrder.begin(), creationOrder.end(), e) != creationOrder.end();
}

void nixlAgentData::dropRemote(const std::string &agent) {
    if (agent == name) return;
    remoteSections.erase(agent);
    auto it = remoteBackends.find(agent);
    if (it != remoteBackends.end()) {
        for (auto &kv : it->second) {
            auto b = backends.find(kv.first);
            if (b != backends.end()) b->second->engine->disconnect(agent);
        }
        remoteBackends.erase(it);
    }
}

void nixlAgentData::finishStats(nixlXferReqH *req) const {
    const auto now = clock_t_::now();
    req->telemetry.xferDuration = chrono_period_us_t(usBetween(req->telemetry.startTime, now));
    if (telemetry)
        telemetry->addXferStats(static_cast<uint64_t>(req->telemetry.xferDuration.count()), req->backendOp == NIXL_WRITE,
                                req->telemetry.totalBytes);
}

// Blob layout (reference nixl_agent.cpp:1460-1498):
//   Agent=<name> Conns=<u64> { t=<backend> c=<conn blob> }* ""="MemSection" <sections>
nixl_status_t nixlAgentData::mdGetLocal(nixl_blob_t &out) const {
    nixlSharedGuard g(lock);
    if (connMd.empty()) return NIXL_ERR_INVALID_PARAM; // nobody could reach us anyway
    nixlSerDes sd;
    sd.addStr("Agent", name);
    const size_t n = connMd.size();
    sd.addBuf("Conns", &n, sizeof(n));
    for (auto &kv : connMd) {
        sd.addStr("t", kv.first);
        sd.addStr("c", kv.second);
    }
    sd.addStr("", "MemSection");
    if (auto st = localSection.serialize(&sd); st != NIXL_SUCCESS) return st;
    out = sd.exportStr();
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgentData::mdGetLocalPartial(const nixl_reg_dlist_t &descs, nixl_blob_t &out,
                                               const nixl_opt_args_t *opt) const {
    nixlSharedGuard g(lock);
    if (connMd.empty()) return NIXL_ERR_INVALID_PARAM;
    backend_set_t engines;
    if (opt && !opt->backends.empty()) {
        for (auto *h : opt->backends)
            if (h && hasBackend(h->engine)) engines.push_back(h->engine);
    } else if (!descs.isEmpty()) {
        engines = memToBackend[descs.getType()];
    }
    // Connection info travels only on request or with an empty list (nixl_agent.cpp:1566-1569).
    const bool with_conn = descs.isEmpty() || (opt && opt->includeConnInfo);
    nixlSerDes sd;
    sd.addStr("Agent", name);
    std::vector<std::pair<nixl_backend_t, nixl_blob_t>> conns;
    if (with_conn) {
        for (auto &kv : connMd) {
            if (opt && !opt->backends.empty()) {
                bool listed = false;
                for (auto *e : engines) listed |= e->getType() == kv.first;
                if (!listed) continue;
            }
            conns.emplace_back(kv.first, kv.second);
        }
    }
    const size_t n = conns.size();
    sd.addBuf("Conns", &n, sizeof(n));
    for (auto &c : conns) {
        sd.addStr("t", c.first);
        sd.addStr("c", c.second);
    }
    sd.addStr("", "MemSection");
    if (auto st = localSection.serializePartial(&sd, engines, descs); st != NIXL_SUCCESS) return st;
    out = sd.exportStr();
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgentData::mdLoadRemote(const nixl_blob_t &blob, std::string &agent_name) {
    NIXL_TRACE_SCOPE(tracer, METADATA, "loadRemoteMD");
    nixlSerDes sd;
    if (sd.importStr(blob) != NIXL_SUCCESS) return NIXL_ERR_MISMATCH;
    const std::string remote = sd.getStr("Agent");
    if (remote.empty()) return NIXL_ERR_MISMATCH;
    if (remote == name) return NIXL_ERR_INVALID_PARAM; // loading ourselves (nixl_agent.cpp:1628)

    size_t conn_count = 0;
    if (sd.getBuf("Conns", &conn_count, sizeof(conn_count)) != NIXL_SUCCESS) return NIXL_ERR_MISMATCH;
    if (conn_count > sd.remaining()) return NIXL_ERR_MISMATCH;

    nixlExclusiveGuard g(lock);
    auto &known = remoteBackends[remote];
    const bool had_any = !known.empty();
    size_t usable = 0;
    for (size_t i = 0; i < conn_count; ++i) {
        const nixl_backend_t type = sd.getStr("t");
        const nixl_blob_t conn = sd.getStr("c");
        if (type.empty() || conn.empty()) {
            if (!had_any && known.empty()) remoteBackends.erase(remote);
            return NIXL_ERR_MISMATCH;
        }
        auto b = backends.find(type);
        if (b == backends.end() || !b->second->engine->supportsRemote()) continue;
        auto k = known.find(type);
        if (k != known.end() && k->second == conn) {
            ++usable;
            continue;
        }
        if (b->second->engine->loadRemoteConnInfo(remote, conn) == NIXL_SUCCESS) {
            known[type] = conn;
            ++usable;
        }
    }
    // Partial metadata may omit connection info if we already know the peer.
    if (usable == 0 && known.empty()) {
        remoteBackends.erase(remote);
        NIXL_ERROR << "agent " << name << ": no backend in common with " << remote;
        return NIXL_ERR_BACKEND; // nixl_agent.cpp:1663
    }
    if (sd.getStr("") != "MemSection") return NIXL_ERR_MISMATCH;

    backend_map_t usable_engines;
    for (auto &kv : known) usable_engines[kv.first] = backends.at(kv.first)->engine;
    auto &slot = remoteSections[remote];
    const bool fresh = !slot;
    if (fresh) slot = std::make_unique<nixlRemoteSection>(remote);
    const nixl_status_t st = slot->loadRemoteData(&sd, usable_engines);
    if (st != NIXL_SUCCESS) {
        if (fresh) {
            remoteSections.erase(remote);
            if (!had_any) dropRemote(remote);
        }
        return st;
    }
    agent_name = remote;
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgentData::mdInvalidateRemote(const std::string &agent) {
    nixlExclusiveGuard g(lock);
    if (agent == name) return NIXL_ERR_INVALID_PARAM;
    const bool known = remoteSections.count(agent) || remoteBackends.count(agent);
    if (!known) return NIXL_ERR_NOT_FOUND;
    dropRemote(agent);
    return NIXL_SUCCESS;
}

// ============================================================ nixlAgent: lifecycle, plugins

nixlAgent::nixlAgent(const std::string &name, const nixlAgentConfig &cfg) : data(std::make_unique<nixlAgentData>(name, cfg)) {}

nixlAgent::~nixlAgent() {
    if (!data) return;
    // Order matters: stop threads that call into the agent, then drop remote metadata and
    // local registrations (both reference engines), then the engines themselves.
    if (data->mdManager) data->mdManager->stop();
    if (data->telemetry)
        for (auto *e : data->creationOrder) data->telemetry->untrackBackend(e);
}

nixl_status_t nixlAgent::getAvailPlugins(std::vector<nixl_backend_t> &plugins) {
    plugins = nixlPluginManager::getInstance().getAvailableBackendPlugins();
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgent::getPluginParams(const nixl_backend_t &type, nixl_mem_list_t &mems, nixl_b_params_t &params) const {
    auto &pm = nixlPluginManager::getInstance();
    auto plugin = pm.loadBackendPlugin(pm.resolveAlias(type));
    if (!plugin) return NIXL_ERR_NOT_FOUND;
    mems = plugin->getBackendMems();
    params = plugin->getBackendOptions();
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgent::getBackendParams(const nixlBackendH *backend, nixl_mem_list_t &mems, nixl_b_params_t &params) const {
    if (!backend) return NIXL_ERR_INVALID_PARAM;
    nixlSharedGuard g(data->lock);
    if (!data->hasBackend(backend->engine)) return NIXL_ERR_NOT_FOUND;
    mems = backend->engine->getSupportedMems();
    params = backend->engine->getCustomParams();
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgent::createBackend(const nixl_backend_t &type, const nixl_b_params_t &params, nixlBackendH *&bknd_hndl) {
    NIXL_TRACE_SCOPE(data->tracer, API, "createBackend");
    auto &pm = nixlPluginManager::getInstance();
    const nixl_backend_t real = pm.resolveAlias(type);
    nixlExclusiveGuard g(data->lock);
    if (data->backends.count(real)) return NIXL_ERR_INVALID_PARAM; // one engine per type
    for (auto &ex : kExclusive) {
        const bool clash = (real == ex.first && data->backends.count(ex.second)) ||
            (real == ex.second && data->backends.count(ex.first));
        if (clash) {
            NIXL_ERROR << "backends " << ex.first << " and " << ex.second << " cannot be used in one agent";
            return NIXL_ERR_NOT_ALLOWED;
        }
    }
    auto plugin = pm.loadBackendPlugin(real);
    if (!plugin) {
        NIXL_ERROR << "backend plugin " << type << " not found";
        data->noteError(NIXL_ERR_NOT_FOUND);
        return NIXL_ERR_NOT_FOUND;
    }
    nixl_b_params_t merged = plugin->getBackendOptions(); // defaults first, user overrides
    for (auto &kv : params) merged[kv.first] = kv.second;

    nixlBackendInitParams init;
    init.localAgent = data->name;
    init.type = real;
    init.customParams = &merged;
    init.enableProgTh = data->config.useProgThread;
    init.pthrDelay = data->config.pthrDelay;
    init.syncMode = data->lock.mode();
    init.enableTelemetry_ = static_cast<bool>(data->telemetry);

    nixlBackendEngine *engine = plugin->createEngine(&init);
    if (!engine || engine->getInitErr()) {
        if (engine) plugin->destroyEngine(engine);
        data->noteError(NIXL_ERR_BACKEND);
        return NIXL_ERR_BACKEND;
    }
    auto handle = std::make_unique<nixlBackendH>(engine, plugin);

    if (engine->supportsRemote()) {
        nixl_blob_t conn;
        if (engine->getConnInfo(conn) != NIXL_SUCCESS) return NIXL_ERR_BACKEND;
        data->connMd[real] = conn;
    }
    if (engine->supportsLocal()) {
        // Same-agent transfers go through the engine's loopback connection.
        if (engine->connect(data->name) != NIXL_SUCCESS) {
            data->connMd.erase(real);
            return NIXL_ERR_BACKEND;
        }
    }
    for (nixl_mem_t m : engine->getSupportedMems())
        if (m >= DRAM_SEG && m <= FILE_SEG) data->memToBackend[m].push_back(engine);
    if (engine->supportsNotif()) data->notifEngines.push_back(engine);
    data->creationOrder.push_back(engine);
    if (data->telemetry) data->telemetry->trackBackend(engine);
    bknd_hndl = handle.get();
    data->backends[real] = std::move(handle);
    return NIXL_SUCCESS;
}

// ============================================================ memory

nixl_status_t nixlAgent::queryMem(const nixl_reg_dlist_t &descs, std::vector<nixl_query_resp_t> &resp,
                                  const nixl_opt_args_t *extra_params) const {
    // Exactly one backend must be named (nixl_agent.cpp:429).
    if (!extra_params || extra_params->backends.size() != 1 || !extra_params->backends[0]) return NIXL_ERR_INVALID_PARAM;
    nixlSharedGuard g(data->lock);
    if (!data->hasBackend(extra_params->backends[0]->engine)) return NIXL_ERR_NOT_FOUND;
    return extra_params->backends[0]->engine->queryMem(descs, resp);
}

nixl_status_t nixlAgent::registerMem(const nixl_reg_dlist_t &descs, const nixl_opt_args_t *extra_params) {
    NIXL_TRACE_SCOPE(data->tracer, REGISTER, "registerMem");
    if (descs.isEmpty()) return NIXL_ERR_INVALID_PARAM;
    const nixl_mem_t mem = descs.getType();
    nixlExclusiveGuard g(data->lock);
    backend_set_t candidates;
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends) {
            if (!h || !data->hasBackend(h->engine)) return NIXL_ERR_NOT_FOUND;
            candidates.push_back(h->engine);
        }
    } else {
        candidates = data->memToBackend[mem];
    }
    if (candidates.empty()) {
        NIXL_ERROR << "no backend supports " << nixlEnumStrings::memTypeStr(mem);
        data->noteError(NIXL_ERR_NOT_FOUND);
        return NIXL_ERR_NOT_FOUND;
    }
    size_t accepted = 0;
    nixl_status_t last = NIXL_ERR_BACKEND;
    for (auto *engine : candidates) {
        std::vector<nixlSectionDesc> added;
        last = data->localSection.addDescList(descs, engine, &added);
        if (last != NIXL_SUCCESS) continue;
        if (engine->supportsLocal()) {
            // Mirror into our own "remote" view so createXferReq(..., own name) resolves (nixl_agent.cpp:475-483).
            if (data->selfSection().loadLocalData(mem, added, engine) != NIXL_SUCCESS) {
                data->localSection.remDescList(descs, engine);
                last = NIXL_ERR_BACKEND;
                continue;
            }
        }
        ++accepted;
    }
    if (accepted == 0) {
        data->noteError(last);
        return last < 0 ? last : NIXL_ERR_BACKEND;
    }
    if (data->telemetry) data->telemetry->updateMemoryRegistered(descs.totalBytes());
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgent::deregisterMem(const nixl_reg_dlist_t &descs, const nixl_opt_args_t *extra_params) {
    NIXL_TRACE_SCOPE(data->tracer, REGISTER, "deregisterMem");
    if (descs.isEmpty()) return NIXL_ERR_INVALID_PARAM;
    const nixl_mem_t mem = descs.getType();
    nixlExclusiveGuard g(data->lock);
    backend_set_t candidates;
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends)
            if (h && data->hasBackend(h->engine)) candidates.push_back(h->engine);
    } else if (const backend_set_t *have = data->localSection.queryBackends(mem)) {
        candidates = *have; // copy: remDescList may edit the set
    }
    size_t removed = 0;
    nixl_status_t bad = NIXL_SUCCESS;
    for (auto *engine : candidates) {
        if (engine->supportsLocal())
            if (auto *self = data->remoteOf(data->name)) self->unloadLocalData(mem, descs, engine);
        const nixl_status_t st = data->localSection.remDescList(descs, engine);
        if (st == NIXL_SUCCESS) ++removed;
        else bad = st;
    }
    if (removed == 0) {
        const nixl_status_t st = bad != NIXL_SUCCESS ? bad : NIXL_ERR_NOT_FOUND;
        data->noteError(st);
        return st;
    }
    if (data->telemetry) data->telemetry->updateMemoryDeregistered(descs.totalBytes());
    return bad;
}

nixl_status_t nixlAgent::makeConnection(const std::string &remote_agent, const nixl_opt_args_t *extra_params) {
    NIXL_TRACE_SCOPE(data->tracer, API, "makeConnection");
    nixlExclusiveGuard g(data->lock);
    auto it = data->remoteBackends.find(remote_agent);
    if (it == data->remoteBackends.end()) return NIXL_ERR_NOT_FOUND;
    std::vector<nixlBackendEngine *> targets;
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends) {
            if (!h || !data->hasBackend(h->engine)) return NIXL_ERR_NOT_FOUND; // a handle of another agent must not be driven from here
            if (it->second.count(h->getType())) targets.push_back(h->engine);
        }
    } else {
        for (auto &kv : it->second) targets.push_back(data->backends.at(kv.first)->engine);
    }
    if (targets.empty()) return NIXL_ERR_BACKEND;
    for (auto *e : targets)
        if (auto st = e->connect(remote_agent); st != NIXL_SUCCESS) return st;
    return NIXL_SUCCESS;
}

// ============================================================ transfer preparation

nixl_status_t nixlAgent::prepXferDlist(const nixl_xfer_dlist_t &descs, nixlDlistH *&dlist_hndl,
                                       const nixl_opt_args_t *extra_params) const {
    return prepXferDlist(NIXL_INIT_AGENT, descs, dlist_hndl, extra_params);
}

nixl_status_t nixlAgent::prepXferDlist(const std::string &agent_name, const nixl_xfer_dlist_t &descs, nixlDlistH *&dlist_hndl,
                                       const nixl_opt_args_t *extra_params) const {
    NIXL_TRACE_SCOPE(data->tracer, PREPARE, "prepXferDlist");
    if (descs.isEmpty()) return NIXL_ERR_INVALID_PARAM;
    const nixl_mem_t mem = descs.getType();
    const bool local_side = agent_name.empty();
    nixlSharedGuard g(data->lock);

    const nixlMemSection *section = &data->localSection;
    uint64_t generation = 0;
    if (!local_side) {
        // Naming ourselves selects our own registrations as a *target* (loopback).
        nixlRemoteSection *rs = data->remoteOf(agent_name);
        if (!rs) {
            data->noteError(NIXL_ERR_NOT_FOUND);
            return NIXL_ERR_NOT_FOUND;
        }
        section = rs;
        generation = rs->generation();
    }
    backend_set_t candidates;
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends)
            if (h && data->hasBackend(h->engine)) candidates.push_back(h->engine);
    } else if (const backend_set_t *have = section->queryBackends(mem)) {
        candidates = *have;
    }
    auto handle = std::make_unique<nixlDlistH>();
    handle->isLocal = local_side;
    handle->remoteAgent = local_side ? std::string() : agent_name;
    handle->generation = generation;
    handle->memType = mem;
    handle->count = static_cast<size_t>(descs.descCount());
    for (auto *engine : candidates) {
        auto resolved = std::make_unique<nixl_stride_dlist_t>(mem);
        if (section->populate(descs, engine, *resolved) == NIXL_SUCCESS) handle->descs[engine] = std::move(resolved);
    }
    if (handle->descs.empty()) {
        NIXL_ERROR << "prepXferDlist: no backend has registrations covering the list";
        data->noteError(NIXL_ERR_NOT_FOUND);
        return NIXL_ERR_NOT_FOUND;
    }
    dlist_hndl = handle.release();
    return NIXL_SUCCESS;
}

namespace {
// Carries the notification choice of a call into a request (nixl_agent.cpp:1147-1169).
void applyNotif(nixlXferReqH *req, const nixl_opt_args_t *extra) {
    if (!extra) return;
    if (extra->notif.has_value()) {
        req->notifMsg = *extra->notif;
        req->hasNotif = true;
    } else if (extra->hasNotif) {
        req->notifMsg = extra->notifMsg;
        req->hasNotif = true;
    } else {
        req->notifMsg.clear();
        req->hasNotif = false;
    }
}

nixl_opt_b_args_t backendArgs(const nixlXferReqH *req, const nixl_opt_args_t *extra) {
    nixl_opt_b_args_t b;
    b.notifMsg = req->notifMsg;
    b.hasNotif = req->hasNotif;
    if (extra) b.customParam = extra->customParam;
    return b;
}
} // namespace

nixl_status_t nixlAgent::makeXferReq(const nixl_xfer_op_t &operation, const nixlDlistH *local_side,
                                     const std::vector<int> &local_indices, const nixlDlistH *remote_side,
                                     const std::vector<int> &remote_indices, nixlXferReqH *&req_hndl,
                                     const nixl_opt_args_t *extra_params) const {
    NIXL_TRACE_SCOPE(data->tracer, PREPARE, "makeXferReq");
    req_hndl = nullptr;
    if (!local_side || !remote_side) return NIXL_ERR_INVALID_PARAM;
    if (!local_side->isLocal || remote_side->isLocal) return NIXL_ERR_INVALID_PARAM; // nixl_agent.cpp:721
    if (local_indices.empty() || local_indices.size() != remote_indices.size()) return NIXL_ERR_INVALID_PARAM;
    for (int i : local_indices)
        if (i < 0 || static_cast<size_t>(i) >= local_side->count) return NIXL_ERR_INVALID_PARAM;
    for (int i : remote_indices)
        if (i < 0 || static_cast<size_t>(i) >= remote_side->count) return NIXL_ERR_INVALID_PARAM;

    nixlSharedGuard g(data->lock);
    nixlRemoteSection *rs = data->remoteOf(remote_side->remoteAgent);
    if (!rs || rs->generation() != remote_side->generation) {
        data->noteError(NIXL_ERR_NOT_FOUND);
        return NIXL_ERR_NOT_FOUND;
    }
    // Backend: first listed one both sides resolved for, else first common one in our
    // creation (preference) order (nixl_agent.cpp:734-753).
    nixlBackendEngine *engine = nullptr;
    auto common = [&](nixlBackendEngine *e) { return local_side->descs.count(e) && remote_side->descs.count(e); };
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends)
            if (h && common(h->engine)) {
                engine = h->engine;
                break;
            }
    } else {
        for (auto *e : data->creationOrder)
            if (common(e)) {
                engine = e;
                break;
            }
    }
    if (!engine) {
        data->noteError(NIXL_ERR_INVALID_PARAM);
        return NIXL_ERR_INVALID_PARAM;
    }
    const nixl_stride_dlist_t &L = *local_side->descs.at(engine);
    const nixl_stride_dlist_t &R = *remote_side->descs.at(engine);
    const bool merge = !(extra_params && extra_params->skipDescMerge);

    auto req = std::make_unique<nixlXferReqH>();
    req->initiatorDescs = std::make_unique<nixl_meta_dlist_t>(local_side->memType);
    req->targetDescs = std::make_unique<nixl_meta_dlist_t>(remote_side->memType);
    req->initiatorDescs->reserve(local_indices.size());
    req->targetDescs->reserve(local_indices.size());
    size_t total = 0;
    for (size_t k = 0; k < local_indices.size(); ++k) {
        const nixlMetaDesc l = L.find(local_indices[k]).getMetaDesc(local_indices[k], 1);
        const nixlMetaDesc r = R.find(remote_indices[k]).getMetaDesc(remote_indices[k], 1);
        if (l.len != r.len) {
            data->noteError(NIXL_ERR_INVALID_PARAM);
            return NIXL_ERR_INVALID_PARAM; // nixl_agent.cpp:830
        }
        total += l.len;
        // Merge when both index lists advance by one and the new block starts exactly where
        // the previous one ended, on both sides, inside the same registrations.
        if (merge && k > 0 && local_indices[k] == local_indices[k - 1] + 1 && remote_indices[k] == remote_indices[k - 1] + 1) {
            nixlMetaDesc &pl = (*req->initiatorDescs)[req->initiatorDescs->descCount() - 1];
            nixlMetaDesc &pr = (*req->targetDescs)[req->targetDescs->descCount() - 1];
            if (pl.devId == l.devId && pr.devId == r.devId && pl.metadataP == l.metadataP && pr.metadataP == r.metadataP &&
                pl.addr + pl.len == l.addr && pr.addr + pr.len == r.addr) {
                pl.len += l.len;
                pr.len += r.len;
                continue;
            }
        }
        req->initiatorDescs->addDesc(l);
        req->targetDescs->addDesc(r);
    }
    req->engine = engine;
    req->remoteAgent = remote_side->remoteAgent;
    req->remoteGeneration = remote_side->generation;
    req->backendOp = operation;
    req->telemetry.totalBytes = total;
    req->telemetry.descCount = static_cast<size_t>(req->initiatorDescs->descCount());
    applyNotif(req.get(), extra_params);
    if (req->hasNotif && !engine->supportsNotif()) {
        data->noteError(NIXL_ERR_BACKEND);
        return NIXL_ERR_BACKEND;
    }
    const nixl_opt_b_args_t bargs = backendArgs(req.get(), extra_params);
    const nixl_status_t st = engine->prepXfer(operation, *req->initiatorDescs, *req->targetDescs, req->remoteAgent,
                                              req->backendHandle, &bargs);
    if (st != NIXL_SUCCESS) {
        data->noteError(st);
        return st;
    }
    req_hndl = req.release();
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgent::createXferReq(const nixl_xfer_op_t &operation, const nixl_xfer_dlist_t &local_descs,
                                       const nixl_xfer_dlist_t &remote_descs, const std::string &remote_agent,
                                       nixlXferReqH *&req_hndl, const nixl_opt_args_t *extra_params) const {
    NIXL_TRACE_SCOPE(data->tracer, PREPARE, "createXferReq");
    req_hndl = nullptr;
    if (local_descs.isEmpty() || local_descs.descCount() != remote_descs.descCount()) return NIXL_ERR_INVALID_PARAM;
    size_t total = 0;
    for (int i = 0; i < local_descs.descCount(); ++i) {
        if (local_descs[i].len != remote_descs[i].len) return NIXL_ERR_INVALID_PARAM; // nixl_agent.cpp:915
        total += local_descs[i].len;
    }
    nixlSharedGuard g(data->lock);
    nixlRemoteSection *rs = data->remoteOf(remote_agent);
    if (!rs) {
        NIXL_ERROR << "createXferReq: metadata of '" << remote_agent << "' is not loaded";
        data->noteError(NIXL_ERR_NOT_FOUND);
        return NIXL_ERR_NOT_FOUND;
    }
    // Candidates: ours for the local memory type, in preference order, that the remote also
    // registered its memory type with (nixl_agent.cpp:931-954).
    const backend_set_t *mine = data->localSection.queryBackends(local_descs.getType());
    const backend_set_t *theirs = rs->queryBackends(remote_descs.getType());
    if (!mine || !theirs || mine->empty() || theirs->empty()) {
        data->noteError(NIXL_ERR_NOT_FOUND);
        return NIXL_ERR_NOT_FOUND;
    }
    backend_set_t candidates;
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends)
            if (h && contains(*mine, h->engine) && contains(*theirs, h->engine)) candidates.push_back(h->engine);
    } else {
        for (auto *e : *mine)
            if (contains(*theirs, e)) candidates.push_back(e);
    }
    auto req = std::make_unique<nixlXferReqH>();
    req->initiatorDescs = std::make_unique<nixl_meta_dlist_t>(local_descs.getType());
    req->targetDescs = std::make_unique<nixl_meta_dlist_t>(remote_descs.getType());
    nixlBackendEngine *engine = nullptr;
    for (auto *e : candidates) {
        if (data->localSection.populate(local_descs, e, *req->initiatorDescs) != NIXL_SUCCESS) continue;
        if (rs->populate(remote_descs, e, *req->targetDescs) != NIXL_SUCCESS) continue;
        engine = e;
        break;
    }
    if (!engine) {
        NIXL_ERROR << "createXferReq: no backend covers both descriptor lists";
        data->noteError(NIXL_ERR_NOT_FOUND);
        return NIXL_ERR_NOT_FOUND;
    }
    req->engine = engine;
    req->remoteAgent = remote_agent;
    req->remoteGeneration = rs->generation();
    req->backendOp = operation;
    req->telemetry.totalBytes = total;
    req->telemetry.descCount = static_cast<size_t>(local_descs.descCount());
    applyNotif(req.get(), extra_params);
    if (req->hasNotif && !engine->supportsNotif()) {
        data->noteError(NIXL_ERR_BACKEND);
        return NIXL_ERR_BACKEND;
    }
    const nixl_opt_b_args_t bargs = backendArgs(req.get(), extra_params);
    const nixl_status_t st = engine->prepXfer(operation, *req->initiatorDescs, *req->targetDescs, remote_agent,
                                              req->backendHandle, &bargs);
    if (st != NIXL_SUCCESS) {
        data->noteError(st);
        return st;
    }
    req_hndl = req.release();
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgent::estimateXferCost(const nixlXferReqH *req, std::chrono::microseconds &duration,
                                          std::chrono::microseconds &err_margin, nixl_cost_t &method,
                                          const nixl_opt_args_t *extra_params) const {
    if (!req || !req->engine) return NIXL_ERR_INVALID_PARAM;
    nixlSharedGuard g(data->lock);
    return req->engine->estimateXferCost(req->backendOp, *req->initiatorDescs, *req->targetDescs, req->remoteAgent,
                                         req->backendHandle, duration, err_margin, method, extra_params);
}

// ============================================================ posting and status

nixl_status_t nixlAgent::postXferReq(nixlXferReqH *req, const nixl_opt_args_t *extra_params) const {
    if (!req) return NIXL_ERR_INVALID_PARAM;
    if (!req->correlation) req->correlation = nixl::trace::CorrelationScope::fresh();
    nixl::trace::CorrelationScope corr(req->correlation);
    NIXL_TRACE_SCOPE(data->tracer, POST, "postXferReq");
    nixlSharedGuard g(data->lock);

    // The remote's metadata must still be the instance this request was resolved against
    // (nixl_agent.cpp:1111-1126).
    nixlRemoteSection *rs = data->remoteOf(req->remoteAgent);
    if (!rs || rs->generation() != req->remoteGeneration) {
        data->noteError(NIXL_ERR_NOT_FOUND);
        return NIXL_ERR_NOT_FOUND;
    }
    if (req->status == NIXL_IN_PROG) {
        req->status = req->engine->checkXfer(req->backendHandle);
        if (req->status == NIXL_IN_PROG) {
            data->noteError(NIXL_ERR_REPOST_ACTIVE);
            return NIXL_ERR_REPOST_ACTIVE; // nixl_agent.cpp:1129-1135
        }
        if (req->status == NIXL_SUCCESS) data->finishStats(req);
    }
    applyNotif(req, extra_params);
    if (req->hasNotif && !req->engine->supportsNotif()) {
        data->noteError(NIXL_ERR_BACKEND);
        return NIXL_ERR_BACKEND;
    }
    const nixl_opt_b_args_t bargs = backendArgs(req, extra_params);
    req->telemetry.startTime = clock_t_::now();
    req->status = req->engine->postXfer(req->backendOp, *req->initiatorDescs, *req->targetDescs, req->remoteAgent,
                                        req->backendHandle, &bargs);
    req->postEnd = clock_t_::now();
    req->telemetry.postDuration = chrono_period_us_t(usBetween(req->telemetry.startTime, req->postEnd));
    if (req->status < 0) {
        data->noteError(req->status);
        if (req->status == NIXL_ERR_REMOTE_DISCONNECT) {
            // The peer is gone: forget its metadata so later calls fail fast (nixl_agent.cpp:1187).
            const std::string gone = req->remoteAgent;
            const nixl_status_t st = req->status;
            data->lock.unlock_shared();
            {
                nixlExclusiveGuard x(data->lock);
                data->dropRemote(gone);
            }
            data->lock.lock_shared();
            return st;
        }
        return req->status;
    }
    if (data->telemetry) data->telemetry->addPostTime(static_cast<uint64_t>(req->telemetry.postDuration.count()));
    if (req->status == NIXL_SUCCESS) data->finishStats(req);
    return req->status;
}

nixl_status_t nixlAgent::getXferStatus(nixlXferReqH *req) const {
    if (!req) return NIXL_ERR_INVALID_PARAM;
    if (req->status != NIXL_IN_PROG) return req->status; // only running requests are re-queried
    nixl::trace::CorrelationScope corr(req->correlation);
    NIXL_TRACE_SCOPE(data->tracer, STATUS, "getXferStatus");
    nixlSharedGuard g(data->lock);
    req->status = req->engine->checkXfer(req->backendHandle);
    if (req->status == NIXL_SUCCESS) data->finishStats(req);
    else if (req->status < 0) {
        data->noteError(req->status);
        if (req->status == NIXL_ERR_REMOTE_DISCONNECT) {
            const std::string gone = req->remoteAgent;
            const nixl_status_t st = req->status;
            data->lock.unlock_shared();
            {
                nixlExclusiveGuard x(data->lock);
                data->dropRemote(gone);
            }
            data->lock.lock_shared();
            return st;
        }
    }
    return req->status;
}

nixl_status_t nixlAgent::getXferTelemetry(const nixlXferReqH *req, nixl_xfer_telem_t &telemetry) const {
    if (!req) return NIXL_ERR_INVALID_PARAM;
    if (!data->telemetry) return NIXL_ERR_NO_TELEMETRY;
    if (req->status == NIXL_ERR_NOT_POSTED) return NIXL_ERR_NOT_POSTED;
    telemetry = req->telemetry;
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgent::queryXferBackend(const nixlXferReqH *req, nixlBackendH *&backend) const {
    if (!req) return NIXL_ERR_INVALID_PARAM;
    nixlSharedGuard g(data->lock);
    for (auto &kv : data->backends)
        if (kv.second->engine == req->engine) {
            backend = kv.second.get();
            return NIXL_SUCCESS;
        }
    return NIXL_ERR_NOT_FOUND;
}

nixl_status_t nixlAgent::releaseXferReq(nixlXferReqH *req) const {
    if (!req) return NIXL_ERR_INVALID_PARAM;
    NIXL_TRACE_SCOPE(data->tracer, API, "releaseXferReq");
    nixlSharedGuard g(data->lock);
    if (req->status == NIXL_IN_PROG) {
        req->status = req->engine->checkXfer(req->backendHandle);
        if (req->status == NIXL_IN_PROG) {
            // Ask the backend to cancel; if it cannot, the caller must wait (nixl_agent.cpp:1287-1313).
            if (req->engine->releaseReqH(req->backendHandle) != NIXL_SUCCESS) return NIXL_ERR_REPOST_ACTIVE;
            req->backendHandle = nullptr;
        }
    }
    delete req;
    return NIXL_SUCCESS;
}

nixl_status_t nixlAgent::releasedDlistH(nixlDlistH *dlist_hndl) const {
    if (!dlist_hndl) return NIXL_ERR_INVALID_PARAM;
    delete dlist_hndl;
    return NIXL_SUCCESS;
}

// ============================================================ memory views

nixl_status_t nixlAgent::prepMemView(const nixl_remote_dlist_t &dlist, nixlMemViewH &mvh, const nixl_opt_args_t *extra_params) const {
    NIXL_TRACE_SCOPE(data->tracer, PREPARE, "prepMemView(remote)");
    if (dlist.isEmpty()) return NIXL_ERR_INVALID_PARAM;
    nixlSharedGuard g(data->lock);
    backend_set_t candidates;
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends)
            if (h && data->hasBackend(h->engine)) candidates.push_back(h->engine);
    } else {
        candidates = data->creationOrder;
    }
    for (auto *engine : candidates) {
        nixl_remote_meta_dlist_t resolved(dlist.getType());
        bool ok = true;
        for (const auto &d : dlist) {
            if (d.remoteAgent == nixl_null_agent) { // hole: keeps indices aligned with rank numbers
                resolved.addDesc(nixlRemoteMetaDesc(nixl_null_agent));
                continue;
            }
            nixlRemoteSection *rs = data->remoteOf(d.remoteAgent);
            const nixlSecDescList *sec = rs ? rs->find(dlist.getType(), engine) : nullptr;
            const int at = sec ? sec->getCoveringIndex(d) : -1;
            if (at < 0) {
                ok = false;
                break;
            }
            nixlRemoteMetaDesc m(d.remoteAgent);
            static_cast<nixlBasicDesc &>(m) = d;
            m.metadataP = (*sec)[at].metadataP;
            resolved.addDesc(m);
        }
        if (!ok) continue;
        nixl_opt_b_args_t bargs;
        if (extra_params) bargs.customParam = extra_params->customParam;
        const nixl_status_t st = engine->prepMemView(resolved, mvh, &bargs);
        if (st == NIXL_ERR_NOT_SUPPORTED) continue;
        return st;
    }
    data->noteError(NIXL_ERR_NOT_FOUND);
    return NIXL_ERR_NOT_FOUND;
}

nixl_status_t nixlAgent::prepMemView(const nixl_local_dlist_t &dlist, nixlMemViewH &mvh, const nixl_opt_args_t *extra_params) const {
    NIXL_TRACE_SCOPE(data->tracer, PREPARE, "prepMemView(local)");
    if (dlist.isEmpty()) return NIXL_ERR_INVALID_PARAM;
    nixlSharedGuard g(data->lock);
    backend_set_t candidates;
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends)
            if (h && data->hasBackend(h->engine)) candidates.push_back(h->engine);
    } else if (const backend_set_t *have = data->localSection.queryBackends(dlist.getType())) {
        candidates = *have;
    }
    for (auto *engine : candidates) {
        nixl_meta_dlist_t resolved(dlist.getType());
        if (data->localSection.populate(dlist, engine, resolved) != NIXL_SUCCESS) continue;
        nixl_opt_b_args_t bargs;
        if (extra_params) bargs.customParam = extra_params->customParam;
        const nixl_status_t st = engine->prepMemView(resolved, mvh, &bargs);
        if (st == NIXL_ERR_NOT_SUPPORTED) continue;
        return st;
    }
    data->noteError(NIXL_ERR_NOT_FOUND);
    return NIXL_ERR_NOT_FOUND;
}

void nixlAgent::releaseMemView(nixlMemViewH mvh) const {
    if (!mvh) return;
    nixlSharedGuard g(data->lock);
    // Views are tagged by their creating engine; every engine ignores handles it does not own.
    for (auto *e : data->creationOrder) e->releaseMemView(mvh);
}

// ============================================================ notifications

nixl_status_t nixlAgent::getNotifs(nixl_notifs_t &notif_map, const nixl_opt_args_t *extra_params) {
    NIXL_TRACE_SCOPE(data->tracer, NOTIF, "getNotifs");
    nixlSharedGuard g(data->lock);
    backend_set_t engines;
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends)
            if (h && h->engine->supportsNotif() && data->hasBackend(h->engine)) engines.push_back(h->engine);
    } else {
        engines = data->notifEngines;
    }
    if (engines.empty()) return NIXL_ERR_BACKEND;
    nixl_status_t bad = NIXL_SUCCESS;
    size_t good = 0;
    for (auto *e : engines) {
        notif_list_t fresh;
        const nixl_status_t st = e->getNotifs(fresh);
        if (st < 0) {
            bad = st;
            continue;
        }
        ++good;
        for (auto &n : fresh) notif_map[n.first].push_back(std::move(n.second));
    }
    return good ? NIXL_SUCCESS : bad;
}

nixl_status_t nixlAgent::genNotif(const std::string &remote_agent, const nixl_blob_t &msg, const nixl_opt_args_t *extra_params) const {
    NIXL_TRACE_SCOPE(data->tracer, NOTIF, "genNotif");
    nixlSharedGuard g(data->lock);
    backend_set_t engines;
    if (extra_params && !extra_params->backends.empty()) {
        for (auto *h : extra_params->backends)
            if (h && h->engine->supportsNotif() && data->hasBackend(h->engine)) engines.push_back(h->engine);
    } else {
        engines = data->notifEngines;
    }
    const bool to_self = remote_agent == data->name;
    const auto *their = to_self ? nullptr : [&]() -> const std::unordered_map<nixl_backend_t, nixl_blob_t> * {
        auto it = data->remoteBackends.find(remote_agent);
        return it == data->remoteBackends.end() ? nullptr : &it->second;
    }();
    if (!to_self && !their) {
        data->noteError(NIXL_ERR_NOT_FOUND);
        return NIXL_ERR_NOT_FOUND;
    }
    for (auto *e : engines) {
        if (to_self ? !e->supportsLocal() : !their->count(e->getType())) continue;
        const nixl_status_t st = e->genNotif(remote_agent, msg);
        if (st < 0) data->noteError(st);
        return st;
    }
    data->noteError(NIXL_ERR_BACKEND);
    return NIXL_ERR_BACKEND;
}

// ============================================================ metadata

nixl_status_t nixlAgent::getLocalMD(nixl_blob_t &str) const {
    NIXL_TRACE_SCOPE(data->tracer, METADATA, "getLocalMD");
    return data->mdGetLocal(str);
}

nixl_status_t nixlAgent::getLocalPartialMD(const nixl_reg_dlist_t &descs, nixl_blob_t &str, const nixl_opt_args_t *extra_params) const {
    NIXL_TRACE_SCOPE(data->tracer, METADATA, "getLocalPartialMD");
    return data->mdGetLocalPartial(descs, str, extra_params);
}

nixl_status_t nixlAgent::loadRemoteMD(const nixl_blob_t &remote_metadata, std::string &agent_name) {
    const nixl_status_t st = data->mdLoadRemote(remote_metadata, agent_name);
    data->noteError(st);
    return st;
}

nixl_status_t nixlAgent::invalidateRemoteMD(const std::string &remote_agent) {
    NIXL_TRACE_SCOPE(data->tracer, METADATA, "invalidateRemoteMD");
    return data->mdInvalidateRemote(remote_agent);
}

nixl_status_t nixlAgent::sendLocalMD(const nixl_opt_args_t *extra_params) const { return data->mdManager->sendLocal(extra_params); }

nixl_status_t nixlAgent::sendLocalPartialMD(const nixl_reg_dlist_t &descs, const nixl_opt_args_t *extra_params) const {
    return data->mdManager->sendLocalPartial(descs, extra_params);
}

nixl_status_t nixlAgent::fetchRemoteMD(const std::string remote_name, const nixl_opt_args_t *extra_params) {
    return data->mdManager->fetchRemote(remote_name, extra_params);
}

nixl_status_t nixlAgent::invalidateLocalMD(const nixl_opt_args_t *extra_params) const {
    return data->mdManager->invalidateLocal(extra_params);
}

nixl_status_t nixlAgent::checkRemoteMD(const std::string remote_name, const nixl_xfer_dlist_t &descs) const {
    nixlSharedGuard g(data->lock);
    nixlRemoteSection *rs = data->remoteOf(remote_name);
    if (!rs) {
        // Known by connection info only (partial metadata without registrations yet).
        if (descs.isEmpty() && data->remoteBackends.count(remote_name)) return NIXL_SUCCESS;
        return NIXL_ERR_NOT_FOUND;
    }
    if (descs.isEmpty()) return NIXL_SUCCESS;
    const backend_set_t *have = rs->queryBackends(descs.getType());
    if (!have) return NIXL_ERR_NOT_FOUND;
    for (auto *e : *have) {
        nixl_meta_dlist_t tmp(descs.getType());
        if (rs->populate(descs, e, tmp) == NIXL_SUCCESS) return NIXL_SUCCESS;
    }
    return NIXL_ERR_NOT_FOUND;
}

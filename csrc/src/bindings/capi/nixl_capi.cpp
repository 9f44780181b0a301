// Implementation of the C API (include/nixl_capi.h): thin, exception-safe shims over nixlAgent.
#include "nixl_capi.h"

#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "nixl.h"

struct nixl_capi_agent_s { std::unique_ptr<nixlAgent> inner; };
struct nixl_capi_params_s { nixl_b_params_t params; };
struct nixl_capi_mem_list_s { nixl_mem_list_t mems; };
struct nixl_capi_string_list_s { std::vector<std::string> strings; };
struct nixl_capi_backend_s { nixlBackendH *backend = nullptr; };
struct nixl_capi_opt_args_s { nixl_opt_args_t args; };
struct nixl_capi_param_iter_s { nixl_b_params_t::const_iterator it, end; };
struct nixl_capi_xfer_dlist_s { nixl_xfer_dlist_t list; explicit nixl_capi_xfer_dlist_s(nixl_mem_t m) : list(m) {} };
struct nixl_capi_xfer_dlist_handle_s { nixlDlistH *handle = nullptr; };
struct nixl_capi_reg_dlist_s { nixl_reg_dlist_t list; explicit nixl_capi_reg_dlist_s(nixl_mem_t m) : list(m) {} };
struct nixl_capi_remote_dlist_s { nixl_remote_dlist_t list; explicit nixl_capi_remote_dlist_s(nixl_mem_t m) : list(m) {} };
struct nixl_capi_xfer_req_s { nixlXferReqH *req = nullptr; };
struct nixl_capi_notif_map_s { nixl_notifs_t map; std::vector<std::string> order; };
struct nixl_capi_query_resp_list_s { std::vector<nixl_query_resp_t> items; };
struct nixl_capi_mem_view_s { nixlMemViewH view = nullptr; };

namespace {

// Library status -> C API status.
nixl_capi_status_t conv(nixl_status_t st) {
    switch (st) {
    case NIXL_SUCCESS: return NIXL_CAPI_SUCCESS;
    case NIXL_IN_PROG: return NIXL_CAPI_IN_PROG;
    case NIXL_ERR_INVALID_PARAM: return NIXL_CAPI_ERROR_INVALID_PARAM;
    case NIXL_ERR_NOT_FOUND: return NIXL_CAPI_ERROR_NOT_FOUND;
    case NIXL_ERR_NO_TELEMETRY: return NIXL_CAPI_ERROR_NO_TELEMETRY;
    case NIXL_ERR_NOT_POSTED:
    case NIXL_ERR_REPOST_ACTIVE:
    case NIXL_ERR_NOT_ALLOWED: return NIXL_CAPI_ERROR_INVALID_STATE;
    default: return NIXL_CAPI_ERROR_BACKEND;
    }
}

template<class F> nixl_capi_status_t guarded(F &&f) {
    try {
        return f();
    } catch (...) {
        return NIXL_CAPI_ERROR_EXCEPTION;
    }
}

const nixl_opt_args_t *opt(nixl_capi_opt_args_t a) { return a ? &a->args : nullptr; }

nixl_capi_status_t blobOut(const std::string &blob, void **data, size_t *len) {
    void *p = std::malloc(blob.size() ? blob.size() : 1);
    if (!p) return NIXL_CAPI_ERROR_EXCEPTION;
    std::memcpy(p, blob.data(), blob.size());
    *data = p;
    *len = blob.size();
    return NIXL_CAPI_SUCCESS;
}

#define REQUIRE(cond) \
    if (!(cond)) return NIXL_CAPI_ERROR_INVALID_PARAM

} // namespace

extern "C" {

bool nixl_capi_is_stub(void) { return false; }

// ------------------------------------------------------------------ agent

nixl_capi_status_t nixl_capi_create_configured_agent(const char *name, const nixl_capi_agent_config_t *cfg, nixl_capi_agent_t *agent) {
    REQUIRE(name && cfg && agent);
    return guarded([&] {
        nixlAgentConfig c(cfg->enable_prog_thread, cfg->enable_listen_thread, static_cast<uint16_t>(cfg->listen_port),
                          static_cast<nixl_thread_sync_t>(cfg->thread_sync), cfg->num_workers, cfg->pthr_delay_us, cfg->lthr_delay_us,
                          cfg->capture_telemetry);
        auto a = new nixl_capi_agent_s{std::make_unique<nixlAgent>(name, c)};
        *agent = a;
        return NIXL_CAPI_SUCCESS;
    });
}

nixl_capi_status_t nixl_capi_create_agent(const char *name, nixl_capi_agent_t *agent) {
    // Default configuration of the FFI layer: progress thread on, listener off.
    nixl_capi_agent_config_t cfg = {true, false, 0, NIXL_CAPI_THREAD_SYNC_DEFAULT, 1, 0, 100000, false};
    return nixl_capi_create_configured_agent(name, &cfg, agent);
}

nixl_capi_status_t nixl_capi_destroy_agent(nixl_capi_agent_t agent) {
    REQUIRE(agent);
    return guarded([&] {
        delete agent;
        return NIXL_CAPI_SUCCESS;
    });
}

// ------------------------------------------------------------------ metadata

nixl_capi_status_t nixl_capi_get_local_md(nixl_capi_agent_t agent, void **data, size_t *len) {
    REQUIRE(agent && data && len);
    return guarded([&] {
        nixl_blob_t md;
        const nixl_status_t st = agent->inner->getLocalMD(md);
        return st == NIXL_SUCCESS ? blobOut(md, data, len) : conv(st);
    });
}

nixl_capi_status_t nixl_capi_get_local_partial_md(nixl_capi_agent_t agent, nixl_capi_reg_dlist_t descs, void **data, size_t *len,
                                                  nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && descs && data && len);
    return guarded([&] {
        nixl_blob_t md;
        const nixl_status_t st = agent->inner->getLocalPartialMD(descs->list, md, opt(opt_args));
        return st == NIXL_SUCCESS ? blobOut(md, data, len) : conv(st);
    });
}

nixl_capi_status_t nixl_capi_load_remote_md(nixl_capi_agent_t agent, const void *data, size_t len, char **agent_name) {
    REQUIRE(agent && data && len && agent_name);
    return guarded([&] {
        std::string name;
        const nixl_status_t st = agent->inner->loadRemoteMD(nixl_blob_t(static_cast<const char *>(data), len), name);
        if (st != NIXL_SUCCESS) return conv(st);
        *agent_name = ::strdup(name.c_str());
        return *agent_name ? NIXL_CAPI_SUCCESS : NIXL_CAPI_ERROR_EXCEPTION;
    });
}

nixl_capi_status_t nixl_capi_invalidate_remote_md(nixl_capi_agent_t agent, const char *remote_agent) {
    REQUIRE(agent && remote_agent);
    return guarded([&] { return conv(agent->inner->invalidateRemoteMD(remote_agent)); });
}

nixl_capi_status_t nixl_capi_invalidate_local_md(nixl_capi_agent_t agent, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent);
    return guarded([&] { return conv(agent->inner->invalidateLocalMD(opt(opt_args))); });
}

nixl_capi_status_t nixl_capi_check_remote_md(nixl_capi_agent_t agent, const char *remote_name, nixl_capi_xfer_dlist_t descs) {
    REQUIRE(agent && remote_name);
    return guarded([&] {
        nixl_xfer_dlist_t empty(DRAM_SEG);
        return conv(agent->inner->checkRemoteMD(remote_name, descs ? descs->list : empty));
    });
}

nixl_capi_status_t nixl_capi_send_local_md(nixl_capi_agent_t agent, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent);
    return guarded([&] { return conv(agent->inner->sendLocalMD(opt(opt_args))); });
}

nixl_capi_status_t nixl_capi_send_local_partial_md(nixl_capi_agent_t agent, nixl_capi_reg_dlist_t descs, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && descs);
    return guarded([&] { return conv(agent->inner->sendLocalPartialMD(descs->list, opt(opt_args))); });
}

nixl_capi_status_t nixl_capi_fetch_remote_md(nixl_capi_agent_t agent, const char *remote_name, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && remote_name);
    return guarded([&] { return conv(agent->inner->fetchRemoteMD(remote_name, opt(opt_args))); });
}

// ------------------------------------------------------------------ plugins / backends

nixl_capi_status_t nixl_capi_get_available_plugins(nixl_capi_agent_t agent, nixl_capi_string_list_t *plugins) {
    REQUIRE(agent && plugins);
    return guarded([&] {
        std::vector<nixl_backend_t> names;
        const nixl_status_t st = agent->inner->getAvailPlugins(names);
        if (st != NIXL_SUCCESS) return conv(st);
        *plugins = new nixl_capi_string_list_s{std::move(names)};
        return NIXL_CAPI_SUCCESS;
    });
}

nixl_capi_status_t nixl_capi_get_plugin_params(nixl_capi_agent_t agent, const char *plugin_name, nixl_capi_mem_list_t *mems,
                                               nixl_capi_params_t *params) {
    REQUIRE(agent && plugin_name && mems && params);
    return guarded([&] {
        auto m = std::make_unique<nixl_capi_mem_list_s>();
        auto p = std::make_unique<nixl_capi_params_s>();
        const nixl_status_t st = agent->inner->getPluginParams(plugin_name, m->mems, p->params);
        if (st != NIXL_SUCCESS) return conv(st);
        *mems = m.release();
        *params = p.release();
        return NIXL_CAPI_SUCCESS;
    });
}

nixl_capi_status_t nixl_capi_create_backend(nixl_capi_agent_t agent, const char *plugin_name, nixl_capi_params_t params,
                                            nixl_capi_backend_t *backend) {
    REQUIRE(agent && plugin_name && backend);
    return guarded([&] {
        nixlBackendH *h = nullptr;
        const nixl_status_t st = agent->inner->createBackend(plugin_name, params ? params->params : nixl_b_params_t(), h);
        if (st != NIXL_SUCCESS) return conv(st);
        *backend = new nixl_capi_backend_s{h};
        return NIXL_CAPI_SUCCESS;
    });
}

nixl_capi_status_t nixl_capi_destroy_backend(nixl_capi_backend_t backend) {
    REQUIRE(backend);
    delete backend; // the engine itself belongs to the agent
    return NIXL_CAPI_SUCCESS;
}

nixl_capi_status_t nixl_capi_get_backend_params(nixl_capi_agent_t agent, nixl_capi_backend_t backend, nixl_capi_mem_list_t *mems,
                                                nixl_capi_params_t *params) {
    REQUIRE(agent && backend && mems && params);
    return guarded([&] {
        auto m = std::make_unique<nixl_capi_mem_list_s>();
        auto p = std::make_unique<nixl_capi_params_s>();
        const nixl_status_t st = agent->inner->getBackendParams(backend->backend, m->mems, p->params);
        if (st != NIXL_SUCCESS) return conv(st);
        *mems = m.release();
        *params = p.release();
        return NIXL_CAPI_SUCCESS;
    });
}

// ------------------------------------------------------------------ containers

nixl_capi_status_t nixl_capi_destroy_string_list(nixl_capi_string_list_t list) {
    REQUIRE(list);
    delete list;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_string_list_size(nixl_capi_string_list_t list, size_t *size) {
    REQUIRE(list && size);
    *size = list->strings.size();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_string_list_get(nixl_capi_string_list_t list, size_t index, const char **str) {
    REQUIRE(list && str && index < list->strings.size());
    *str = list->strings[index].c_str();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_destroy_mem_list(nixl_capi_mem_list_t list) {
    REQUIRE(list);
    delete list;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_mem_list_is_empty(nixl_capi_mem_list_t list, bool *is_empty) {
    REQUIRE(list && is_empty);
    *is_empty = list->mems.empty();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_mem_list_size(nixl_capi_mem_list_t list, size_t *size) {
    REQUIRE(list && size);
    *size = list->mems.size();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_mem_list_get(nixl_capi_mem_list_t list, size_t index, nixl_capi_mem_type_t *mem_type) {
    REQUIRE(list && mem_type && index < list->mems.size());
    *mem_type = static_cast<nixl_capi_mem_type_t>(list->mems[index]);
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_mem_type_to_string(nixl_capi_mem_type_t mem_type, const char **str) {
    REQUIRE(str);
    static const char *names[] = {"DRAM_SEG", "VRAM_SEG", "BLK_SEG", "OBJ_SEG", "FILE_SEG", "UNKNOWN"};
    REQUIRE(mem_type >= NIXL_CAPI_MEM_DRAM && mem_type <= NIXL_CAPI_MEM_UNKNOWN);
    *str = names[mem_type];
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_create_params(nixl_capi_params_t *params) {
    REQUIRE(params);
    *params = new nixl_capi_params_s();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_destroy_params(nixl_capi_params_t params) {
    REQUIRE(params);
    delete params;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_params_add(nixl_capi_params_t params, const char *key, const char *value) {
    REQUIRE(params && key && value);
    params->params[key] = value;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_params_is_empty(nixl_capi_params_t params, bool *is_empty) {
    REQUIRE(params && is_empty);
    *is_empty = params->params.empty();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_params_create_iterator(nixl_capi_params_t params, nixl_capi_param_iter_t *iter) {
    REQUIRE(params && iter);
    *iter = new nixl_capi_param_iter_s{params->params.cbegin(), params->params.cend()};
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_params_iterator_next(nixl_capi_param_iter_t iter, const char **key, const char **value, bool *has_next) {
    REQUIRE(iter && key && value && has_next);
    if (iter->it == iter->end) {
        *has_next = false;
        return NIXL_CAPI_ERROR_INVALID_PARAM;
    }
    *key = iter->it->first.c_str();
    *value = iter->it->second.c_str();
    ++iter->it;
    *has_next = iter->it != iter->end;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_params_destroy_iterator(nixl_capi_param_iter_t iter) {
    REQUIRE(iter);
    delete iter;
    return NIXL_CAPI_SUCCESS;
}

// ------------------------------------------------------------------ optional arguments

nixl_capi_status_t nixl_capi_create_opt_args(nixl_capi_opt_args_t *args) {
    REQUIRE(args);
    *args = new nixl_capi_opt_args_s();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_destroy_opt_args(nixl_capi_opt_args_t args) {
    REQUIRE(args);
    delete args;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_opt_args_add_backend(nixl_capi_opt_args_t args, nixl_capi_backend_t backend) {
    REQUIRE(args && backend);
    args->args.backends.push_back(backend->backend);
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_opt_args_set_notif_msg(nixl_capi_opt_args_t args, const void *data, size_t len) {
    REQUIRE(args && (data || len == 0));
    args->args.notifMsg.assign(static_cast<const char *>(data), len);
    args->args.notif = args->args.notifMsg;
    args->args.hasNotif = true;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_opt_args_get_notif_msg(nixl_capi_opt_args_t args, void **data, size_t *len) {
    REQUIRE(args && data && len);
    return blobOut(args->args.notifMsg, data, len);
}
nixl_capi_status_t nixl_capi_opt_args_set_has_notif(nixl_capi_opt_args_t args, bool has_notif) {
    REQUIRE(args);
    args->args.hasNotif = has_notif;
    if (has_notif) args->args.notif = args->args.notifMsg;
    else args->args.notif.reset();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_opt_args_get_has_notif(nixl_capi_opt_args_t args, bool *has_notif) {
    REQUIRE(args && has_notif);
    *has_notif = args->args.hasNotif;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_opt_args_set_skip_desc_merge(nixl_capi_opt_args_t args, bool skip_merge) {
    REQUIRE(args);
    args->args.skipDescMerge = skip_merge;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_opt_args_get_skip_desc_merge(nixl_capi_opt_args_t args, bool *skip_merge) {
    REQUIRE(args && skip_merge);
    *skip_merge = args->args.skipDescMerge;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_opt_args_set_ip_addr(nixl_capi_opt_args_t args, const char *ip_addr) {
    REQUIRE(args && ip_addr);
    args->args.ipAddr = ip_addr;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_opt_args_set_port(nixl_capi_opt_args_t args, uint16_t port) {
    REQUIRE(args);
    args->args.port = port;
    return NIXL_CAPI_SUCCESS;
}

// ------------------------------------------------------------------ memory

nixl_capi_status_t nixl_capi_register_mem(nixl_capi_agent_t agent, nixl_capi_reg_dlist_t dlist, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && dlist);
    return guarded([&] { return conv(agent->inner->registerMem(dlist->list, opt(opt_args))); });
}
nixl_capi_status_t nixl_capi_deregister_mem(nixl_capi_agent_t agent, nixl_capi_reg_dlist_t dlist, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && dlist);
    return guarded([&] { return conv(agent->inner->deregisterMem(dlist->list, opt(opt_args))); });
}
nixl_capi_status_t nixl_capi_agent_make_connection(nixl_capi_agent_t agent, const char *remote_agent, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && remote_agent);
    return guarded([&] { return conv(agent->inner->makeConnection(remote_agent, opt(opt_args))); });
}
nixl_capi_status_t nixl_capi_create_query_resp_list(nixl_capi_query_resp_list_t *list) {
    REQUIRE(list);
    *list = new nixl_capi_query_resp_list_s();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_destroy_query_resp_list(nixl_capi_query_resp_list_t list) {
    REQUIRE(list);
    delete list;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_query_resp_list_size(nixl_capi_query_resp_list_t list, size_t *size) {
    REQUIRE(list && size);
    *size = list->items.size();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_query_resp_list_has_value(nixl_capi_query_resp_list_t list, size_t index, bool *has_value) {
    REQUIRE(list && has_value && index < list->items.size());
    *has_value = list->items[index].has_value();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_query_resp_list_get_params(nixl_capi_query_resp_list_t list, size_t index, nixl_capi_params_t *params) {
    REQUIRE(list && params && index < list->items.size() && list->items[index].has_value());
    *params = new nixl_capi_params_s{*list->items[index]};
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_query_mem(nixl_capi_agent_t agent, nixl_capi_reg_dlist_t descs, nixl_capi_query_resp_list_t resp,
                                       nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && descs && resp);
    return guarded([&] { return conv(agent->inner->queryMem(descs->list, resp->items, opt(opt_args))); });
}

// ------------------------------------------------------------------ transfers

nixl_capi_status_t nixl_capi_prep_xfer_dlist(nixl_capi_agent_t agent, const char *agent_name, nixl_capi_xfer_dlist_t descs,
                                             nixl_capi_xfer_dlist_handle_t *dlist_hndl, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && agent_name && descs && dlist_hndl);
    return guarded([&] {
        nixlDlistH *h = nullptr;
        const nixl_status_t st = agent->inner->prepXferDlist(agent_name, descs->list, h, opt(opt_args));
        if (st != NIXL_SUCCESS) return conv(st);
        *dlist_hndl = new nixl_capi_xfer_dlist_handle_s{h};
        return NIXL_CAPI_SUCCESS;
    });
}
nixl_capi_status_t nixl_capi_release_xfer_dlist_handle(nixl_capi_agent_t agent, nixl_capi_xfer_dlist_handle_t dlist_handle) {
    REQUIRE(agent && dlist_handle);
    return guarded([&] {
        const nixl_status_t st = agent->inner->releasedDlistH(dlist_handle->handle);
        delete dlist_handle;
        return conv(st);
    });
}
nixl_capi_status_t nixl_capi_make_xfer_req(nixl_capi_agent_t agent, nixl_capi_xfer_op_t operation, nixl_capi_xfer_dlist_handle_t local_descs,
                                           const int *local_indices, size_t local_indices_count,
                                           nixl_capi_xfer_dlist_handle_t remote_descs, const int *remote_indices,
                                           size_t remote_indices_count, nixl_capi_xfer_req_t *req_hndl, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && local_descs && remote_descs && local_indices && remote_indices && req_hndl);
    return guarded([&] {
        const std::vector<int> li(local_indices, local_indices + local_indices_count), ri(remote_indices, remote_indices + remote_indices_count);
        nixlXferReqH *req = nullptr;
        const nixl_status_t st = agent->inner->makeXferReq(static_cast<nixl_xfer_op_t>(operation), local_descs->handle, li,
                                                           remote_descs->handle, ri, req, opt(opt_args));
        if (st != NIXL_SUCCESS) return conv(st);
        *req_hndl = new nixl_capi_xfer_req_s{req};
        return NIXL_CAPI_SUCCESS;
    });
}
nixl_capi_status_t nixl_capi_create_xfer_req(nixl_capi_agent_t agent, nixl_capi_xfer_op_t operation, nixl_capi_xfer_dlist_t local_descs,
                                             nixl_capi_xfer_dlist_t remote_descs, const char *remote_agent, nixl_capi_xfer_req_t *req_hndl,
                                             nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && local_descs && remote_descs && remote_agent && req_hndl);
    return guarded([&] {
        nixlXferReqH *req = nullptr;
        const nixl_status_t st = agent->inner->createXferReq(static_cast<nixl_xfer_op_t>(operation), local_descs->list, remote_descs->list,
                                                             remote_agent, req, opt(opt_args));
        if (st != NIXL_SUCCESS) return conv(st);
        *req_hndl = new nixl_capi_xfer_req_s{req};
        return NIXL_CAPI_SUCCESS;
    });
}
nixl_capi_status_t nixl_capi_estimate_xfer_cost(nixl_capi_agent_t agent, nixl_capi_xfer_req_t req_hndl, nixl_capi_opt_args_t opt_args,
                                                int64_t *duration_us, int64_t *err_margin_us, nixl_capi_cost_t *method) {
    REQUIRE(agent && req_hndl && duration_us && err_margin_us && method);
    return guarded([&] {
        std::chrono::microseconds d{0}, e{0};
        nixl_cost_t m = nixl_cost_t::ANALYTICAL_BACKEND;
        const nixl_status_t st = agent->inner->estimateXferCost(req_hndl->req, d, e, m, opt(opt_args));
        if (st != NIXL_SUCCESS) return conv(st);
        *duration_us = d.count();
        *err_margin_us = e.count();
        *method = static_cast<nixl_capi_cost_t>(m);
        return NIXL_CAPI_SUCCESS;
    });
}
nixl_capi_status_t nixl_capi_post_xfer_req(nixl_capi_agent_t agent, nixl_capi_xfer_req_t req_hndl, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && req_hndl);
    return guarded([&] { return conv(agent->inner->postXferReq(req_hndl->req, opt(opt_args))); });
}
nixl_capi_status_t nixl_capi_get_xfer_status(nixl_capi_agent_t agent, nixl_capi_xfer_req_t req_hndl) {
    REQUIRE(agent && req_hndl);
    return guarded([&] { return conv(agent->inner->getXferStatus(req_hndl->req)); });
}
nixl_capi_status_t nixl_capi_query_xfer_backend(nixl_capi_agent_t agent, nixl_capi_xfer_req_t req_hndl, nixl_capi_backend_t *backend) {
    REQUIRE(agent && req_hndl && backend);
    return guarded([&] {
        nixlBackendH *h = nullptr;
        const nixl_status_t st = agent->inner->queryXferBackend(req_hndl->req, h);
        if (st != NIXL_SUCCESS) return conv(st);
        *backend = new nixl_capi_backend_s{h};
        return NIXL_CAPI_SUCCESS;
    });
}
nixl_capi_status_t nixl_capi_release_xfer_req(nixl_capi_agent_t agent, nixl_capi_xfer_req_t req) {
    REQUIRE(agent && req);
    return guarded([&] {
        const nixl_status_t st = agent->inner->releaseXferReq(req->req);
        if (st == NIXL_SUCCESS) req->req = nullptr;
        return conv(st);
    });
}
nixl_capi_status_t nixl_capi_destroy_xfer_req(nixl_capi_xfer_req_t req) {
    REQUIRE(req);
    delete req; // the wrapper only; release_xfer_req frees the request itself
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_get_xfer_telemetry(nixl_capi_agent_t agent, nixl_capi_xfer_req_t req_hndl, nixl_capi_xfer_telemetry_t telemetry) {
    REQUIRE(agent && req_hndl && telemetry);
    return guarded([&] {
        nixl_xfer_telem_t t;
        const nixl_status_t st = agent->inner->getXferTelemetry(req_hndl->req, t);
        if (st != NIXL_SUCCESS) return conv(st);
        telemetry->start_time_us =
            static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::microseconds>(t.startTime.time_since_epoch()).count());
        telemetry->post_duration_us = static_cast<uint64_t>(t.postDuration.count());
        telemetry->xfer_duration_us = static_cast<uint64_t>(t.xferDuration.count());
        telemetry->total_bytes = t.totalBytes;
        telemetry->desc_count = t.descCount;
        return NIXL_CAPI_SUCCESS;
    });
}

// ------------------------------------------------------------------ notifications

nixl_capi_status_t nixl_capi_create_notif_map(nixl_capi_notif_map_t *notif_map) {
    REQUIRE(notif_map);
    *notif_map = new nixl_capi_notif_map_s();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_destroy_notif_map(nixl_capi_notif_map_t notif_map) {
    REQUIRE(notif_map);
    delete notif_map;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_get_notifs(nixl_capi_agent_t agent, nixl_capi_notif_map_t notif_map, nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && notif_map);
    return guarded([&] {
        const nixl_status_t st = agent->inner->getNotifs(notif_map->map, opt(opt_args));
        notif_map->order.clear();
        for (auto &kv : notif_map->map) notif_map->order.push_back(kv.first);
        return conv(st);
    });
}
nixl_capi_status_t nixl_capi_gen_notif(nixl_capi_agent_t agent, const char *remote_agent, const void *data, size_t len,
                                       nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && remote_agent && (data || len == 0));
    return guarded([&] { return conv(agent->inner->genNotif(remote_agent, nixl_blob_t(static_cast<const char *>(data), len), opt(opt_args))); });
}
nixl_capi_status_t nixl_capi_notif_map_size(nixl_capi_notif_map_t map, size_t *size) {
    REQUIRE(map && size);
    *size = map->map.size();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_notif_map_get_agent_at(nixl_capi_notif_map_t map, size_t index, const char **agent_name) {
    REQUIRE(map && agent_name && index < map->order.size());
    *agent_name = map->order[index].c_str();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_notif_map_get_notifs_size(nixl_capi_notif_map_t map, const char *agent_name, size_t *size) {
    REQUIRE(map && agent_name && size);
    auto it = map->map.find(agent_name);
    REQUIRE(it != map->map.end());
    *size = it->second.size();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_notif_map_get_notif(nixl_capi_notif_map_t map, const char *agent_name, size_t index, const void **data,
                                                 size_t *len) {
    REQUIRE(map && agent_name && data && len);
    auto it = map->map.find(agent_name);
    REQUIRE(it != map->map.end() && index < it->second.size());
    *data = it->second[index].data();
    *len = it->second[index].size();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_notif_map_clear(nixl_capi_notif_map_t map) {
    REQUIRE(map);
    map->map.clear();
    map->order.clear();
    return NIXL_CAPI_SUCCESS;
}

// ------------------------------------------------------------------ descriptor lists

#define DLIST_COMMON(prefix, type_t)                                                                                       \
    nixl_capi_status_t nixl_capi_destroy_##prefix(type_t dlist) {                                                         \
        REQUIRE(dlist);                                                                                                    \
        delete dlist;                                                                                                      \
        return NIXL_CAPI_SUCCESS;                                                                                          \
    }                                                                                                                      \
    nixl_capi_status_t nixl_capi_##prefix##_get_type(type_t dlist, nixl_capi_mem_type_t *mem_type) {                      \
        REQUIRE(dlist && mem_type);                                                                                        \
        *mem_type = static_cast<nixl_capi_mem_type_t>(dlist->list.getType());                                             \
        return NIXL_CAPI_SUCCESS;                                                                                          \
    }                                                                                                                      \
    nixl_capi_status_t nixl_capi_##prefix##_desc_count(type_t dlist, size_t *count) {                                     \
        REQUIRE(dlist && count);                                                                                           \
        *count = static_cast<size_t>(dlist->list.descCount());                                                            \
        return NIXL_CAPI_SUCCESS;                                                                                          \
    }                                                                                                                      \
    nixl_capi_status_t nixl_capi_##prefix##_is_empty(type_t dlist, bool *is_empty) {                                      \
        REQUIRE(dlist && is_empty);                                                                                        \
        *is_empty = dlist->list.isEmpty();                                                                                 \
        return NIXL_CAPI_SUCCESS;                                                                                          \
    }                                                                                                                      \
    nixl_capi_status_t nixl_capi_##prefix##_trim(type_t dlist) {                                                          \
        REQUIRE(dlist);                                                                                                    \
        return NIXL_CAPI_SUCCESS; /* lists carry no spare capacity worth trimming */                                      \
    }                                                                                                                      \
    nixl_capi_status_t nixl_capi_##prefix##_rem_desc(type_t dlist, int index) {                                           \
        REQUIRE(dlist && index >= 0 && index < dlist->list.descCount());                                                  \
        dlist->list.remDesc(index);                                                                                        \
        return NIXL_CAPI_SUCCESS;                                                                                          \
    }                                                                                                                      \
    nixl_capi_status_t nixl_capi_##prefix##_clear(type_t dlist) {                                                         \
        REQUIRE(dlist);                                                                                                    \
        dlist->list.clear();                                                                                               \
        return NIXL_CAPI_SUCCESS;                                                                                          \
    }                                                                                                                      \
    nixl_capi_status_t nixl_capi_##prefix##_resize(type_t dlist, size_t new_size) {                                       \
        REQUIRE(dlist);                                                                                                    \
        dlist->list.resize(new_size);                                                                                      \
        return NIXL_CAPI_SUCCESS;                                                                                          \
    }                                                                                                                      \
    nixl_capi_status_t nixl_capi_##prefix##_print(type_t dlist) {                                                         \
        REQUIRE(dlist);                                                                                                    \
        dlist->list.print();                                                                                               \
        return NIXL_CAPI_SUCCESS;                                                                                          \
    }

DLIST_COMMON(xfer_dlist, nixl_capi_xfer_dlist_t)
DLIST_COMMON(reg_dlist, nixl_capi_reg_dlist_t)

nixl_capi_status_t nixl_capi_create_xfer_dlist(nixl_capi_mem_type_t mem_type, nixl_capi_xfer_dlist_t *dlist) {
    REQUIRE(dlist && mem_type >= NIXL_CAPI_MEM_DRAM && mem_type <= NIXL_CAPI_MEM_FILE);
    *dlist = new nixl_capi_xfer_dlist_s(static_cast<nixl_mem_t>(mem_type));
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_xfer_dlist_add_desc(nixl_capi_xfer_dlist_t dlist, uintptr_t addr, size_t len, uint64_t dev_id) {
    REQUIRE(dlist);
    dlist->list.addDesc(nixlBasicDesc(addr, len, dev_id));
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_xfer_dlist_len(nixl_capi_xfer_dlist_t dlist, size_t *len) {
    REQUIRE(dlist && len);
    *len = dlist->list.totalBytes();
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_create_reg_dlist(nixl_capi_mem_type_t mem_type, nixl_capi_reg_dlist_t *dlist) {
    REQUIRE(dlist && mem_type >= NIXL_CAPI_MEM_DRAM && mem_type <= NIXL_CAPI_MEM_FILE);
    *dlist = new nixl_capi_reg_dlist_s(static_cast<nixl_mem_t>(mem_type));
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_reg_dlist_add_desc(nixl_capi_reg_dlist_t dlist, uintptr_t addr, size_t len, uint64_t dev_id,
                                                const void *metadata, size_t metadata_len) {
    REQUIRE(dlist && (metadata || metadata_len == 0));
    dlist->list.addDesc(nixlBlobDesc(addr, len, dev_id, nixl_blob_t(static_cast<const char *>(metadata), metadata_len)));
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_create_remote_dlist(nixl_capi_mem_type_t mem_type, nixl_capi_remote_dlist_t *dlist) {
    REQUIRE(dlist && mem_type >= NIXL_CAPI_MEM_DRAM && mem_type <= NIXL_CAPI_MEM_FILE);
    *dlist = new nixl_capi_remote_dlist_s(static_cast<nixl_mem_t>(mem_type));
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_destroy_remote_dlist(nixl_capi_remote_dlist_t dlist) {
    REQUIRE(dlist);
    delete dlist;
    return NIXL_CAPI_SUCCESS;
}
nixl_capi_status_t nixl_capi_remote_dlist_add_desc(nixl_capi_remote_dlist_t dlist, uintptr_t addr, size_t len, uint64_t dev_id,
                                                   const char *remote_agent) {
    REQUIRE(dlist && remote_agent);
    dlist->list.addDesc(nixlRemoteDesc(addr, len, dev_id, remote_agent));
    return NIXL_CAPI_SUCCESS;
}

// ------------------------------------------------------------------ memory views

nixl_capi_status_t nixl_capi_prep_mem_view_local(nixl_capi_agent_t agent, nixl_capi_xfer_dlist_t descs, nixl_capi_mem_view_t *mvh,
                                                 nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && descs && mvh);
    return guarded([&] {
        nixlMemViewH v = nullptr;
        const nixl_status_t st = agent->inner->prepMemView(descs->list, v, opt(opt_args));
        if (st != NIXL_SUCCESS) return conv(st);
        *mvh = new nixl_capi_mem_view_s{v};
        return NIXL_CAPI_SUCCESS;
    });
}
nixl_capi_status_t nixl_capi_prep_mem_view_remote(nixl_capi_agent_t agent, nixl_capi_remote_dlist_t descs, nixl_capi_mem_view_t *mvh,
                                                  nixl_capi_opt_args_t opt_args) {
    REQUIRE(agent && descs && mvh);
    return guarded([&] {
        nixlMemViewH v = nullptr;
        const nixl_status_t st = agent->inner->prepMemView(descs->list, v, opt(opt_args));
        if (st != NIXL_SUCCESS) return conv(st);
        *mvh = new nixl_capi_mem_view_s{v};
        return NIXL_CAPI_SUCCESS;
    });
}
nixl_capi_status_t nixl_capi_release_mem_view(nixl_capi_agent_t agent, nixl_capi_mem_view_t mvh) {
    REQUIRE(agent && mvh);
    return guarded([&] {
        agent->inner->releaseMemView(mvh->view);
        delete mvh;
        return NIXL_CAPI_SUCCESS;
    });
}

} // extern "C"

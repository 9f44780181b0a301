// pybind11 module `nixl_b200._bindings`: thin, typed access to the C++ agent.
//
// Surface parity with the reference's src/bindings/python/nixl_bindings.cpp: memory-type,
// operation, status and sync-mode constants; one exception class per error status;
// descriptor lists built from tuple lists or N x 3 numpy arrays (and picklable);
// nixlAgentConfig; every nixlAgent method; opaque handles travel as integers.
// The user-facing wrapper (nixl_agent) lives in nixl_b200/_api.py.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <tuple>

#include "core/agent_data.h"
#include "core/plugin_manager.h"
#include "nixl.h"
#include "utils/topology.h"
#include "serdes/serdes.h"

namespace py = pybind11;

namespace {

struct ErrorTypes {
    py::object base;
    py::object byStatus[13]; // index = -status
};
ErrorTypes *g_err = nullptr;

// Raises the exception class that belongs to `st` (no-op for SUCCESS / IN_PROG).
void throwIf(nixl_status_t st, const char *what) {
    if (st >= 0) return;
    const int idx = -static_cast<int>(st);
    py::object cls = (idx >= 1 && idx <= 12) ? g_err->byStatus[idx] : g_err->base;
    const std::string msg = std::string(what) + ": " + nixlEnumStrings::statusStr(st);
    PyErr_SetString(cls.ptr(), msg.c_str());
    throw py::error_already_set();
}

template<class H> H *asHandle(uintptr_t v) { return reinterpret_cast<H *>(v); }

using xfer_tuple = std::tuple<uintptr_t, size_t, uint64_t>;
using reg_tuple = std::tuple<uintptr_t, size_t, uint64_t, std::string>;

// Accepts None, a list of tuples, or an (N,3) uint64 array.
void fillXfer(nixl_xfer_dlist_t &l, const py::object &descs) {
    if (descs.is_none()) return;
    if (py::isinstance<py::array>(descs)) {
        auto arr = py::array_t<uint64_t, py::array::c_style | py::array::forcecast>::ensure(descs);
        if (!arr || arr.ndim() != 2 || arr.shape(1) != 3) throw py::value_error("descriptor array must have shape (N, 3)");
        const ssize_t n = arr.shape(0);
        l.resize(static_cast<size_t>(n));
        // Rows are {addr, len, devId}: the exact layout of nixlBasicDesc.
        if (n) std::memcpy(static_cast<void *>(&l[0]), arr.data(), static_cast<size_t>(n) * sizeof(nixlBasicDesc));
        return;
    }
    for (auto item : descs) {
        auto t = item.cast<xfer_tuple>();
        l.addDesc(nixlBasicDesc(std::get<0>(t), std::get<1>(t), std::get<2>(t)));
    }
}

nixl_opt_args_t makeOpt(const std::vector<uintptr_t> &backends, const py::object &notif = py::none()) {
    nixl_opt_args_t o;
    for (auto b : backends) o.backends.push_back(asHandle<nixlBackendH>(b));
    if (!notif.is_none()) o.notif = notif.cast<std::string>();
    return o;
}

py::dict paramsToDict(const nixl_b_params_t &p) {
    py::dict d;
    for (auto &kv : p) d[py::str(kv.first)] = py::str(kv.second);
    return d;
}

} // namespace

PYBIND11_MODULE(_bindings, m) {
    m.doc() = "Native bindings of the B200 transfer library (NIXL-compatible API)";

    // Plug-in search path of the process (the manager is a singleton shared by all agents).
    m.def("add_plugin_directory", [](const std::string &dir) { nixlPluginManager::getInstance().addPluginDirectory(dir); });
    // The host's GPUs and network devices from the PCI sysfs tree, and for every GPU the interfaces nearest to it.
    m.def(
        "pci_topology",
        [](const std::string &root) {
            const nixl::pciTopology t = nixl::pciTopology::scan(root);
            auto dev = [](const nixl::pciDevice &d) {
                py::dict o;
                o["bdf"] = d.bdf;
                o["numa_node"] = d.numaNode;
                o["chain"] = d.chain;
                o["vendor"] = d.vendor;
                o["device"] = d.device;
                o["interfaces"] = d.netInterfaces;
                return o;
            };
            py::dict out;
            py::list gpus, nics, near;
            for (const auto &g : t.gpus()) gpus.append(dev(g));
            for (const auto &n : t.nics()) nics.append(dev(n));
            for (size_t g = 0; g < t.gpus().size(); ++g) {
                py::list row;
                for (const nixl::pciDevice *n : t.nicsNearGpu(g)) {
                    py::dict e;
                    e["bdf"] = n->bdf;
                    e["interfaces"] = n->netInterfaces;
                    e["distance"] = nixl::pciTopology::distance(t.gpus()[g], *n);
                    row.append(e);
                }
                near.append(row);
            }
            out["gpus"] = gpus;
            out["nics"] = nics;
            out["nics_near_gpu"] = near;
            out["text"] = t.toString();
            return out;
        },
        py::arg("root") = "");
    m.def("get_plugin_directories", [] { return nixlPluginManager::getInstance().getPluginDirectories(); });

    m.attr("DRAM_SEG") = static_cast<int>(DRAM_SEG);
    m.attr("VRAM_SEG") = static_cast<int>(VRAM_SEG);
    m.attr("BLK_SEG") = static_cast<int>(BLK_SEG);
    m.attr("OBJ_SEG") = static_cast<int>(OBJ_SEG);
    m.attr("FILE_SEG") = static_cast<int>(FILE_SEG);
    m.attr("NIXL_READ") = static_cast<int>(NIXL_READ);
    m.attr("NIXL_WRITE") = static_cast<int>(NIXL_WRITE);
    m.attr("NIXL_IN_PROG") = static_cast<int>(NIXL_IN_PROG);
    m.attr("NIXL_SUCCESS") = static_cast<int>(NIXL_SUCCESS);
    m.attr("NIXL_ERR_NOT_POSTED") = static_cast<int>(NIXL_ERR_NOT_POSTED);
    m.attr("NIXL_ERR_INVALID_PARAM") = static_cast<int>(NIXL_ERR_INVALID_PARAM);
    m.attr("NIXL_ERR_BACKEND") = static_cast<int>(NIXL_ERR_BACKEND);
    m.attr("NIXL_ERR_NOT_FOUND") = static_cast<int>(NIXL_ERR_NOT_FOUND);
    m.attr("NIXL_ERR_MISMATCH") = static_cast<int>(NIXL_ERR_MISMATCH);
    m.attr("NIXL_ERR_NOT_ALLOWED") = static_cast<int>(NIXL_ERR_NOT_ALLOWED);
    m.attr("NIXL_ERR_REPOST_ACTIVE") = static_cast<int>(NIXL_ERR_REPOST_ACTIVE);
    m.attr("NIXL_ERR_UNKNOWN") = static_cast<int>(NIXL_ERR_UNKNOWN);
    m.attr("NIXL_ERR_NOT_SUPPORTED") = static_cast<int>(NIXL_ERR_NOT_SUPPORTED);
    m.attr("NIXL_ERR_REMOTE_DISCONNECT") = static_cast<int>(NIXL_ERR_REMOTE_DISCONNECT);
    m.attr("NIXL_ERR_CANCELED") = static_cast<int>(NIXL_ERR_CANCELED);
    m.attr("NIXL_ERR_NO_TELEMETRY") = static_cast<int>(NIXL_ERR_NO_TELEMETRY);
    m.attr("NIXL_THREAD_SYNC_NONE") = static_cast<int>(nixl_thread_sync_t::NIXL_THREAD_SYNC_NONE);
    m.attr("NIXL_THREAD_SYNC_STRICT") = static_cast<int>(nixl_thread_sync_t::NIXL_THREAD_SYNC_STRICT);
    m.attr("NIXL_THREAD_SYNC_RW") = static_cast<int>(nixl_thread_sync_t::NIXL_THREAD_SYNC_RW);
    m.attr("NIXL_THREAD_SYNC_DEFAULT") = static_cast<int>(nixl_thread_sync_t::NIXL_THREAD_SYNC_DEFAULT);
    m.attr("NIXL_COST_ANALYTICAL_BACKEND") = static_cast<int>(nixl_cost_t::ANALYTICAL_BACKEND);
    m.attr("DEFAULT_COMM_PORT") = static_cast<int>(default_comm_port);
    m.attr("NIXL_INIT_AGENT") = std::string(NIXL_INIT_AGENT);
    m.attr("NIXL_NULL_AGENT") = nixl_null_agent;
    // The NVLink backend offers the device API whenever a GPU is present; the attribute name
    // is the one programs written for the reference probe.
    m.attr("HAVE_UCX_GPU_DEVICE_API") = true;

    // ---- exceptions ----
    static ErrorTypes err;
    g_err = &err;
    err.base = py::reinterpret_steal<py::object>(PyErr_NewException("nixl_b200._bindings.nixlError", PyExc_RuntimeError, nullptr));
    m.attr("nixlError") = err.base;
    static const char *names[13] = {nullptr,
                                    "nixlNotPostedError",
                                    "nixlInvalidParamError",
                                    "nixlBackendError",
                                    "nixlNotFoundError",
                                    "nixlMismatchError",
                                    "nixlNotAllowedError",
                                    "nixlRepostActiveError",
                                    "nixlUnknownError",
                                    "nixlNotSupportedError",
                                    "nixlRemoteDisconnectError",
                                    "nixlCancelledError",
                                    "nixlNoTelemetryError"};
    for (int i = 1; i <= 12; ++i) {
        const std::string full = std::string("nixl_b200._bindings.") + names[i];
        err.byStatus[i] = py::reinterpret_steal<py::object>(PyErr_NewException(full.c_str(), err.base.ptr(), nullptr));
        m.attr(names[i]) = err.byStatus[i];
    }

    // ---- descriptor lists ----
    py::class_<nixl_xfer_dlist_t>(m, "nixlXferDList")
        .def(py::init([](int mem, const py::object &descs) {
                 nixl_xfer_dlist_t l(static_cast<nixl_mem_t>(mem));
                 fillXfer(l, descs);
                 return l;
             }),
             py::arg("type"), py::arg("descs") = py::none())
        .def("getType", [](const nixl_xfer_dlist_t &l) { return static_cast<int>(l.getType()); })
        .def("descCount", &nixl_xfer_dlist_t::descCount)
        .def("isEmpty", &nixl_xfer_dlist_t::isEmpty)
        .def("__len__", &nixl_xfer_dlist_t::descCount)
        .def("__getitem__",
             [](const nixl_xfer_dlist_t &l, ssize_t i) {
                 if (i < 0) i += l.descCount();
                 if (i < 0 || i >= l.descCount()) throw py::index_error();
                 return xfer_tuple(l[i].addr, l[i].len, l[i].devId);
             })
        .def("__setitem__",
             [](nixl_xfer_dlist_t &l, ssize_t i, const xfer_tuple &t) {
                 if (i < 0) i += l.descCount();
                 if (i < 0 || i >= l.descCount()) throw py::index_error();
                 l[i] = nixlBasicDesc(std::get<0>(t), std::get<1>(t), std::get<2>(t));
             })
        .def("__eq__", [](const nixl_xfer_dlist_t &a, const nixl_xfer_dlist_t &b) { return a == b; })
        .def("addDesc", [](nixl_xfer_dlist_t &l, const xfer_tuple &t) { l.addDesc(nixlBasicDesc(std::get<0>(t), std::get<1>(t), std::get<2>(t))); })
        .def("append", [](nixl_xfer_dlist_t &l, const xfer_tuple &t) { l.addDesc(nixlBasicDesc(std::get<0>(t), std::get<1>(t), std::get<2>(t))); })
        .def("index", [](const nixl_xfer_dlist_t &l, const xfer_tuple &t) {
            const int i = l.getIndex(nixlBasicDesc(std::get<0>(t), std::get<1>(t), std::get<2>(t)));
            if (i < 0) throw py::value_error("descriptor not in list");
            return i;
        })
        .def("remDesc", [](nixl_xfer_dlist_t &l, int i) { l.remDesc(i); })
        .def("clear", &nixl_xfer_dlist_t::clear)
        .def("totalBytes", &nixl_xfer_dlist_t::totalBytes)
        .def("to_array",
             [](const nixl_xfer_dlist_t &l) {
                 py::array_t<uint64_t> a({static_cast<ssize_t>(l.descCount()), static_cast<ssize_t>(3)});
                 if (l.descCount()) std::memcpy(a.mutable_data(), l.data(), static_cast<size_t>(l.descCount()) * sizeof(nixlBasicDesc));
                 return a;
             })
        .def("print", &nixl_xfer_dlist_t::print)
        .def("__repr__", [](const nixl_xfer_dlist_t &l) { return l.to_string(l.descCount() > 16); })
        .def(py::pickle(
            [](const nixl_xfer_dlist_t &l) {
                nixlSerDes sd;
                l.serialize(&sd);
                return py::bytes(sd.exportStr());
            },
            [](const py::bytes &b) {
                nixlSerDes sd;
                if (sd.importStr(b) != NIXL_SUCCESS) throw py::value_error("not a serialized descriptor list");
                nixl_xfer_dlist_t l(&sd);
                if (!l.valid()) throw py::value_error("corrupt serialized descriptor list");
                return l;
            }));

    py::class_<nixl_reg_dlist_t>(m, "nixlRegDList")
        .def(py::init([](int mem, const py::object &descs) {
                 nixl_reg_dlist_t l(static_cast<nixl_mem_t>(mem));
                 if (!descs.is_none())
                     for (auto item : descs) {
                         auto t = item.cast<py::tuple>();
                         if (t.size() < 3) throw py::value_error("registration descriptor is (addr, len, devId[, meta])");
                         std::string meta;
                         if (t.size() > 3) meta = t[3].cast<std::string>();
                         l.addDesc(nixlBlobDesc(t[0].cast<uintptr_t>(), t[1].cast<size_t>(), t[2].cast<uint64_t>(), meta));
                     }
                 return l;
             }),
             py::arg("type"), py::arg("descs") = py::none())
        .def("getType", [](const nixl_reg_dlist_t &l) { return static_cast<int>(l.getType()); })
        .def("descCount", &nixl_reg_dlist_t::descCount)
        .def("isEmpty", &nixl_reg_dlist_t::isEmpty)
        .def("__len__", &nixl_reg_dlist_t::descCount)
        .def("__getitem__",
             [](const nixl_reg_dlist_t &l, ssize_t i) {
                 if (i < 0) i += l.descCount();
                 if (i < 0 || i >= l.descCount()) throw py::index_error();
                 return py::make_tuple(l[i].addr, l[i].len, l[i].devId, py::bytes(l[i].metaInfo));
             })
        .def("__eq__", [](const nixl_reg_dlist_t &a, const nixl_reg_dlist_t &b) { return a == b; })
        .def("addDesc", [](nixl_reg_dlist_t &l, const reg_tuple &t) {
            l.addDesc(nixlBlobDesc(std::get<0>(t), std::get<1>(t), std::get<2>(t), std::get<3>(t)));
        })
        .def("remDesc", [](nixl_reg_dlist_t &l, int i) { l.remDesc(i); })
        .def("clear", &nixl_reg_dlist_t::clear)
        .def("trim", &nixl_reg_dlist_t::trim)
        .def("totalBytes", &nixl_reg_dlist_t::totalBytes)
        .def("print", &nixl_reg_dlist_t::print)
        .def("__repr__", [](const nixl_reg_dlist_t &l) { return l.to_string(l.descCount() > 16); })
        .def(py::pickle(
            [](const nixl_reg_dlist_t &l) {
                nixlSerDes sd;
                l.serialize(&sd);
                return py::bytes(sd.exportStr());
            },
            [](const py::bytes &b) {
                nixlSerDes sd;
                if (sd.importStr(b) != NIXL_SUCCESS) throw py::value_error("not a serialized descriptor list");
                nixl_reg_dlist_t l(&sd);
                if (!l.valid()) throw py::value_error("corrupt serialized descriptor list");
                return l;
            }));

    py::class_<nixl_remote_dlist_t>(m, "nixlRemoteDList")
        .def(py::init([](int mem, const py::object &descs) {
                 nixl_remote_dlist_t l(static_cast<nixl_mem_t>(mem));
                 if (!descs.is_none())
                     for (auto item : descs) {
                         auto t = item.cast<reg_tuple>();
                         l.addDesc(nixlRemoteDesc(std::get<0>(t), std::get<1>(t), std::get<2>(t), std::get<3>(t)));
                     }
                 return l;
             }),
             py::arg("type"), py::arg("descs") = py::none())
        .def("getType", [](const nixl_remote_dlist_t &l) { return static_cast<int>(l.getType()); })
        .def("descCount", &nixl_remote_dlist_t::descCount)
        .def("__len__", &nixl_remote_dlist_t::descCount)
        .def("__getitem__",
             [](const nixl_remote_dlist_t &l, ssize_t i) {
                 if (i < 0) i += l.descCount();
                 if (i < 0 || i >= l.descCount()) throw py::index_error();
                 return py::make_tuple(l[i].addr, l[i].len, l[i].devId, l[i].remoteAgent);
             })
        .def("addDesc", [](nixl_remote_dlist_t &l, const reg_tuple &t) {
            l.addDesc(nixlRemoteDesc(std::get<0>(t), std::get<1>(t), std::get<2>(t), std::get<3>(t)));
        })
        .def("clear", &nixl_remote_dlist_t::clear);

    // ---- config + telemetry struct ----
    py::class_<nixlAgentConfig>(m, "nixlAgentConfig")
        .def(py::init([](bool prog, bool listen, int port, int sync, unsigned workers, uint64_t pthr, uint64_t lthr, bool telem) {
                 return nixlAgentConfig(prog, listen, static_cast<uint16_t>(port), static_cast<nixl_thread_sync_t>(sync), workers, pthr,
                                        lthr, telem);
             }),
             py::arg("use_prog_thread") = false, py::arg("use_listen_thread") = false, py::arg("port") = 0,
             py::arg("sync_mode") = static_cast<int>(nixl_thread_sync_t::NIXL_THREAD_SYNC_DEFAULT), py::arg("num_workers") = 1,
             py::arg("pthr_delay_us") = 0, py::arg("lthr_delay_us") = 100000, py::arg("capture_telemetry") = false)
        .def_readwrite("useProgThread", &nixlAgentConfig::useProgThread)
        .def_readwrite("useListenThread", &nixlAgentConfig::useListenThread)
        .def_readwrite("listenPort", &nixlAgentConfig::listenPort)
        .def_readwrite("captureTelemetry", &nixlAgentConfig::captureTelemetry)
        .def_readwrite("pthrDelay", &nixlAgentConfig::pthrDelay)
        .def_readwrite("lthrDelay", &nixlAgentConfig::lthrDelay);

    py::class_<nixl_xfer_telem_t>(m, "nixlXferTelemetry")
        .def(py::init<>())
        .def_property_readonly("startTime",
                               [](const nixl_xfer_telem_t &t) {
                                   return std::chrono::duration_cast<std::chrono::microseconds>(t.startTime.time_since_epoch()).count();
                               })
        .def_property_readonly("postDuration", [](const nixl_xfer_telem_t &t) { return t.postDuration.count(); })
        .def_property_readonly("xferDuration", [](const nixl_xfer_telem_t &t) { return t.xferDuration.count(); })
        .def_readonly("totalBytes", &nixl_xfer_telem_t::totalBytes)
        .def_readonly("descCount", &nixl_xfer_telem_t::descCount);

    // ---- agent ----
    py::class_<nixlAgent>(m, "nixlAgent")
        // The constructor may probe metadata stores over the network and createBackend initialises
        // CUDA: neither should stall other Python threads.
        .def(py::init<const std::string &, const nixlAgentConfig &>(), py::call_guard<py::gil_scoped_release>())
        .def("getAvailPlugins",
             [](nixlAgent &a) {
                 std::vector<nixl_backend_t> v;
                 throwIf(a.getAvailPlugins(v), "getAvailPlugins");
                 return v;
             })
        .def("getPluginParams",
             [](nixlAgent &a, const std::string &type) {
                 nixl_mem_list_t mems;
                 nixl_b_params_t params;
                 throwIf(a.getPluginParams(type, mems, params), "getPluginParams");
                 std::vector<int> m2(mems.begin(), mems.end());
                 return py::make_tuple(paramsToDict(params), m2);
             })
        .def("getBackendParams",
             [](nixlAgent &a, uintptr_t backend) {
                 nixl_mem_list_t mems;
                 nixl_b_params_t params;
                 throwIf(a.getBackendParams(asHandle<nixlBackendH>(backend), mems, params), "getBackendParams");
                 std::vector<int> m2(mems.begin(), mems.end());
                 return py::make_tuple(paramsToDict(params), m2);
             })
        .def("createBackend",
             [](nixlAgent &a, const std::string &type, const nixl_b_params_t &params) {
                 nixlBackendH *h = nullptr;
                 nixl_status_t st;
                 {
                     py::gil_scoped_release nogil;
                     st = a.createBackend(type, params, h);
                 }
                 throwIf(st, "createBackend");
                 return reinterpret_cast<uintptr_t>(h);
             })
        .def("registerMem",
             [](nixlAgent &a, const nixl_reg_dlist_t &descs, const std::vector<uintptr_t> &backends) {
                 nixl_opt_args_t o = makeOpt(backends);
                 py::gil_scoped_release nogil;
                 return static_cast<int>(a.registerMem(descs, &o));
             },
             py::arg("descs"), py::arg("backends") = std::vector<uintptr_t>{})
        .def("deregisterMem",
             [](nixlAgent &a, const nixl_reg_dlist_t &descs, const std::vector<uintptr_t> &backends) {
                 nixl_opt_args_t o = makeOpt(backends);
                 py::gil_scoped_release nogil;
                 return static_cast<int>(a.deregisterMem(descs, &o));
             },
             py::arg("descs"), py::arg("backends") = std::vector<uintptr_t>{})
        .def("queryMem",
             [](nixlAgent &a, const nixl_reg_dlist_t &descs, uintptr_t backend) {
                 nixl_opt_args_t o = makeOpt({backend});
                 std::vector<nixl_query_resp_t> resp;
                 throwIf(a.queryMem(descs, resp, &o), "queryMem");
                 py::list out;
                 for (auto &r : resp) {
                     if (r.has_value()) out.append(paramsToDict(*r));
                     else out.append(py::none());
                 }
                 return out;
             })
        .def("makeConnection",
             [](nixlAgent &a, const std::string &remote, const std::vector<uintptr_t> &backends) {
                 nixl_opt_args_t o = makeOpt(backends);
                 return static_cast<int>(a.makeConnection(remote, &o));
             },
             py::arg("remote_agent"), py::arg("backends") = std::vector<uintptr_t>{})
        .def("prepXferDlist",
             [](nixlAgent &a, const std::string &agent_name, const nixl_xfer_dlist_t &descs, const std::vector<uintptr_t> &backends) {
                 nixl_opt_args_t o = makeOpt(backends);
                 nixlDlistH *h = nullptr;
                 {
                     py::gil_scoped_release nogil;
                     const nixl_status_t st = a.prepXferDlist(agent_name, descs, h, &o);
                     py::gil_scoped_acquire gil;
                     throwIf(st, "prepXferDlist");
                 }
                 return reinterpret_cast<uintptr_t>(h);
             },
             py::arg("agent_name"), py::arg("descs"), py::arg("backends") = std::vector<uintptr_t>{})
        .def("makeXferReq",
             [](nixlAgent &a, int op, uintptr_t local_side, const py::object &local_idx, uintptr_t remote_side,
                const py::object &remote_idx, const py::object &notif, const std::vector<uintptr_t> &backends, bool skip_merge) {
                 nixl_opt_args_t o = makeOpt(backends, notif);
                 o.skipDescMerge = skip_merge;
                 auto toVec = [](const py::object &src) {
                     if (py::isinstance<py::array>(src)) {
                         auto arr = py::array_t<int32_t, py::array::c_style | py::array::forcecast>::ensure(src);
                         if (!arr || arr.ndim() != 1) throw py::value_error("index array must be one-dimensional");
                         return std::vector<int>(arr.data(), arr.data() + arr.shape(0));
                     }
                     return src.cast<std::vector<int>>();
                 };
                 const std::vector<int> li = toVec(local_idx), ri = toVec(remote_idx);
                 nixlXferReqH *req = nullptr;
                 throwIf(a.makeXferReq(static_cast<nixl_xfer_op_t>(op), asHandle<nixlDlistH>(local_side), li,
                                       asHandle<nixlDlistH>(remote_side), ri, req, &o),
                         "makeXferReq");
                 return reinterpret_cast<uintptr_t>(req);
             },
             py::arg("operation"), py::arg("local_side"), py::arg("local_indices"), py::arg("remote_side"), py::arg("remote_indices"),
             py::arg("notif_msg") = py::none(), py::arg("backends") = std::vector<uintptr_t>{}, py::arg("skip_desc_merge") = false)
        .def("createXferReq",
             [](nixlAgent &a, int op, const nixl_xfer_dlist_t &local, const nixl_xfer_dlist_t &remote, const std::string &remote_agent,
                const py::object &notif, const std::vector<uintptr_t> &backends) {
                 nixl_opt_args_t o = makeOpt(backends, notif);
                 nixlXferReqH *req = nullptr;
                 throwIf(a.createXferReq(static_cast<nixl_xfer_op_t>(op), local, remote, remote_agent, req, &o), "createXferReq");
                 return reinterpret_cast<uintptr_t>(req);
             },
             py::arg("operation"), py::arg("local_descs"), py::arg("remote_descs"), py::arg("remote_agent"),
             py::arg("notif_msg") = py::none(), py::arg("backends") = std::vector<uintptr_t>{})
        .def("estimateXferCost",
             [](nixlAgent &a, uintptr_t req) {
                 std::chrono::microseconds d{0}, e{0};
                 nixl_cost_t method = nixl_cost_t::ANALYTICAL_BACKEND;
                 throwIf(a.estimateXferCost(asHandle<nixlXferReqH>(req), d, e, method), "estimateXferCost");
                 return py::make_tuple(d.count(), e.count(), static_cast<int>(method));
             })
        .def("postXferReq",
             [](nixlAgent &a, uintptr_t req, const py::object &notif, const std::string &custom) {
                 nixlXferReqH *r = asHandle<nixlXferReqH>(req);
                 nixl_status_t st;
                 if (notif.is_none() && custom.empty()) {
                     st = a.postXferReq(r);
                 } else {
                     nixl_opt_args_t o;
                     // Option structs without a notification clear the request's own one, so a
                     // post that only carries a custom parameter re-states it.
                     if (!notif.is_none()) o.notif = notif.cast<std::string>();
                     else if (r && r->hasNotif) o.notif = r->notifMsg;
                     o.customParam = custom;
                     st = a.postXferReq(r, &o);
                 }
                 throwIf(st, "postXferReq");
                 return static_cast<int>(st);
             },
             py::arg("req"), py::arg("notif_msg") = py::none(), py::arg("custom_param") = std::string())
        .def("getXferStatus",
             [](nixlAgent &a, uintptr_t req) {
                 const nixl_status_t st = a.getXferStatus(asHandle<nixlXferReqH>(req));
                 throwIf(st, "getXferStatus");
                 return static_cast<int>(st);
             })
        .def("getXferTelemetry",
             [](nixlAgent &a, uintptr_t req) {
                 nixl_xfer_telem_t t;
                 throwIf(a.getXferTelemetry(asHandle<nixlXferReqH>(req), t), "getXferTelemetry");
                 return t;
             })
        .def("queryXferBackend",
             [](nixlAgent &a, uintptr_t req) {
                 nixlBackendH *b = nullptr;
                 throwIf(a.queryXferBackend(asHandle<nixlXferReqH>(req), b), "queryXferBackend");
                 return reinterpret_cast<uintptr_t>(b);
             })
        .def("releaseXferReq", [](nixlAgent &a, uintptr_t req) { return static_cast<int>(a.releaseXferReq(asHandle<nixlXferReqH>(req))); })
        .def("releasedDlistH", [](nixlAgent &a, uintptr_t h) { return static_cast<int>(a.releasedDlistH(asHandle<nixlDlistH>(h))); })
        .def("prepMemView",
             [](nixlAgent &a, const py::object &dlist, const std::vector<uintptr_t> &backends) {
                 nixl_opt_args_t o = makeOpt(backends);
                 nixlMemViewH mvh = nullptr;
                 if (py::isinstance<nixl_remote_dlist_t>(dlist)) throwIf(a.prepMemView(dlist.cast<const nixl_remote_dlist_t &>(), mvh, &o), "prepMemView");
                 else throwIf(a.prepMemView(dlist.cast<const nixl_xfer_dlist_t &>(), mvh, &o), "prepMemView");
                 return reinterpret_cast<uintptr_t>(mvh);
             },
             py::arg("dlist"), py::arg("backends") = std::vector<uintptr_t>{})
        .def("releaseMemView", [](nixlAgent &a, uintptr_t mvh) { a.releaseMemView(reinterpret_cast<nixlMemViewH>(mvh)); })
        .def("getNotifs",
             [](nixlAgent &a, py::dict existing, const std::vector<uintptr_t> &backends) {
                 nixl_opt_args_t o = makeOpt(backends);
                 nixl_notifs_t fresh;
                 throwIf(a.getNotifs(fresh, &o), "getNotifs");
                 for (auto &kv : fresh) {
                     py::str key(kv.first);
                     py::list msgs = existing.contains(key) ? existing[key].cast<py::list>() : py::list();
                     for (auto &msg : kv.second) msgs.append(py::bytes(msg));
                     existing[key] = msgs;
                 }
                 return existing;
             },
             py::arg("notif_map"), py::arg("backends") = std::vector<uintptr_t>{})
        .def("genNotif",
             [](nixlAgent &a, const std::string &remote, const std::string &msg, const std::vector<uintptr_t> &backends) {
                 nixl_opt_args_t o = makeOpt(backends);
                 const nixl_status_t st = a.genNotif(remote, msg, &o);
                 throwIf(st, "genNotif");
                 return static_cast<int>(st);
             },
             py::arg("remote_agent"), py::arg("msg"), py::arg("backends") = std::vector<uintptr_t>{})
        .def("getLocalMD",
             [](nixlAgent &a) {
                 nixl_blob_t md;
                 throwIf(a.getLocalMD(md), "getLocalMD");
                 return py::bytes(md);
             })
        .def("getLocalPartialMD",
             [](nixlAgent &a, const nixl_reg_dlist_t &descs, bool inc_conn, const std::vector<uintptr_t> &backends) {
                 nixl_opt_args_t o = makeOpt(backends);
                 o.includeConnInfo = inc_conn;
                 nixl_blob_t md;
                 throwIf(a.getLocalPartialMD(descs, md, &o), "getLocalPartialMD");
                 return py::bytes(md);
             },
             py::arg("descs"), py::arg("inc_conn_info") = false, py::arg("backends") = std::vector<uintptr_t>{})
        .def("loadRemoteMD",
             [](nixlAgent &a, const std::string &md) {
                 std::string name;
                 throwIf(a.loadRemoteMD(md, name), "loadRemoteMD");
                 return py::bytes(name);
             })
        .def("invalidateRemoteMD", [](nixlAgent &a, const std::string &remote) { return static_cast<int>(a.invalidateRemoteMD(remote)); })
        .def("sendLocalMD",
             [](nixlAgent &a, const std::string &ip, int port, const std::string &label) {
                 nixl_opt_args_t o;
                 o.ipAddr = ip;
                 o.port = port;
                 o.metadataLabel = label;
                 throwIf(a.sendLocalMD(&o), "sendLocalMD");
             },
             py::arg("ip_addr") = std::string(), py::arg("port") = static_cast<int>(default_comm_port), py::arg("label") = std::string())
        .def("sendLocalPartialMD",
             [](nixlAgent &a, const nixl_reg_dlist_t &descs, bool inc_conn, const std::vector<uintptr_t> &backends, const std::string &ip,
                int port, const std::string &label) {
                 nixl_opt_args_t o = makeOpt(backends);
                 o.includeConnInfo = inc_conn;
                 o.ipAddr = ip;
                 o.port = port;
                 o.metadataLabel = label;
                 throwIf(a.sendLocalPartialMD(descs, &o), "sendLocalPartialMD");
             },
             py::arg("descs"), py::arg("inc_conn_info") = false, py::arg("backends") = std::vector<uintptr_t>{},
             py::arg("ip_addr") = std::string(), py::arg("port") = static_cast<int>(default_comm_port), py::arg("label") = std::string())
        .def("fetchRemoteMD",
             [](nixlAgent &a, const std::string &remote, const std::string &ip, int port, const std::string &label) {
                 nixl_opt_args_t o;
                 o.ipAddr = ip;
                 o.port = port;
                 o.metadataLabel = label;
                 throwIf(a.fetchRemoteMD(remote, &o), "fetchRemoteMD");
             },
             py::arg("remote_agent"), py::arg("ip_addr") = std::string(), py::arg("port") = static_cast<int>(default_comm_port),
             py::arg("label") = std::string())
        .def("invalidateLocalMD",
             [](nixlAgent &a, const std::string &ip, int port) {
                 nixl_opt_args_t o;
                 o.ipAddr = ip;
                 o.port = port;
                 throwIf(a.invalidateLocalMD(&o), "invalidateLocalMD");
             },
             py::arg("ip_addr") = std::string(), py::arg("port") = static_cast<int>(default_comm_port))
        .def("checkRemoteMD", [](nixlAgent &a, const std::string &remote, const nixl_xfer_dlist_t &descs) {
            return a.checkRemoteMD(remote, descs) == NIXL_SUCCESS;
        });

    m.def("status_str", [](int st) { return nixlEnumStrings::statusStr(static_cast<nixl_status_t>(st)); });
    m.def("mem_type_str", [](int mem) { return nixlEnumStrings::memTypeStr(static_cast<nixl_mem_t>(mem)); });
}

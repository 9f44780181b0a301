"""C API (libnixl_capi.so) driven through ctypes: two agents, DRAM write with notification,
containers and iterators.  Mirrors the scenarios of the reference's Rust binding tests
(src/bindings/rust/tests/tests.rs), which exercise the same C functions."""
import ctypes
import os

import numpy as np

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "nixl_b200", "lib", "libnixl_capi.so")
os.environ.setdefault("NIXL_PLUGIN_DIR", os.path.join(os.path.dirname(LIB), "plugins"))

c = ctypes.CDLL(LIB)
VP = ctypes.c_void_p


def ok(rc):
    assert rc == 0, rc


def test_capi_roundtrip():
    assert c.nixl_capi_is_stub() == 0
    a, b = VP(), VP()
    ok(c.nixl_capi_create_agent(b"capi_a", ctypes.byref(a)))
    ok(c.nixl_capi_create_agent(b"capi_b", ctypes.byref(b)))

    plugins = VP()
    ok(c.nixl_capi_get_available_plugins(a, ctypes.byref(plugins)))
    n = ctypes.c_size_t()
    ok(c.nixl_capi_string_list_size(plugins, ctypes.byref(n)))
    names = []
    for i in range(n.value):
        s = ctypes.c_char_p()
        ok(c.nixl_capi_string_list_get(plugins, ctypes.c_size_t(i), ctypes.byref(s)))
        names.append(s.value.decode())
    assert "NVLINK" in names and "POSIX" in names
    ok(c.nixl_capi_destroy_string_list(plugins))

    mems, params = VP(), VP()
    ok(c.nixl_capi_get_plugin_params(a, b"NVLINK", ctypes.byref(mems), ctypes.byref(params)))
    it = VP()
    ok(c.nixl_capi_params_create_iterator(params, ctypes.byref(it)))
    keys = []
    while True:
        k, v, more = ctypes.c_char_p(), ctypes.c_char_p(), ctypes.c_bool()
        if c.nixl_capi_params_iterator_next(it, ctypes.byref(k), ctypes.byref(v), ctypes.byref(more)) != 0:
            break
        keys.append(k.value.decode())
        if not more.value:
            break
    assert "copy_path" in keys
    ok(c.nixl_capi_params_destroy_iterator(it))
    msize = ctypes.c_size_t()
    ok(c.nixl_capi_mem_list_size(mems, ctypes.byref(msize)))
    assert msize.value == 2

    ba, bb = VP(), VP()
    ok(c.nixl_capi_create_backend(a, b"NVLINK", params, ctypes.byref(ba)))
    ok(c.nixl_capi_create_backend(b, b"NVLINK", params, ctypes.byref(bb)))
    ok(c.nixl_capi_destroy_params(params))
    ok(c.nixl_capi_destroy_mem_list(mems))

    src = np.random.default_rng(0).integers(0, 255, 1 << 20, dtype=np.uint8)
    dst = np.zeros_like(src)
    for agent, arr in ((a, src), (b, dst)):
        reg = VP()
        ok(c.nixl_capi_create_reg_dlist(0, ctypes.byref(reg)))
        ok(c.nixl_capi_reg_dlist_add_desc(reg, ctypes.c_size_t(arr.ctypes.data), ctypes.c_size_t(arr.nbytes), ctypes.c_uint64(0), None, ctypes.c_size_t(0)))
        ok(c.nixl_capi_register_mem(agent, reg, None))
        ok(c.nixl_capi_destroy_reg_dlist(reg))

    md, mdlen = VP(), ctypes.c_size_t()
    ok(c.nixl_capi_get_local_md(b, ctypes.byref(md), ctypes.byref(mdlen)))
    name = ctypes.c_char_p()
    ok(c.nixl_capi_load_remote_md(a, md, mdlen, ctypes.byref(name)))
    assert name.value == b"capi_b"

    local, remote = VP(), VP()
    ok(c.nixl_capi_create_xfer_dlist(0, ctypes.byref(local)))
    ok(c.nixl_capi_create_xfer_dlist(0, ctypes.byref(remote)))
    for i in range(4):
        off = i * (1 << 18)
        ok(c.nixl_capi_xfer_dlist_add_desc(local, ctypes.c_size_t(src.ctypes.data + off), ctypes.c_size_t(1 << 18), ctypes.c_uint64(0)))
        ok(c.nixl_capi_xfer_dlist_add_desc(remote, ctypes.c_size_t(dst.ctypes.data + off), ctypes.c_size_t(1 << 18), ctypes.c_uint64(0)))
    total = ctypes.c_size_t()
    ok(c.nixl_capi_xfer_dlist_len(local, ctypes.byref(total)))
    assert total.value == 1 << 20
    assert c.nixl_capi_check_remote_md(a, b"capi_b", remote) == 0
    assert c.nixl_capi_check_remote_md(a, b"nobody", None) == -6

    opt = VP()
    ok(c.nixl_capi_create_opt_args(ctypes.byref(opt)))
    ok(c.nixl_capi_opt_args_set_notif_msg(opt, b"done!", ctypes.c_size_t(5)))
    req = VP()
    ok(c.nixl_capi_create_xfer_req(a, 1, local, remote, b"capi_b", ctypes.byref(req), opt))
    rc = c.nixl_capi_post_xfer_req(a, req, None)
    assert rc in (0, 1)
    while rc == 1:
        rc = c.nixl_capi_get_xfer_status(a, req)
    assert rc == 0 and (src == dst).all()
    dur, margin, method = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int()
    ok(c.nixl_capi_estimate_xfer_cost(a, req, None, ctypes.byref(dur), ctypes.byref(margin), ctypes.byref(method)))
    assert dur.value > 0
    ok(c.nixl_capi_release_xfer_req(a, req))
    ok(c.nixl_capi_destroy_xfer_req(req))

    nm = VP()
    ok(c.nixl_capi_create_notif_map(ctypes.byref(nm)))
    for _ in range(100000):
        ok(c.nixl_capi_get_notifs(b, nm, None))
        ok(c.nixl_capi_notif_map_size(nm, ctypes.byref(n)))
        if n.value:
            break
    assert n.value == 1
    who = ctypes.c_char_p()
    ok(c.nixl_capi_notif_map_get_agent_at(nm, ctypes.c_size_t(0), ctypes.byref(who)))
    assert who.value == b"capi_a"
    data, dlen = VP(), ctypes.c_size_t()
    ok(c.nixl_capi_notif_map_get_notif(nm, b"capi_a", ctypes.c_size_t(0), ctypes.byref(data), ctypes.byref(dlen)))
    assert ctypes.string_at(data, dlen.value) == b"done!"
    ok(c.nixl_capi_destroy_notif_map(nm))
    ok(c.nixl_capi_destroy_opt_args(opt))
    ok(c.nixl_capi_destroy_xfer_dlist(local))
    ok(c.nixl_capi_destroy_xfer_dlist(remote))
    ok(c.nixl_capi_invalidate_remote_md(a, b"capi_b"))
    ok(c.nixl_capi_destroy_backend(ba))
    ok(c.nixl_capi_destroy_backend(bb))
    ok(c.nixl_capi_destroy_agent(a))
    ok(c.nixl_capi_destroy_agent(b))

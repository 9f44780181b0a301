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


def _agent(name, backend=b"NVLINK"):
    a, params, mems, bh = VP(), VP(), VP(), VP()
    ok(c.nixl_capi_create_agent(name, ctypes.byref(a)))
    ok(c.nixl_capi_get_plugin_params(a, backend, ctypes.byref(mems), ctypes.byref(params)))
    ok(c.nixl_capi_create_backend(a, backend, params, ctypes.byref(bh)))
    ok(c.nixl_capi_destroy_params(params))
    ok(c.nixl_capi_destroy_mem_list(mems))
    return a, bh


def _register(agent, arr):
    reg = VP()
    ok(c.nixl_capi_create_reg_dlist(0, ctypes.byref(reg)))
    ok(c.nixl_capi_reg_dlist_add_desc(reg, ctypes.c_size_t(arr.ctypes.data), ctypes.c_size_t(arr.nbytes), ctypes.c_uint64(0), None, ctypes.c_size_t(0)))
    ok(c.nixl_capi_register_mem(agent, reg, None))
    return reg


def test_capi_containers():
    """Parameter maps, memory-type lists, descriptor lists and option blocks on their own."""
    params = VP()
    ok(c.nixl_capi_create_params(ctypes.byref(params)))
    empty = ctypes.c_bool()
    ok(c.nixl_capi_params_is_empty(params, ctypes.byref(empty)))
    assert empty.value
    ok(c.nixl_capi_params_add(params, b"alpha", b"1"))
    ok(c.nixl_capi_params_add(params, b"beta", b"two"))
    ok(c.nixl_capi_params_is_empty(params, ctypes.byref(empty)))
    assert not empty.value
    it, seen = VP(), {}
    ok(c.nixl_capi_params_create_iterator(params, ctypes.byref(it)))
    while True:
        k, v, more = ctypes.c_char_p(), ctypes.c_char_p(), ctypes.c_bool()
        if c.nixl_capi_params_iterator_next(it, ctypes.byref(k), ctypes.byref(v), ctypes.byref(more)) != 0:
            break
        seen[k.value] = v.value
        if not more.value:
            break
    assert seen == {b"alpha": b"1", b"beta": b"two"}
    ok(c.nixl_capi_params_destroy_iterator(it))
    ok(c.nixl_capi_destroy_params(params))

    for code, text in ((0, b"DRAM"), (1, b"VRAM"), (4, b"FILE")):
        s = ctypes.c_char_p()
        ok(c.nixl_capi_mem_type_to_string(code, ctypes.byref(s)))
        assert text in s.value.upper()

    for kind in ("xfer", "reg"):
        f = lambda name: getattr(c, f"nixl_capi_{kind}_dlist_{name}")  # noqa: E731
        dl = VP()
        ok(getattr(c, f"nixl_capi_create_{kind}_dlist")(1, ctypes.byref(dl)))
        mt, cnt, emp = ctypes.c_int(), ctypes.c_size_t(), ctypes.c_bool()
        ok(f("get_type")(dl, ctypes.byref(mt)))
        assert mt.value == 1
        ok(f("is_empty")(dl, ctypes.byref(emp)))
        assert emp.value
        for i in range(3):
            if kind == "xfer":
                ok(f("add_desc")(dl, ctypes.c_size_t(0x1000 * (i + 1)), ctypes.c_size_t(256), ctypes.c_uint64(i)))
            else:
                ok(f("add_desc")(dl, ctypes.c_size_t(0x1000 * (i + 1)), ctypes.c_size_t(256), ctypes.c_uint64(i), b"meta", ctypes.c_size_t(4)))
        ok(f("desc_count")(dl, ctypes.byref(cnt)))
        assert cnt.value == 3
        ok(f("rem_desc")(dl, 1))
        ok(f("desc_count")(dl, ctypes.byref(cnt)))
        assert cnt.value == 2
        assert f("rem_desc")(dl, 7) != 0  # out of range
        ok(f("resize")(dl, ctypes.c_size_t(5)))
        ok(f("desc_count")(dl, ctypes.byref(cnt)))
        assert cnt.value == 5
        ok(f("trim")(dl))
        ok(f("print")(dl))
        ok(f("clear")(dl))
        ok(f("is_empty")(dl, ctypes.byref(emp)))
        assert emp.value
        ok(getattr(c, f"nixl_capi_destroy_{kind}_dlist")(dl))

    opt = VP()
    ok(c.nixl_capi_create_opt_args(ctypes.byref(opt)))
    flag = ctypes.c_bool(True)
    ok(c.nixl_capi_opt_args_get_has_notif(opt, ctypes.byref(flag)))
    assert not flag.value
    ok(c.nixl_capi_opt_args_set_notif_msg(opt, b"\x00bin\xff", ctypes.c_size_t(5)))
    ok(c.nixl_capi_opt_args_get_has_notif(opt, ctypes.byref(flag)))
    assert flag.value
    data, n = VP(), ctypes.c_size_t()
    ok(c.nixl_capi_opt_args_get_notif_msg(opt, ctypes.byref(data), ctypes.byref(n)))
    assert ctypes.string_at(data, n.value) == b"\x00bin\xff"
    ok(c.nixl_capi_opt_args_set_has_notif(opt, False))
    ok(c.nixl_capi_opt_args_get_has_notif(opt, ctypes.byref(flag)))
    assert not flag.value
    ok(c.nixl_capi_opt_args_set_skip_desc_merge(opt, True))
    ok(c.nixl_capi_opt_args_get_skip_desc_merge(opt, ctypes.byref(flag)))
    assert flag.value
    ok(c.nixl_capi_opt_args_set_ip_addr(opt, b"127.0.0.1"))
    ok(c.nixl_capi_opt_args_set_port(opt, ctypes.c_uint16(5555)))
    ok(c.nixl_capi_destroy_opt_args(opt))
    # null handles are refused, not dereferenced
    assert c.nixl_capi_params_add(None, b"k", b"v") != 0
    assert c.nixl_capi_xfer_dlist_len(None, ctypes.byref(n)) != 0
    assert c.nixl_capi_create_agent(None, ctypes.byref(VP())) != 0


def test_capi_prepared_lists_backend_params_and_notifications():
    """prepXferDlist + makeXferReq by index, READ, backend query, stand-alone notification, deregistration."""
    a, ba = _agent(b"capi2_a")
    b, bb = _agent(b"capi2_b")
    mems, params = VP(), VP()
    ok(c.nixl_capi_get_backend_params(a, ba, ctypes.byref(mems), ctypes.byref(params)))
    empty, n, mt = ctypes.c_bool(), ctypes.c_size_t(), ctypes.c_int()
    ok(c.nixl_capi_mem_list_is_empty(mems, ctypes.byref(empty)))
    ok(c.nixl_capi_mem_list_size(mems, ctypes.byref(n)))
    assert not empty.value and n.value == 2
    kinds = set()
    for i in range(n.value):
        ok(c.nixl_capi_mem_list_get(mems, ctypes.c_size_t(i), ctypes.byref(mt)))
        kinds.add(mt.value)
    assert kinds == {0, 1}
    assert c.nixl_capi_mem_list_get(mems, ctypes.c_size_t(9), ctypes.byref(mt)) != 0
    ok(c.nixl_capi_destroy_mem_list(mems))
    ok(c.nixl_capi_destroy_params(params))

    mine = np.arange(1 << 16, dtype=np.uint8)
    theirs = np.random.default_rng(3).integers(0, 255, 1 << 16, dtype=np.uint8)
    want = theirs.copy()
    reg_a, reg_b = _register(a, mine), _register(b, theirs)
    md, mdlen, name = VP(), ctypes.c_size_t(), ctypes.c_char_p()
    ok(c.nixl_capi_get_local_md(b, ctypes.byref(md), ctypes.byref(mdlen)))
    ok(c.nixl_capi_load_remote_md(a, md, mdlen, ctypes.byref(name)))
    ok(c.nixl_capi_agent_make_connection(a, b"capi2_b", None))
    assert c.nixl_capi_agent_make_connection(a, b"stranger", None) != 0

    # sixteen 4 KiB pieces on each side, prepared once; the request picks pieces by index (reversed on the remote side)
    local, remote = VP(), VP()
    ok(c.nixl_capi_create_xfer_dlist(0, ctypes.byref(local)))
    ok(c.nixl_capi_create_xfer_dlist(0, ctypes.byref(remote)))
    for i in range(16):
        ok(c.nixl_capi_xfer_dlist_add_desc(local, ctypes.c_size_t(mine.ctypes.data + i * 4096), ctypes.c_size_t(4096), ctypes.c_uint64(0)))
        ok(c.nixl_capi_xfer_dlist_add_desc(remote, ctypes.c_size_t(theirs.ctypes.data + i * 4096), ctypes.c_size_t(4096), ctypes.c_uint64(0)))
    hl, hr = VP(), VP()
    ok(c.nixl_capi_prep_xfer_dlist(a, b"", local, ctypes.byref(hl), None))  # empty name: the initiator's own side
    ok(c.nixl_capi_prep_xfer_dlist(a, b"capi2_b", remote, ctypes.byref(hr), None))
    li = (ctypes.c_int * 4)(0, 1, 2, 3)
    ri = (ctypes.c_int * 4)(15, 14, 13, 12)
    req = VP()
    ok(c.nixl_capi_make_xfer_req(a, 0, hl, li, ctypes.c_size_t(4), hr, ri, ctypes.c_size_t(4), ctypes.byref(req), None))  # READ
    backend = VP()
    ok(c.nixl_capi_query_xfer_backend(a, req, ctypes.byref(backend)))
    assert backend.value  # a handle of its own to the same engine: released like any backend handle
    ok(c.nixl_capi_destroy_backend(backend))
    rc = c.nixl_capi_post_xfer_req(a, req, None)
    while rc == 1:
        rc = c.nixl_capi_get_xfer_status(a, req)
    assert rc == 0
    for j in range(4):
        assert (mine[j * 4096:(j + 1) * 4096] == want[(15 - j) * 4096:(16 - j) * 4096]).all()
    assert (mine[4 * 4096:] == np.arange(1 << 16, dtype=np.uint8)[4 * 4096:]).all()
    # mismatching index counts are refused
    bad = VP()
    assert c.nixl_capi_make_xfer_req(a, 0, hl, li, ctypes.c_size_t(4), hr, ri, ctypes.c_size_t(3), ctypes.byref(bad), None) != 0
    ok(c.nixl_capi_release_xfer_req(a, req))
    ok(c.nixl_capi_destroy_xfer_req(req))
    ok(c.nixl_capi_release_xfer_dlist_handle(a, hl))
    ok(c.nixl_capi_release_xfer_dlist_handle(a, hr))

    # a notification of its own, binary payload, and the map accessors
    ok(c.nixl_capi_gen_notif(a, b"capi2_b", b"he\x00llo", ctypes.c_size_t(6), None))
    ok(c.nixl_capi_gen_notif(a, b"capi2_b", b"again", ctypes.c_size_t(5), None))
    nm = VP()
    ok(c.nixl_capi_create_notif_map(ctypes.byref(nm)))
    for _ in range(200000):
        ok(c.nixl_capi_get_notifs(b, nm, None))
        ok(c.nixl_capi_notif_map_get_notifs_size(nm, b"capi2_a", ctypes.byref(n)))
        if n.value >= 2:
            break
    assert n.value == 2
    data, dlen = VP(), ctypes.c_size_t()
    ok(c.nixl_capi_notif_map_get_notif(nm, b"capi2_a", ctypes.c_size_t(0), ctypes.byref(data), ctypes.byref(dlen)))
    assert ctypes.string_at(data, dlen.value) == b"he\x00llo"
    assert c.nixl_capi_notif_map_get_notif(nm, b"capi2_a", ctypes.c_size_t(5), ctypes.byref(data), ctypes.byref(dlen)) != 0
    assert c.nixl_capi_notif_map_get_notifs_size(nm, b"nobody", ctypes.byref(n)) != 0 or n.value == 0
    ok(c.nixl_capi_notif_map_clear(nm))
    ok(c.nixl_capi_notif_map_size(nm, ctypes.byref(n)))
    assert n.value == 0
    ok(c.nixl_capi_destroy_notif_map(nm))
    assert c.nixl_capi_gen_notif(a, b"stranger", b"x", ctypes.c_size_t(1), None) != 0

    ok(c.nixl_capi_destroy_xfer_dlist(local))
    ok(c.nixl_capi_destroy_xfer_dlist(remote))
    ok(c.nixl_capi_deregister_mem(a, reg_a, None))
    ok(c.nixl_capi_deregister_mem(b, reg_b, None))
    assert c.nixl_capi_deregister_mem(a, reg_a, None) != 0  # already gone
    ok(c.nixl_capi_destroy_reg_dlist(reg_a))
    ok(c.nixl_capi_destroy_reg_dlist(reg_b))
    for h in (ba, bb):
        ok(c.nixl_capi_destroy_backend(h))
    for h in (a, b):
        ok(c.nixl_capi_destroy_agent(h))


def test_capi_query_mem_and_partial_metadata(tmp_path):
    """queryMem on files through the POSIX backend, and metadata restricted to some registrations."""
    a, ba = _agent(b"capi3_a", b"POSIX")
    present = tmp_path / "there.bin"
    present.write_bytes(b"x" * 100)
    reg = VP()
    ok(c.nixl_capi_create_reg_dlist(4, ctypes.byref(reg)))
    for path in (present, tmp_path / "missing.bin"):
        meta = str(path).encode()
        ok(c.nixl_capi_reg_dlist_add_desc(reg, ctypes.c_size_t(0), ctypes.c_size_t(0), ctypes.c_uint64(0), meta, ctypes.c_size_t(len(meta))))
    resp = VP()
    ok(c.nixl_capi_create_query_resp_list(ctypes.byref(resp)))
    assert c.nixl_capi_query_mem(a, reg, resp, None) != 0  # exactly one backend has to be named
    opt = VP()
    ok(c.nixl_capi_create_opt_args(ctypes.byref(opt)))
    ok(c.nixl_capi_opt_args_add_backend(opt, ba))
    ok(c.nixl_capi_query_mem(a, reg, resp, opt))
    ok(c.nixl_capi_destroy_opt_args(opt))
    n, has = ctypes.c_size_t(), ctypes.c_bool()
    ok(c.nixl_capi_query_resp_list_size(resp, ctypes.byref(n)))
    assert n.value == 2
    ok(c.nixl_capi_query_resp_list_has_value(resp, ctypes.c_size_t(0), ctypes.byref(has)))
    assert has.value
    params = VP()
    ok(c.nixl_capi_query_resp_list_get_params(resp, ctypes.c_size_t(0), ctypes.byref(params)))
    empty = ctypes.c_bool()
    ok(c.nixl_capi_params_is_empty(params, ctypes.byref(empty)))
    assert not empty.value
    ok(c.nixl_capi_destroy_params(params))
    ok(c.nixl_capi_query_resp_list_has_value(resp, ctypes.c_size_t(1), ctypes.byref(has)))
    assert not has.value
    assert c.nixl_capi_query_resp_list_has_value(resp, ctypes.c_size_t(2), ctypes.byref(has)) != 0
    ok(c.nixl_capi_destroy_query_resp_list(resp))
    ok(c.nixl_capi_destroy_reg_dlist(reg))
    ok(c.nixl_capi_destroy_backend(ba))
    ok(c.nixl_capi_destroy_agent(a))

    # partial metadata: a later registration reaches the peer without resending everything
    b, bb = _agent(b"capi3_b")
    d, bd = _agent(b"capi3_d")
    first, second = np.zeros(4096, dtype=np.uint8), np.zeros(4096, dtype=np.uint8)
    r1 = _register(b, first)
    md, mdlen, name = VP(), ctypes.c_size_t(), ctypes.c_char_p()
    ok(c.nixl_capi_get_local_md(b, ctypes.byref(md), ctypes.byref(mdlen)))
    ok(c.nixl_capi_load_remote_md(d, md, mdlen, ctypes.byref(name)))
    assert name.value == b"capi3_b"
    r2 = _register(b, second)
    probe = VP()
    ok(c.nixl_capi_create_xfer_dlist(0, ctypes.byref(probe)))
    ok(c.nixl_capi_xfer_dlist_add_desc(probe, ctypes.c_size_t(first.ctypes.data), ctypes.c_size_t(4096), ctypes.c_uint64(0)))
    assert c.nixl_capi_check_remote_md(d, b"capi3_b", probe) == 0
    ok(c.nixl_capi_xfer_dlist_clear(probe))
    ok(c.nixl_capi_xfer_dlist_add_desc(probe, ctypes.c_size_t(second.ctypes.data), ctypes.c_size_t(4096), ctypes.c_uint64(0)))
    assert c.nixl_capi_check_remote_md(d, b"capi3_b", probe) != 0  # not told yet
    ok(c.nixl_capi_get_local_partial_md(b, r2, ctypes.byref(md), ctypes.byref(mdlen), None))
    ok(c.nixl_capi_load_remote_md(d, md, mdlen, ctypes.byref(name)))
    assert c.nixl_capi_check_remote_md(d, b"capi3_b", probe) == 0
    ok(c.nixl_capi_destroy_xfer_dlist(probe))
    for r in (r1, r2):
        ok(c.nixl_capi_deregister_mem(b, r, None))
        ok(c.nixl_capi_destroy_reg_dlist(r))
    for h in (bb, bd):
        ok(c.nixl_capi_destroy_backend(h))
    for h in (b, d):
        ok(c.nixl_capi_destroy_agent(h))


class _AgentConfig(ctypes.Structure):
    _fields_ = [("enable_prog_thread", ctypes.c_bool), ("enable_listen_thread", ctypes.c_bool), ("listen_port", ctypes.c_int),
                ("thread_sync", ctypes.c_int), ("num_workers", ctypes.c_uint), ("pthr_delay_us", ctypes.c_uint64),
                ("lthr_delay_us", ctypes.c_uint64), ("capture_telemetry", ctypes.c_bool)]


class _Telemetry(ctypes.Structure):
    _fields_ = [("start_time_us", ctypes.c_uint64), ("post_duration_us", ctypes.c_uint64), ("xfer_duration_us", ctypes.c_uint64),
                ("total_bytes", ctypes.c_uint64), ("desc_count", ctypes.c_uint64)]


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_capi_list_editing_remote_lists_and_memory_views():
    """The editing calls of both descriptor-list kinds, the remote list, and the memory-view calls (which need a GPU
    backend: on a host-only agent they must answer with an error, not crash)."""
    for kind in ("xfer", "reg"):
        f = lambda name: getattr(c, f"nixl_capi_{kind}_dlist_{name}")  # noqa: E731
        dl = VP()
        ok(getattr(c, f"nixl_capi_create_{kind}_dlist")(0, ctypes.byref(dl)))
        empty, n, mt = ctypes.c_bool(), ctypes.c_size_t(), ctypes.c_int(-1)
        ok(f("is_empty")(dl, ctypes.byref(empty)))
        ok(f("get_type")(dl, ctypes.byref(mt)))
        assert empty.value and mt.value == 0
        for i in range(5):
            if kind == "xfer":
                ok(f("add_desc")(dl, ctypes.c_size_t(0x1000 * (i + 1)), ctypes.c_size_t(256), ctypes.c_uint64(0)))
            else:
                ok(f("add_desc")(dl, ctypes.c_size_t(0x1000 * (i + 1)), ctypes.c_size_t(256), ctypes.c_uint64(0), b"m", ctypes.c_size_t(1)))
        ok(f("desc_count")(dl, ctypes.byref(n)))
        assert n.value == 5
        ok(f("rem_desc")(dl, 1))
        assert f("rem_desc")(dl, 17) != 0  # no such index
        ok(f("desc_count")(dl, ctypes.byref(n)))
        assert n.value == 4
        ok(f("resize")(dl, ctypes.c_size_t(6)))  # grows with empty descriptors
        ok(f("desc_count")(dl, ctypes.byref(n)))
        assert n.value == 6
        ok(f("trim")(dl))  # drops what is beyond address, length and device; the entries stay
        ok(f("desc_count")(dl, ctypes.byref(n)))
        assert n.value == 6
        ok(f("resize")(dl, ctypes.c_size_t(4)))
        ok(f("desc_count")(dl, ctypes.byref(n)))
        assert n.value == 4
        ok(f("print")(dl))
        ok(f("clear")(dl))
        ok(f("is_empty")(dl, ctypes.byref(empty)))
        assert empty.value
        ok(getattr(c, f"nixl_capi_destroy_{kind}_dlist")(dl))

    a, ba = _agent(b"capi4_a")
    buf = np.zeros(4096, dtype=np.uint8)
    reg = _register(a, buf)
    local, remote, view = VP(), VP(), VP()
    ok(c.nixl_capi_create_xfer_dlist(0, ctypes.byref(local)))
    ok(c.nixl_capi_xfer_dlist_add_desc(local, ctypes.c_size_t(buf.ctypes.data), ctypes.c_size_t(4096), ctypes.c_uint64(0)))
    ok(c.nixl_capi_create_remote_dlist(0, ctypes.byref(remote)))
    ok(c.nixl_capi_remote_dlist_add_desc(remote, ctypes.c_size_t(buf.ctypes.data), ctypes.c_size_t(4096), ctypes.c_uint64(0), b"capi4_a"))
    assert c.nixl_capi_remote_dlist_add_desc(remote, ctypes.c_size_t(0), ctypes.c_size_t(1), ctypes.c_uint64(0), None) != 0
    rc = c.nixl_capi_prep_mem_view_local(a, local, ctypes.byref(view), None)
    if rc == 0:  # a GPU is present: the view exists and can be released
        ok(c.nixl_capi_release_mem_view(a, view))
        ok(c.nixl_capi_prep_mem_view_remote(a, remote, ctypes.byref(view), None))
        ok(c.nixl_capi_release_mem_view(a, view))
    else:
        assert c.nixl_capi_prep_mem_view_remote(a, remote, ctypes.byref(view), None) != 0
    assert c.nixl_capi_release_mem_view(a, None) != 0
    ok(c.nixl_capi_destroy_remote_dlist(remote))
    ok(c.nixl_capi_destroy_xfer_dlist(local))
    ok(c.nixl_capi_deregister_mem(a, reg, None))
    ok(c.nixl_capi_destroy_reg_dlist(reg))
    ok(c.nixl_capi_destroy_backend(ba))
    ok(c.nixl_capi_destroy_agent(a))


def test_capi_configured_agents_exchange_metadata_over_the_socket_and_report_telemetry():
    """Agents built from a configuration block (listener thread, telemetry capture): metadata pushed and fetched
    through the peer-to-peer socket, per-request telemetry, and the invalidation of what was pushed."""
    os.environ["NIXL_TELEMETRY_ENABLE"] = "y"
    try:
        port_a, port_b = _free_port(), _free_port()
        agents = []
        for name, port in ((b"capi5_a", port_a), (b"capi5_b", port_b)):
            cfg = _AgentConfig(False, True, port, 2, 1, 0, 1000, True)
            h, params, mems, bh = VP(), VP(), VP(), VP()
            ok(c.nixl_capi_create_configured_agent(name, ctypes.byref(cfg), ctypes.byref(h)))
            ok(c.nixl_capi_get_plugin_params(h, b"NVLINK", ctypes.byref(mems), ctypes.byref(params)))
            ok(c.nixl_capi_create_backend(h, b"NVLINK", params, ctypes.byref(bh)))
            ok(c.nixl_capi_destroy_params(params))
            ok(c.nixl_capi_destroy_mem_list(mems))
            agents.append((h, bh))
        (a, ba), (b, bb) = agents
        assert c.nixl_capi_create_configured_agent(b"nobody", None, ctypes.byref(VP())) != 0
        mine = np.arange(8192, dtype=np.uint8)
        theirs = np.zeros(8192, dtype=np.uint8)
        reg_a, reg_b = _register(a, mine), _register(b, theirs)

        to_b, to_a = VP(), VP()
        ok(c.nixl_capi_create_opt_args(ctypes.byref(to_b)))
        ok(c.nixl_capi_opt_args_set_ip_addr(to_b, b"127.0.0.1"))
        ok(c.nixl_capi_opt_args_set_port(to_b, ctypes.c_uint16(port_b)))
        ok(c.nixl_capi_create_opt_args(ctypes.byref(to_a)))
        ok(c.nixl_capi_opt_args_set_ip_addr(to_a, b"127.0.0.1"))
        ok(c.nixl_capi_opt_args_set_port(to_a, ctypes.c_uint16(port_a)))

        def loaded(agent, name):
            for _ in range(2000):
                if c.nixl_capi_check_remote_md(agent, name, None) == 0:
                    return True
                import time
                time.sleep(0.005)
            return False

        ok(c.nixl_capi_send_local_md(b, to_a))            # b pushes its metadata to a's listener
        assert loaded(a, b"capi5_b")
        ok(c.nixl_capi_fetch_remote_md(b, b"capi5_a", to_a))  # b asks a's listener for a's metadata
        assert loaded(b, b"capi5_a")

        local, remote, req = VP(), VP(), VP()
        ok(c.nixl_capi_create_xfer_dlist(0, ctypes.byref(local)))
        ok(c.nixl_capi_create_xfer_dlist(0, ctypes.byref(remote)))
        for i in range(2):
            ok(c.nixl_capi_xfer_dlist_add_desc(local, ctypes.c_size_t(mine.ctypes.data + i * 4096), ctypes.c_size_t(4096), ctypes.c_uint64(0)))
            ok(c.nixl_capi_xfer_dlist_add_desc(remote, ctypes.c_size_t(theirs.ctypes.data + (1 - i) * 4096), ctypes.c_size_t(4096), ctypes.c_uint64(0)))
        ok(c.nixl_capi_create_xfer_req(a, 1, local, remote, b"capi5_b", ctypes.byref(req), None))  # WRITE
        rc = c.nixl_capi_post_xfer_req(a, req, None)
        while rc == 1:
            rc = c.nixl_capi_get_xfer_status(a, req)
        assert rc == 0
        assert (theirs[4096:] == mine[:4096]).all() and (theirs[:4096] == mine[4096:]).all()
        t = _Telemetry()
        ok(c.nixl_capi_get_xfer_telemetry(a, req, ctypes.byref(t)))
        assert t.total_bytes == 8192 and t.desc_count == 2 and t.start_time_us > 0
        assert c.nixl_capi_get_xfer_telemetry(a, req, None) != 0
        ok(c.nixl_capi_release_xfer_req(a, req))
        ok(c.nixl_capi_destroy_xfer_req(req))

        # a later registration travels as partial metadata; then b withdraws what it pushed
        extra = np.zeros(4096, dtype=np.uint8)
        reg_x = _register(b, extra)
        ok(c.nixl_capi_send_local_partial_md(b, reg_x, to_a))
        probe = VP()
        ok(c.nixl_capi_create_xfer_dlist(0, ctypes.byref(probe)))
        ok(c.nixl_capi_xfer_dlist_add_desc(probe, ctypes.c_size_t(extra.ctypes.data), ctypes.c_size_t(4096), ctypes.c_uint64(0)))
        for _ in range(2000):
            if c.nixl_capi_check_remote_md(a, b"capi5_b", probe) == 0:
                break
            import time
            time.sleep(0.005)
        assert c.nixl_capi_check_remote_md(a, b"capi5_b", probe) == 0
        ok(c.nixl_capi_invalidate_local_md(b, to_a))
        for _ in range(2000):
            if c.nixl_capi_check_remote_md(a, b"capi5_b", None) != 0:
                break
            import time
            time.sleep(0.005)
        assert c.nixl_capi_check_remote_md(a, b"capi5_b", None) != 0  # a forgot b

        ok(c.nixl_capi_destroy_xfer_dlist(probe))
        ok(c.nixl_capi_destroy_xfer_dlist(local))
        ok(c.nixl_capi_destroy_xfer_dlist(remote))
        ok(c.nixl_capi_destroy_opt_args(to_a))
        ok(c.nixl_capi_destroy_opt_args(to_b))
        for agent, reg in ((a, reg_a), (b, reg_b), (b, reg_x)):
            ok(c.nixl_capi_deregister_mem(agent, reg, None))
            ok(c.nixl_capi_destroy_reg_dlist(reg))
        for h in (ba, bb):
            ok(c.nixl_capi_destroy_backend(h))
        for h in (a, b):
            ok(c.nixl_capi_destroy_agent(h))
    finally:
        os.environ.pop("NIXL_TELEMETRY_ENABLE", None)


def test_every_function_of_the_header_is_exported_and_exercised():
    import re

    header = open(os.path.join(os.path.dirname(LIB), "..", "..", "csrc", "include", "nixl_capi.h")).read()
    names = sorted(set(re.findall(r"\b(nixl_capi_[a-z0-9_]+)\s*\(", header)))
    assert len(names) >= 100
    assert [n for n in names if not hasattr(c, n)] == []
    me = open(__file__).read()
    def touched(name):
        if name in me:
            return True
        m = re.fullmatch(r"nixl_capi_(?:xfer|reg)_dlist_([a-z_]+)", name)  # the editing calls are looked up as f("<op>") for both kinds
        return bool(m) and f'f("{m.group(1)}")' in me

    untouched = [n for n in names if not touched(n)]
    assert untouched == [], untouched

"""Python API on CPU: two agents in one process, torch CPU tensors, notifications,
descriptor helpers, metadata helpers.  Mirrors the reference's test/python/test_nixl_api.py
and examples/python/basic_two_peers.py scenarios."""
import pickle

import numpy as np
import pytest
import torch

import nixl_b200
from nixl_b200 import _bindings as nb
from nixl_b200 import nixl_agent, nixl_agent_config


def _wait(agent, handle, limit=200000):
    for _ in range(limit):
        state = agent.check_xfer_state(handle)
        if state != "PROC":
            return state
    return "TIMEOUT"


@pytest.fixture
def pair():
    a = nixl_agent("py_a", nixl_agent_config(enable_prog_thread=False))
    b = nixl_agent("py_b", nixl_agent_config(enable_prog_thread=True))
    yield a, b
    del a, b


def test_plugins_visible(pair):
    a, _ = pair
    assert "NVLINK" in a.get_plugin_list() and "POSIX" in a.get_plugin_list()
    assert set(a.get_plugin_mem_types("NVLINK")) == {"DRAM_SEG", "VRAM_SEG"}
    assert "copy_path" in a.get_plugin_params("NVLINK")
    assert "UCX" in a.backends  # default backend name resolves to the NVLink backend
    assert a.get_backend_mem_types("UCX") == ["DRAM_SEG", "VRAM_SEG"]


def test_descriptor_helpers(pair):
    a, _ = pair
    t = torch.arange(1024, dtype=torch.float32)
    xl = a.get_xfer_descs(t)
    assert len(xl) == 1 and xl[0] == (t.data_ptr(), 4096, 0)
    arr = np.array([[4096, 128, 0], [8192, 256, 1]], dtype=np.uint64)
    xa = a.get_xfer_descs(arr, "DRAM")
    assert xa[1] == (8192, 256, 1) and xa.totalBytes() == 384
    assert (xa.to_array() == arr).all()
    rl = a.get_reg_descs([(4096, 128, 0, "meta")], "FILE")
    assert rl[0][3] == b"meta" and rl.getType() == nb.FILE_SEG
    again = pickle.loads(pickle.dumps(xa))
    assert again == xa
    again_r = a.deserialize_descs(a.get_serialized_descs(rl))
    assert again_r == rl
    with pytest.raises(ValueError):
        a.get_xfer_descs(t.t().reshape(32, 32).t())  # non-contiguous


def test_write_read_with_notifications(pair):
    a, b = pair
    src = torch.randint(0, 255, (64, 1 << 16), dtype=torch.uint8)
    dst = torch.zeros_like(src)
    reg_a = a.register_memory(src)
    reg_b = b.register_memory(dst)
    name = a.add_remote_agent(b.get_agent_metadata())
    assert name == "py_b"
    assert b.add_remote_agent(a.get_agent_metadata()) == "py_a"
    assert a.check_remote_metadata("py_b", a.get_xfer_descs(dst))

    h = a.initialize_xfer("WRITE", [src[i] for i in range(64)], [dst[i] for i in range(64)], "py_b", b"wr-1")
    assert a.transfer(h) in ("DONE", "PROC")
    assert _wait(a, h) == "DONE"
    assert torch.equal(src, dst)
    for _ in range(10000):
        if b.check_remote_xfer_done("py_a", b"wr-"):
            break
    else:
        pytest.fail("notification never arrived")
    assert a.query_xfer_backend(h) == "UCX"
    dur, margin, method = a.estimate_xfer_cost(h)
    assert dur > 0 and margin > 0 and method == nb.NIXL_COST_ANALYTICAL_BACKEND
    a.release_xfer_handle(h)

    dst.add_(1)
    h = a.initialize_xfer("READ", src, dst, "py_b")
    assert a.transfer(h) in ("DONE", "PROC")
    assert _wait(a, h) == "DONE"
    assert torch.equal(src, dst)
    a.release_xfer_handle(h)

    b.send_notif("py_a", b"ping")
    got = {}
    for _ in range(10000):
        got = a.get_new_notifs()
        if got:
            break
    assert got == {"py_b": [b"ping"]}

    a.remove_remote_agent("py_b")
    with pytest.raises(nb.nixlNotFoundError):
        a.initialize_xfer("WRITE", src, dst, "py_b")
    a.deregister_memory(reg_a)
    b.deregister_memory(reg_b)


def test_prepped_transfers(pair):
    a, b = pair
    src = torch.randint(0, 255, (32, 4096), dtype=torch.uint8)
    dst = torch.zeros_like(src)
    a.register_memory(src)
    b.register_memory(dst)
    a.add_remote_agent(b.get_agent_metadata())
    lside = a.prep_xfer_dlist("NIXL_INIT_AGENT", [src[i] for i in range(32)])
    rside = a.prep_xfer_dlist("py_b", [dst[i] for i in range(32)])
    perm = np.random.default_rng(0).permutation(32).astype(np.int32)
    h = a.make_prepped_xfer("WRITE", lside, list(range(32)), rside, perm, b"prepped")
    assert a.transfer(h) in ("DONE", "PROC")
    assert _wait(a, h) == "DONE"
    for i in range(32):
        assert torch.equal(src[i], dst[perm[i]])
    a.release_xfer_handle(h)
    with pytest.raises(nb.nixlInvalidParamError):
        a.make_prepped_xfer("WRITE", lside, [0, 1], rside, [0])
    a.release_dlist_handle(lside)
    a.release_dlist_handle(rside)


def test_error_types():
    a = nixl_agent("py_err", nixl_agent_config(backends=[]))
    with pytest.raises(nb.nixlNotFoundError):
        a.create_backend("NO_SUCH_BACKEND")
    with pytest.raises(nb.nixlInvalidParamError):
        a.get_agent_metadata()  # no backend that supports remote access
    assert issubclass(nb.nixlNotFoundError, nb.nixlError)
    assert nixl_b200.__version__


def test_python_logging_follows_nixl_log_level(monkeypatch, capsys):
    import logging

    from nixl_b200 import logging as nlog

    monkeypatch.setenv("NIXL_LOG_LEVEL", "warn")
    root = nlog.setup_logging(force=True)
    assert root.level == logging.WARNING
    log = nlog.get_logger("tests.sample")
    assert log.name == "nixl.tests.sample" and not log.isEnabledFor(logging.INFO) and log.isEnabledFor(logging.ERROR)
    monkeypatch.setenv("NIXL_LOG_LEVEL", "TRACE")
    assert nlog.level_from_env() == logging.DEBUG
    monkeypatch.setenv("NIXL_LOG_LEVEL", "chatty")
    with pytest.raises(ValueError):
        nlog.level_from_env()
    root = nlog.setup_logging(force=True)  # falls back to INFO and says so
    assert root.level == logging.INFO
    monkeypatch.delenv("NIXL_LOG_LEVEL")
    nlog.setup_logging(force=True)


def test_handles_own_their_native_objects():
    import gc

    import torch

    from nixl_b200 import nixl_agent, nixl_agent_config
    from nixl_b200._api import nixl_prepped_dlist_handle, nixl_xfer_handle

    a = nixl_agent("own_a", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
    b = nixl_agent("own_b", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
    src, dst = torch.arange(1024, dtype=torch.uint8), torch.zeros(1024, dtype=torch.uint8)
    a.register_memory(src)
    b.register_memory(dst)
    a.add_remote_agent(b.get_agent_metadata())
    h = a.initialize_xfer("WRITE", src, dst, "own_b")
    assert isinstance(h, nixl_xfer_handle) and isinstance(h, int) and "released=False" in repr(h)
    assert a.transfer(h) in ("DONE", "PROC")
    while a.check_xfer_state(h) == "PROC":
        pass
    assert torch.equal(src, dst)
    h.release()
    h.release()  # idempotent
    a.release_xfer_handle(h)  # also fine after release()
    assert "released=True" in repr(h)
    # prepared lists: wrapper in, wrapper out; dropping the last reference frees them
    side_l = a.prep_xfer_dlist("NIXL_INIT_AGENT", src)
    side_r = a.prep_xfer_dlist("own_b", dst)
    assert isinstance(side_l, nixl_prepped_dlist_handle)
    h2 = a.make_prepped_xfer("WRITE", side_l, [0], side_r, [0])
    assert a.transfer(h2) in ("DONE", "PROC")
    while a.check_xfer_state(h2) == "PROC":
        pass
    del h2
    gc.collect()
    a.release_dlist_handle(side_l)
    del side_r
    gc.collect()


def test_raw_buffer_helpers_move_through_an_agent():
    from nixl_b200 import _utils, nixl_agent, nixl_agent_config

    n = 10000
    a, b = _utils.malloc_passthru(n), _utils.malloc_passthru(n)
    assert a % 4096 == 0 and b % 4096 == 0
    try:
        _utils.ba_buf(a, n)
        import ctypes

        ctypes.memset(b, 0, n)
        with pytest.raises(AssertionError):
            _utils.verify_transfer(a, b, n)
        src = nixl_agent("raw_src", nixl_agent_config(backends=["NVLINK"]))
        dst = nixl_agent("raw_dst", nixl_agent_config(backends=["NVLINK"]))
        reg_a = src.register_memory([(a, n, 0, "")], "DRAM")
        reg_b = dst.register_memory([(b, n, 0, "")], "DRAM")
        src.add_remote_agent(dst.get_agent_metadata())
        h = src.initialize_xfer("WRITE", src.get_xfer_descs([(a, n, 0)], "DRAM"), src.get_xfer_descs([(b, n, 0)], "DRAM"), "raw_dst")
        state = src.transfer(h)
        while state == "PROC":
            state = src.check_xfer_state(h)
        assert state == "DONE"
        _utils.verify_transfer(a, b, n)
        src.release_xfer_handle(h)
        src.deregister_memory(reg_a)
        dst.deregister_memory(reg_b)
    finally:
        _utils.free_passthru(a)
        _utils.free_passthru(b)


def test_reference_import_names_resolve_to_this_package():
    import nixl
    import nixl._bindings as bindings
    import nixl_ep
    from nixl._api import nixl_agent, nixl_agent_config
    from nixl.logging import get_logger

    assert nixl_agent is nixl_b200.nixl_agent and nixl_agent_config is nixl_b200.nixl_agent_config
    assert bindings is nixl_b200._bindings and hasattr(bindings, "nixlAgent")
    assert nixl.nixl_agent is nixl_agent and callable(get_logger)
    assert nixl_ep.Buffer is nixl_b200.parallel.Buffer and hasattr(nixl_ep, "EventOverlap")
    agent = nixl_agent("via_reference_names", nixl_agent_config(backends=[]))
    assert "NVLINK" in agent.get_plugin_list()


def test_utils_package_reads_measured_peaks(tmp_path):
    from nixl_b200 import utils

    peaks = tmp_path / "peaks.json"
    peaks.write_text('{"hbm_gbs": 6547.2, "bf16_tflops": 1641.0}')
    assert utils.measured_peaks(str(peaks))["hbm_gbs"] == 6547.2
    assert utils.measured_peaks(str(tmp_path / "absent.json")) == {}
    peaks.write_text("not json")
    assert utils.measured_peaks(str(peaks)) == {}
    assert utils.malloc_passthru is not None and utils.verify_transfer is not None


def test_agent_has_every_public_method_of_the_reference_wrapper():
    """The method names of the reference's ``nixl_agent`` (src/api/python/_api.py), as a fixed list."""
    from nixl_b200 import nixl_agent

    expected = """add_remote_agent check_remote_metadata check_remote_xfer_done check_xfer_state create_backend deregister_memory
    deserialize_descs estimate_xfer_cost fetch_remote_metadata get_agent_metadata get_backend_mem_types get_backend_params
    get_new_notifs get_partial_agent_metadata get_plugin_list get_plugin_mem_types get_plugin_params get_reg_descs
    get_remote_descs get_serialized_descs get_xfer_descs get_xfer_telemetry initialize_xfer invalidate_local_metadata
    make_connection make_prepped_xfer prep_mem_view prep_xfer_dlist query_memory query_xfer_backend register_memory
    release_dlist_handle release_mem_view release_xfer_handle remove_remote_agent send_local_metadata send_notif
    send_partial_agent_metadata transfer update_notifs""".split()
    assert len(expected) == 40
    missing = [name for name in expected if not callable(getattr(nixl_agent, name, None))]
    assert missing == []


def test_ep_buffer_has_every_public_method_of_the_reference_buffer():
    """The method names of the reference's ``nixl_ep.Buffer`` (examples/device/ep/nixl_ep/buffer.py), as a fixed list."""
    from nixl_b200.parallel import Buffer

    expected = """barrier capture clean_mask_buffer combine connect_ranks destroy disconnect_ranks dispatch get_combine_config
    get_comm_stream get_dispatch_config get_dispatch_layout get_local_buffer_tensor get_low_latency_buffer_size_hint
    get_next_combine_buffer get_rdma_size_hint ht_combine ht_dispatch is_sm90_compiled low_latency_combine low_latency_dispatch
    query_mask_buffer set_num_sms set_tcp_store_group update_mask_buffer update_memory_buffers""".split()
    assert len(expected) == 26
    assert [name for name in expected if not hasattr(Buffer, name)] == []
    assert Buffer.is_sm90_compiled() is True
    import nixl_ep

    assert nixl_ep.Buffer is Buffer


def test_interpreter_exit_with_unreleased_handles_is_clean():
    """Handles, registration descriptors and agents left alive at exit are collected in arbitrary order while module
    globals disappear; a transfer handle must be released exactly once whatever that order is."""
    import os
    import subprocess
    import sys
    import textwrap

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = textwrap.dedent("""
        import numpy as np, nixl_b200, os
        from nixl._api import nixl_agent, nixl_agent_config
        cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"])
        a, b = nixl_agent("exit_a", cfg), nixl_agent("exit_b", cfg)
        src = np.arange(65536, dtype=np.uint8); dst = np.zeros_like(src)
        ra = a.register_memory([(src.ctypes.data, src.nbytes, 0, "")], "DRAM")
        rb = b.register_memory([(dst.ctypes.data, dst.nbytes, 0, "")], "DRAM")
        a.add_remote_agent(b.get_agent_metadata())
        hs = []
        for i in range(3):
            h = a.initialize_xfer("WRITE", a.get_xfer_descs([(src.ctypes.data, src.nbytes, 0)], "DRAM"),
                                  a.get_xfer_descs([(dst.ctypes.data, dst.nbytes, 0)], "DRAM"), "exit_b", b"hi")
            st = a.transfer(h)
            while st == "PROC":
                st = a.check_xfer_state(h)
            hs.append(h)
        side = a.prep_xfer_dlist("NIXL_INIT_AGENT", [(src.ctypes.data, 4096, 0)], "DRAM")
        assert (src == dst).all()
        print("ok")
    """)
    for _ in range(3):
        res = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, cwd="/", env={**os.environ, "PYTHONPATH": root})
        assert res.returncode == 0 and res.stdout.strip() == "ok", (res.returncode, res.stderr[-500:])


def test_released_handles_are_refused_in_python(pair):
    """A handle object remembers that it was released: using it again raises instead of handing a dangling native
    pointer to the library."""
    a, b = pair
    src, dst = np.arange(8192, dtype=np.uint8), np.zeros(8192, dtype=np.uint8)
    a.register_memory([(src.ctypes.data, src.nbytes, 0, "")], "DRAM")
    b.register_memory([(dst.ctypes.data, dst.nbytes, 0, "")], "DRAM")
    a.add_remote_agent(b.get_agent_metadata())
    h = a.initialize_xfer("WRITE", a.get_xfer_descs([(src.ctypes.data, 4096, 0)], "DRAM"), a.get_xfer_descs([(dst.ctypes.data, 4096, 0)], "DRAM"), b.name)
    assert a.transfer(h) in ("DONE", "PROC")
    assert _wait(a, h) == "DONE"
    a.release_xfer_handle(h)
    a.release_xfer_handle(h)  # releasing twice is harmless
    assert a.transfer(h) == "ERR" and a.check_xfer_state(h) == "ERR"  # refused before anything native runs
    for call in (lambda: a.estimate_xfer_cost(h), lambda: a.query_xfer_backend(h), lambda: a.get_xfer_telemetry(h)):
        with pytest.raises(nixl_b200._bindings.nixlInvalidParamError):
            call()
    side_l = a.prep_xfer_dlist("NIXL_INIT_AGENT", [(src.ctypes.data, 4096, 0)], "DRAM")
    side_r = a.prep_xfer_dlist(b.name, [(dst.ctypes.data, 4096, 0)], "DRAM")
    a.release_dlist_handle(side_r)
    with pytest.raises(nixl_b200._bindings.nixlInvalidParamError):
        a.make_prepped_xfer("WRITE", side_l, [0], side_r, [0])
    a.release_dlist_handle(side_l)


def test_pci_topology_of_a_made_up_tree(tmp_path):
    """`nixl_b200.utils.pci_topology`: a GPU and a NIC under one switch, a second NIC under the chipset."""
    from nixl_b200.utils import pci_topology

    bus = tmp_path / "bus"
    bus.mkdir()

    def add(chain, vendor, cls, numa, ifs=()):
        d = tmp_path / "devices" / chain
        d.mkdir(parents=True)
        (d / "vendor").write_text(vendor + "\n")
        (d / "class").write_text(cls + "\n")
        (d / "device").write_text("0x2901\n")
        (d / "numa_node").write_text(f"{numa}\n")
        for i in ifs:
            (d / "net" / i).mkdir(parents=True)
        (bus / chain.rsplit("/", 1)[-1]).symlink_to(d)

    add("pci0000:15/0000:15:01.0/0000:16:00.0/0000:17:00.0/0000:1b:00.0", "0x10de", "0x030200", 0)
    add("pci0000:15/0000:15:01.0/0000:16:00.0/0000:17:01.0/0000:1c:00.0", "0x15b3", "0x020700", 0, ["ib0"])
    add("pci0000:00/0000:00:1f.0/0000:02:00.0", "0x8086", "0x020000", 0, ["eno1"])
    topo = pci_topology(str(bus))
    assert [g["bdf"] for g in topo["gpus"]] == ["0000:1b:00.0"] and topo["gpus"][0]["chain"][0] == "pci0000:15"
    assert [n["interfaces"] for n in topo["nics"]] == [["eno1"], ["ib0"]]
    near = topo["nics_near_gpu"][0]
    assert [n["interfaces"] for n in near] == [["ib0"], ["eno1"]] and near[0]["distance"] == 4 and near[1]["distance"] > 100
    assert "gpu0 0000:1b:00.0" in topo["text"]
    assert pci_topology(str(tmp_path / "absent")) == {"gpus": [], "nics": [], "nics_near_gpu": [], "text": ""}

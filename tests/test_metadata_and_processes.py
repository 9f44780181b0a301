"""Metadata exchange through a torch TCPStore and a two-process transfer on 127.0.0.1.

Mirrors the reference's test/gtest/md_manager.cpp (TCPStore fixture) and test/nixl/nixl_test.cpp
(target / initiator processes).  The two-process case moves DRAM between processes (the
NVLink backend's cross-process DRAM path) and checks the completion notification; it needs
permission to read another process's memory, which a default container grants to children of
the same user - the test skips otherwise."""
import datetime
import multiprocessing as mp
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_tcpstore_metadata_roundtrip(monkeypatch):
    port = _free_port()
    store = dist.TCPStore("127.0.0.1", port, is_master=True, wait_for_workers=False, timeout=datetime.timedelta(seconds=20))
    monkeypatch.setenv("NIXL_TCPSTORE_ENDPOINT", f"127.0.0.1:{port}")
    monkeypatch.setenv("NIXL_TCPSTORE_TIMEOUT_MS", "5000")
    from nixl_b200 import nixl_agent, nixl_agent_config

    a = nixl_agent("store_a", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
    b = nixl_agent("store_b", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
    ta, tb = torch.arange(4096, dtype=torch.uint8), torch.zeros(4096, dtype=torch.uint8)
    a.register_memory(ta)
    b.register_memory(tb)
    a.send_local_metadata()  # publishes under nixl/agents/metadata/store_a/NULL_AGENT
    b.send_local_metadata()
    b.fetch_remote_metadata("store_a")
    a.fetch_remote_metadata("store_b")
    deadline = time.time() + 10
    while time.time() < deadline and not (a.check_remote_metadata("store_b") and b.check_remote_metadata("store_a")):
        time.sleep(0.01)
    assert a.check_remote_metadata("store_b", a.get_xfer_descs(tb))
    # the key is visible to a plain torch client under the documented name
    assert store.check(["nixl/agents/metadata/store_a/NULL_AGENT"])
    h = a.initialize_xfer("WRITE", ta, tb, "store_b")
    assert a.transfer(h) in ("DONE", "PROC")
    while a.check_xfer_state(h) == "PROC":
        pass
    assert torch.equal(ta, tb)
    a.release_xfer_handle(h)
    a.invalidate_local_metadata()
    deadline = time.time() + 5
    while time.time() < deadline and store.check(["nixl/agents/metadata/store_a/NULL_AGENT"]):
        time.sleep(0.01)
    assert not store.check(["nixl/agents/metadata/store_a/NULL_AGENT"])
    del a, b


def _target(port_t, port_i, ready, result):
    from nixl_b200 import nixl_agent, nixl_agent_config

    agent = nixl_agent("target", nixl_agent_config(enable_prog_thread=False, enable_listen_thread=True, listen_port=port_t, backends=["NVLINK"]))
    buf = torch.zeros(1 << 20, dtype=torch.uint8)
    agent.register_memory(buf)
    result["addr"] = buf.data_ptr()
    ready.set()
    deadline = time.time() + 30
    while time.time() < deadline:
        if agent.check_remote_xfer_done("initiator", b"written"):
            result["sum"] = int(buf.to(torch.int64).sum())
            result["ok"] = True
            # answer so the initiator can also test the reverse direction of notifications
            agent.send_notif("initiator", b"thanks")
            time.sleep(0.2)
            return
        time.sleep(0.001)
    result["ok"] = False


def test_two_processes_over_localhost():
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    result = mgr.dict()
    ready = ctx.Event()
    port_t, port_i = _free_port(), _free_port()
    proc = ctx.Process(target=_target, args=(port_t, port_i, ready, result))
    proc.start()
    try:
        assert ready.wait(60)
        from nixl_b200 import _bindings as nb
        from nixl_b200 import nixl_agent, nixl_agent_config

        agent = nixl_agent("initiator", nixl_agent_config(enable_prog_thread=False, enable_listen_thread=True, listen_port=port_i, backends=["NVLINK"]))
        src = torch.randint(0, 255, (1 << 20,), dtype=torch.uint8)
        agent.register_memory(src)
        agent.fetch_remote_metadata("target", "127.0.0.1", port_t)
        agent.send_local_metadata("127.0.0.1", port_t)
        deadline = time.time() + 20
        while time.time() < deadline and not agent.check_remote_metadata("target"):
            time.sleep(0.005)
        assert agent.check_remote_metadata("target")
        remote = agent.get_xfer_descs([(result["addr"], 1 << 20, 0)], "DRAM")
        h = agent.initialize_xfer("WRITE", src, remote, "target", b"written")
        try:
            state = agent.agent.postXferReq(h)
        except nb.nixlBackendError:
            pytest.skip("cross-process memory access (process_vm_writev) is not permitted here")
        while state != nb.NIXL_SUCCESS:
            state = agent.agent.getXferStatus(h)
        proc.join(40)
        assert result.get("ok") is True
        assert result["sum"] == int(src.to(torch.int64).sum())
        got = {}
        deadline = time.time() + 5
        while time.time() < deadline and not got:
            got = agent.get_new_notifs()
        assert got == {"target": [b"thanks"]}
        # the target process is gone now: the next post must report it, not hang
        time.sleep(0.1)
        with pytest.raises(nb.nixlRemoteDisconnectError):
            agent.agent.postXferReq(h)
    finally:
        if proc.is_alive():
            proc.terminate()
        proc.join(5)


def _start_fake_etcd(*flags):
    """The fake gateway runs in its own process: the agent's constructor probes the endpoint from
    inside a native call, during which a server thread of this interpreter could not run."""
    import subprocess
    import sys

    proc = subprocess.Popen([sys.executable, os.path.join(os.path.dirname(os.path.abspath(__file__)), "fake_etcd_gateway.py"), *flags],
                            stdout=subprocess.PIPE, text=True)
    port = int(proc.stdout.readline())
    return proc, port


def _etcd_keys(port):
    import json
    import urllib.request

    return json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/keys", timeout=5).read())


@pytest.mark.parametrize("watch", [True, False], ids=["watch-stream", "poll-only"])
def test_etcd_gateway_metadata_roundtrip_and_invalidation(monkeypatch, watch):
    """With a watch stream the DELETE event invalidates the peer at once (the poll interval is set far beyond the
    test's patience, so only the stream can do it); a gateway without the endpoint is polled."""
    proc, port = _start_fake_etcd(*([] if watch else ["--no-watch"]))
    monkeypatch.delenv("NIXL_TCPSTORE_ENDPOINT", raising=False)
    monkeypatch.setenv("NIXL_ETCD_ENDPOINTS", f"http://127.0.0.1:1,http://127.0.0.1:{port}")  # the first endpoint is dead
    monkeypatch.setenv("NIXL_ETCD_POLL_MS", "60000" if watch else "50")
    from nixl_b200 import nixl_agent, nixl_agent_config

    try:
        a = nixl_agent("etcd_a", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
        b = nixl_agent("etcd_b", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
        ta, tb = torch.arange(8192, dtype=torch.uint8), torch.zeros(8192, dtype=torch.uint8)
        a.register_memory(ta)
        b.register_memory(tb)
        b.fetch_remote_metadata("etcd_a")  # asked for before it exists: the fetch waits for the key
        time.sleep(0.2)
        a.send_local_metadata()
        b.send_local_metadata()
        a.fetch_remote_metadata("etcd_b")
        deadline = time.time() + 10
        while time.time() < deadline and not (a.check_remote_metadata("etcd_b") and b.check_remote_metadata("etcd_a")):
            time.sleep(0.01)
        assert a.check_remote_metadata("etcd_b") and b.check_remote_metadata("etcd_a")
        assert "/nixl/agents/etcd_a/metadata" in _etcd_keys(port)  # documented key layout: <namespace>/<agent>/<label>
        import json
        import urllib.request

        streams = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/watchers", timeout=5).read())
        assert streams == (2 if watch else 0)  # one stream per agent
        h = a.initialize_xfer("WRITE", ta, tb, "etcd_b")
        assert a.transfer(h) in ("DONE", "PROC")
        while a.check_xfer_state(h) == "PROC":
            pass
        assert torch.equal(ta, tb)
        a.release_xfer_handle(h)
        # a withdraws its metadata: its key disappears and b, which watches what it fetched, forgets a
        a.invalidate_local_metadata()
        deadline = time.time() + 10
        while time.time() < deadline and ("/nixl/agents/etcd_a/metadata" in _etcd_keys(port) or b.check_remote_metadata("etcd_a")):
            time.sleep(0.02)
        assert "/nixl/agents/etcd_a/metadata" not in _etcd_keys(port)
        assert not b.check_remote_metadata("etcd_a")
        del a, b
    finally:
        proc.terminate()
        proc.wait(timeout=10)


def test_the_metadata_listener_survives_strangers():
    """Anyone who can reach the listener's port can send it bytes: noise, a frame that announces a gigabyte and sends
    none of it, an unknown command, a connection dropped inside a frame.  The agent keeps serving its real peers, and its
    memory does not follow announced lengths."""
    import resource
    import struct

    from nixl_b200 import nixl_agent, nixl_agent_config

    port = _free_port()
    a = nixl_agent("md_victim", nixl_agent_config(enable_prog_thread=False, enable_listen_thread=True, listen_port=port, backends=["NVLINK"]))
    buf = torch.zeros(4096, dtype=torch.uint8)
    a.register_memory(buf)

    def dial():
        s = socket.create_connection(("127.0.0.1", port), timeout=5)
        return s

    before = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss
    socks = []
    for payload in (os.urandom(512), struct.pack("<Q", 1 << 30), struct.pack("<Q", (1 << 30) + 1), struct.pack("<Q", 64) + b"NIXLCOMM:WHAT" + b"x" * 51,
                    struct.pack("<Q", 1000) + b"NIXLCOMM:LOAD" + b"\x00" * 10, struct.pack("<Q", 13) + b"NIXLCOMM:LOAD", b"\x01\x02\x03"):
        s = dial()
        s.sendall(payload)
        socks.append(s)
    for _ in range(8):  # several that announce a gigabyte each and then just sit there
        s = dial()
        s.sendall(struct.pack("<Q", 1 << 30) + b"NIXLCOMM:LOAD")
        socks.append(s)
    time.sleep(0.5)
    for s in socks[::2]:
        s.close()
    grown_kb = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss - before
    assert grown_kb < 512 << 10, grown_kb  # nothing like the announced gigabytes was set aside
    # a real peer is served as if nothing had happened
    b = nixl_agent("md_friend", nixl_agent_config(enable_prog_thread=False, enable_listen_thread=True, listen_port=_free_port(), backends=["NVLINK"]))
    b.fetch_remote_metadata("md_victim", "127.0.0.1", port)
    deadline = time.time() + 20
    while time.time() < deadline and not b.check_remote_metadata("md_victim"):
        time.sleep(0.01)
    assert b.check_remote_metadata("md_victim")
    for s in socks[1::2]:
        s.close()

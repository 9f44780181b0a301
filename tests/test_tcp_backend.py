"""The TCP backend through the Python API: the transport for peers that NVLink does not reach (another host; here the
loopback interface).  Two processes exchange metadata over the agents' listeners, the initiator WRITEs and READs CPU
tensors of the target, a notification follows the data; and an agent that has both backends still reaches a same-host
peer, whichever of the two the agent picks."""
import multiprocessing as mp
import socket
import time

import pytest
import torch


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _target(port_t, backends, ready, go_on, result):
    from nixl_b200 import nixl_agent, nixl_agent_config

    agent = nixl_agent("tcp_py_target", nixl_agent_config(enable_prog_thread=False, enable_listen_thread=True, listen_port=port_t, backends=backends))
    buf = torch.zeros(3 << 20, dtype=torch.uint8)
    agent.register_memory(buf)
    result["addr"] = buf.data_ptr()
    ready.set()
    deadline = time.time() + 30
    while time.time() < deadline:
        if agent.check_remote_xfer_done("tcp_py_initiator", b"written"):
            result["sum"] = int(buf.to(torch.int64).sum())
            buf += 1  # what the initiator reads back
            agent.send_notif("tcp_py_initiator", b"changed")
            result["ok"] = True
            go_on.wait(30)
            return
        time.sleep(0.001)
    result["ok"] = False


@pytest.mark.parametrize("backends", [["TCP"], ["NVLINK", "TCP"]], ids=["tcp-only", "nvlink-and-tcp"])
def test_two_processes_write_read_and_notify_over_sockets(backends):
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    result = mgr.dict()
    ready, go_on = ctx.Event(), ctx.Event()
    port_t, port_i = _free_port(), _free_port()
    proc = ctx.Process(target=_target, args=(port_t, backends, ready, go_on, result))
    proc.start()
    try:
        assert ready.wait(60)
        from nixl_b200 import _bindings as nb
        from nixl_b200 import nixl_agent, nixl_agent_config

        agent = nixl_agent("tcp_py_initiator", nixl_agent_config(enable_prog_thread=False, enable_listen_thread=True, listen_port=port_i, backends=backends))
        assert "TCP" in agent.get_plugin_list()
        mems = agent.get_backend_mem_types("TCP")
        assert "DRAM_SEG" in mems
        src = torch.randint(0, 200, (3 << 20,), dtype=torch.uint8)
        agent.register_memory(src)
        agent.fetch_remote_metadata("tcp_py_target", "127.0.0.1", port_t)
        agent.send_local_metadata("127.0.0.1", port_t)
        deadline = time.time() + 20
        while time.time() < deadline and not agent.check_remote_metadata("tcp_py_target"):
            time.sleep(0.005)
        assert agent.check_remote_metadata("tcp_py_target")
        remote = agent.get_xfer_descs([(result["addr"], 3 << 20, 0)], "DRAM")
        h = agent.initialize_xfer("WRITE", src, remote, "tcp_py_target", b"written")
        if backends == ["TCP"]:
            assert agent.query_xfer_backend(h) == "TCP"
        try:
            state = agent.transfer(h)
        except nb.nixlBackendError:
            pytest.skip("the backend the agent picked cannot reach the other process here")
        deadline = time.time() + 30
        while state == "PROC" and time.time() < deadline:
            state = agent.check_xfer_state(h)
        if state == "ERR" and backends != ["TCP"]:
            pytest.skip("cross-process memory access (process_vm_writev) is not permitted here")
        assert state == "DONE"
        got = {}
        deadline = time.time() + 20
        while time.time() < deadline and not got:
            got = agent.get_new_notifs()
        assert got == {"tcp_py_target": [b"changed"]}
        assert result["sum"] == int(src.to(torch.int64).sum())
        back = torch.zeros_like(src)
        agent.register_memory(back)
        h2 = agent.initialize_xfer("READ", back, remote, "tcp_py_target")
        state = agent.transfer(h2)
        deadline = time.time() + 30
        while state == "PROC" and time.time() < deadline:
            state = agent.check_xfer_state(h2)
        assert state == "DONE"
        assert torch.equal(back, src + 1)
        agent.release_xfer_handle(h)
        agent.release_xfer_handle(h2)
        go_on.set()
        proc.join(40)
        assert result.get("ok") is True
    finally:
        go_on.set()
        if proc.is_alive():
            proc.terminate()
        proc.join(5)

"""The TCP backend through the Python API: the transport for peers that NVLink does not reach (another host; here the
loopback interface).  Two processes exchange metadata over the agents' listeners, the initiator WRITEs and READs CPU
tensors of the target, a notification follows the data; and an agent that has both backends still reaches a same-host
peer, whichever of the two the agent picks."""
import multiprocessing as mp
import os
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


def test_kv_block_mover_checks_what_it_is_given():
    """`KVBlockTransfer` over two agents of one process (TCP backend, loopback): READ as well as WRITE, and the errors a
    caller can make: a block number out of range, lists of different length, a peer whose blocks have another size."""
    from nixl_b200 import nixl_agent, nixl_agent_config
    from nixl_b200.ops import KVBlockTransfer, describe_blocks

    a = nixl_agent("kvb_a", nixl_agent_config(backends=["TCP"]))
    b = nixl_agent("kvb_b", nixl_agent_config(backends=["TCP"]))
    mine = [torch.arange(16 * 512, dtype=torch.float32).reshape(16, 512) + 1000 * i for i in range(3)]
    theirs = [torch.zeros(24, 512, dtype=torch.float32) for _ in range(3)]
    for t in mine:
        a.register_memory(t)
    for t in theirs:
        b.register_memory(t)
    a.add_remote_agent(b.get_agent_metadata())
    mover = KVBlockTransfer(a, mine, "kvb_b", describe_blocks(b, theirs))
    assert mover.blocks == 16 and mover.remote_blocks == 24 and mover.bytes_moved(2) == 2 * 3 * 2048
    mover.wait(mover.post([0, 5, 15], [23, 1, 7], "WRITE", b"three"))
    for i in range(3):
        assert torch.equal(theirs[i][23], mine[i][0]) and torch.equal(theirs[i][1], mine[i][5]) and torch.equal(theirs[i][7], mine[i][15])
        assert float(theirs[i][[0, 2, 3, 22]].abs().sum()) == 0
    deadline = time.time() + 5
    got = {}
    while time.time() < deadline and not got:
        got = b.get_new_notifs()
    assert got == {"kvb_a": [b"three"]}
    theirs[2][9] += 7.0
    mover.wait(mover.post([3], [9], "READ"))
    assert torch.equal(mine[2][3], theirs[2][9]) and float(mine[0][3].abs().sum()) == 0
    with pytest.raises(IndexError):
        mover.post([16], [0])
    with pytest.raises(IndexError):
        mover.post([0], [24])
    with pytest.raises(ValueError):
        mover.post([0, 1], [0])
    other = [torch.zeros(24, 256, dtype=torch.float32) for _ in range(3)]
    for t in other:
        b.register_memory(t)
    with pytest.raises(ValueError):
        KVBlockTransfer(a, mine, "kvb_b", describe_blocks(b, other))
    with pytest.raises(ValueError):
        KVBlockTransfer(a, mine, "kvb_b", describe_blocks(b, theirs[:2] + [theirs[0][:5]]))
    with pytest.raises(ValueError):
        describe_blocks(b, [theirs[0].t()])
    mover.close()


def test_the_agent_takes_nvlink_inside_a_box_and_tcp_across_boxes():
    """Three agents with both backends; the NVLINK engines of two of them are told (``host_id``) that they share a box,
    the third that it sits in another one.  A request to the neighbour runs on NVLINK, a request to the other box on
    TCP, without the caller naming a backend; both move their bytes."""
    from nixl_b200 import nixl_agent, nixl_agent_config

    def make(name, box):
        a = nixl_agent(name, nixl_agent_config(backends=[]))
        a.create_backend("NVLINK", {"host_id": box})
        a.create_backend("TCP", {"address": "127.0.0.1"})
        return a

    here, neighbour, far = make("box_a0", "box-a"), make("box_a1", "box-a"), make("box_b0", "box-b")
    src = torch.arange(1 << 16, dtype=torch.int32)
    near_dst, far_dst = torch.zeros_like(src), torch.zeros_like(src)
    here.register_memory(src)
    neighbour.register_memory(near_dst)
    far.register_memory(far_dst)
    assert here.add_remote_agent(neighbour.get_agent_metadata()) == "box_a1"
    assert here.add_remote_agent(far.get_agent_metadata()) == "box_b0"  # its NVLINK part is refused, its TCP part taken
    for peer, dst, backend in (("box_a1", near_dst, "NVLINK"), ("box_b0", far_dst, "TCP")):
        h = here.initialize_xfer("WRITE", src, dst, peer, b"done")
        assert here.query_xfer_backend(h) == backend
        state = here.transfer(h)
        while state == "PROC":
            state = here.check_xfer_state(h)
        assert state == "DONE" and torch.equal(src, dst)
        here.release_xfer_handle(h)
    deadline = time.time() + 5
    while time.time() < deadline and not far.check_remote_xfer_done("box_a0", b"done"):
        time.sleep(0.001)
    else:
        assert time.time() < deadline
    # naming the backend that cannot reach the peer is an error, not a silent detour
    with pytest.raises(Exception):
        here.initialize_xfer("WRITE", src, far_dst, "box_b0", backends=["NVLINK"])


def test_connecting_ahead_of_time_and_forgetting_a_peer():
    """`make_connection` opens the rails before the first request; `remove_remote_agent` closes them, and a peer that is
    added again is reached again on new ones."""
    from nixl_b200 import nixl_agent, nixl_agent_config

    port = _free_port()
    a = nixl_agent("conn_a", nixl_agent_config(backends=[]))
    b = nixl_agent("conn_b", nixl_agent_config(backends=[]))
    a.create_backend("TCP", {"address": "127.0.0.1", "rails": "3"})
    b.create_backend("TCP", {"address": "127.0.0.1", "rails": "3", "port": str(port)})
    src = torch.arange(4096, dtype=torch.int32)
    dst = torch.zeros_like(src)
    a.register_memory(src)
    b.register_memory(dst)
    meta = b.get_agent_metadata()
    a.add_remote_agent(meta)

    def established_to_peer():
        # the kernel's table: established connections whose far end is conn_b's listener port (the initiator's halves)
        rows = []
        for table in ("/proc/net/tcp", "/proc/net/tcp6"):  # (the second one is absent on a host without IPv6)
            if os.path.exists(table):
                with open(table) as f:
                    rows += [l.split() for l in list(f)[1:]]
        return sum(1 for r in rows if r[3] == "01" and r[2].endswith(":%04X" % port))

    before = established_to_peer()
    assert before == 0
    a.make_connection("conn_b", ["TCP"])
    assert established_to_peer() == 3  # the rails are up before any request
    for _ in range(2):
        h = a.initialize_xfer("WRITE", src, dst, "conn_b")
        state = a.transfer(h)
        while state == "PROC":
            state = a.check_xfer_state(h)
        assert state == "DONE" and torch.equal(src, dst)
        a.release_xfer_handle(h)
        dst.zero_()
    a.remove_remote_agent("conn_b")
    deadline = time.time() + 5
    while time.time() < deadline and established_to_peer() > before:
        time.sleep(0.01)
    assert established_to_peer() <= before  # the rails are gone (the serving ends notice and close)
    with pytest.raises(Exception):
        a.initialize_xfer("WRITE", src, dst, "conn_b")
    a.add_remote_agent(meta)
    h = a.initialize_xfer("WRITE", src, dst, "conn_b")
    state = a.transfer(h)
    while state == "PROC":
        state = a.check_xfer_state(h)
    assert state == "DONE" and torch.equal(src, dst)
    a.release_xfer_handle(h)

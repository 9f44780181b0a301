"""GPU transfers through the public API, checked against plain torch copies.

Scenarios follow the reference's test/gtest/test_transfer.cpp (VRAM and DRAM, WRITE and
READ, notifications, batches) plus what is new here: the table path for large batches,
odd sizes and offsets, the bulk (TMA) copy path and stream-ordered posting."""
import pytest
import torch

from nixl_b200 import _bindings as nb
from nixl_b200 import nixl_agent, nixl_agent_config

pytestmark = pytest.mark.gpu


def _wait(agent, handle, limit=50_000_000):
    state = "PROC"
    for _ in range(limit):
        state = agent.check_xfer_state(handle)
        if state != "PROC":
            break
    return state


def _pair(tag, params=None):
    cfg = nixl_agent_config(enable_prog_thread=False, backends=[])
    a, b = nixl_agent(f"{tag}_a", cfg), nixl_agent(f"{tag}_b", cfg)
    a.create_backend("NVLINK", params or {})
    b.create_backend("NVLINK", params or {})
    return a, b


def _connect(a, b):
    a.add_remote_agent(b.get_agent_metadata())
    b.add_remote_agent(a.get_agent_metadata())


@pytest.mark.parametrize("path", ["vector", "bulk"])
@pytest.mark.parametrize("op", ["WRITE", "READ"])
def test_vram_to_vram_batches(path, op):
    a, b = _pair(f"vv_{path}_{op}", {"copy_path": path})
    torch.manual_seed(0)
    for n_desc, size in [(1, 4096), (16, 65536), (256, 4096), (3, (1 << 22) + 48), (40, 1000)]:
        mine = torch.randint(0, 255, (n_desc, size), dtype=torch.uint8, device="cuda:0")
        theirs = torch.randint(0, 255, (n_desc, size), dtype=torch.uint8, device="cuda:0")
        ra, rb = a.register_memory(mine), b.register_memory(theirs)
        _connect(a, b)
        want = mine.clone() if op == "WRITE" else theirs.clone()
        h = a.initialize_xfer(op, [mine[i] for i in range(n_desc)], [theirs[i] for i in range(n_desc)], b.name)
        assert a.transfer(h) in ("DONE", "PROC")
        assert _wait(a, h) == "DONE"
        torch.cuda.synchronize()
        assert torch.equal(mine, want) and torch.equal(theirs, want), (n_desc, size)
        # repost of the same handle
        (theirs if op == "WRITE" else mine).zero_()
        assert a.transfer(h) in ("DONE", "PROC")
        assert _wait(a, h) == "DONE"
        torch.cuda.synchronize()
        assert torch.equal(mine, want) and torch.equal(theirs, want)
        a.release_xfer_handle(h)
        a.deregister_memory(ra)
        b.deregister_memory(rb)


@pytest.mark.parametrize("path", ["vector", "bulk"])
def test_unaligned_offsets(path):
    a, b = _pair(f"ua_{path}", {"copy_path": path})
    src = torch.randint(0, 255, (1 << 20,), dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda:0")
    a.register_memory(src)
    b.register_memory(dst)
    _connect(a, b)
    cases = [(1, 1, 100), (3, 19, 4097), (16, 32, 65536), (5, 8, 70001), (7, 7, 333333), (0, 4, 15)]
    local = [(src.data_ptr() + so, n, 0) for so, _, n in cases]
    # spread destinations so they do not overlap
    remote, off = [], 0
    for _, do, n in cases:
        remote.append((dst.data_ptr() + off + do, n, 0))
        off += ((n + do + 63) // 64) * 64
    h = a.initialize_xfer("WRITE", a.get_xfer_descs(local, "VRAM"), a.get_xfer_descs(remote, "VRAM"), b.name)
    a.transfer(h)
    assert _wait(a, h) == "DONE"
    torch.cuda.synchronize()
    expect = torch.zeros_like(dst)
    for (so, _, n), (raddr, _, _) in zip(cases, remote):
        o = raddr - dst.data_ptr()
        expect[o : o + n] = src[so : so + n]
    assert torch.equal(dst, expect)
    a.release_xfer_handle(h)


def test_dram_vram_paths():
    a, b = _pair("dv")
    host = torch.randint(0, 255, (8, 1 << 18), dtype=torch.uint8).pin_memory()
    pageable = torch.randint(0, 255, (8, 1 << 18), dtype=torch.uint8)
    dev = torch.zeros(8, 1 << 18, dtype=torch.uint8, device="cuda:0")
    a.register_memory(host)
    a.register_memory(pageable)
    b.register_memory(dev)
    _connect(a, b)
    for h_src in (host, pageable):
        dev.zero_()
        h = a.initialize_xfer("WRITE", h_src, dev, b.name)
        a.transfer(h)
        assert _wait(a, h) == "DONE"
        torch.cuda.synchronize()
        assert torch.equal(dev.cpu(), h_src)
        a.release_xfer_handle(h)
        dev.add_(3)
        h = a.initialize_xfer("READ", h_src, dev, b.name)
        a.transfer(h)
        assert _wait(a, h) == "DONE"
        torch.cuda.synchronize()
        assert torch.equal(dev.cpu(), h_src)
        a.release_xfer_handle(h)


def test_notification_after_data_and_stream_order():
    a, b = _pair("ns")
    src = torch.empty(1 << 26, dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros_like(src)
    a.register_memory(src)
    b.register_memory(dst)
    _connect(a, b)
    stream = torch.cuda.Stream()
    h = a.initialize_xfer("WRITE", src, dst, b.name, b"after-data")
    with torch.cuda.stream(stream):
        src.fill_(7)  # producer kernel on the user's stream; the transfer must run after it
        assert a.transfer(h, custom_param=f"stream={stream.cuda_stream}") in ("DONE", "PROC")
    assert _wait(a, h) == "DONE"
    assert b.check_remote_xfer_done(f"{a.name}", b"after-data")
    torch.cuda.synchronize()
    assert int(dst.min()) == 7 and int(dst.max()) == 7
    a.release_xfer_handle(h)


def test_repost_while_active_is_rejected():
    a, b = _pair("rp")
    src = torch.ones(1 << 28, dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros_like(src)
    a.register_memory(src)
    b.register_memory(dst)
    _connect(a, b)
    h = a.initialize_xfer("WRITE", src, dst, b.name)
    first = a.transfer(h)
    if first == "PROC":
        try:
            st = a.agent.postXferReq(h)
            assert st in (nb.NIXL_SUCCESS, nb.NIXL_IN_PROG)  # finished in between: a legal repost
        except nb.nixlRepostActiveError:
            pass
    assert _wait(a, h) == "DONE"
    a.release_xfer_handle(h)


def test_telemetry_and_cost():
    cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"], capture_telemetry=True)
    a, b = nixl_agent("tm_a", cfg), nixl_agent("tm_b", cfg)
    src = torch.ones(1 << 24, dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros_like(src)
    a.register_memory(src)
    b.register_memory(dst)
    _connect(a, b)
    h = a.initialize_xfer("WRITE", src, dst, b.name)
    a.transfer(h)
    assert _wait(a, h) == "DONE"
    t = a.get_xfer_telemetry(h)
    assert t.totalBytes == 1 << 24 and t.descCount == 1 and t.xferDuration >= 0
    a.release_xfer_handle(h)


@pytest.mark.gpu
def test_gds_vram_file_roundtrip(tmp_path):
    """GPU memory -> file -> other GPU buffer through the staged GDS engine (several 8 MiB chunks and a ragged tail)."""
    a = nixl_agent("gds_gpu", nixl_agent_config(backends=[]))
    a.create_backend("GDS", {"thread_count": "2"})
    n = (20 << 20) + 4096 + 24
    src = torch.randint(0, 255, (n,), dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros_like(src)
    a.register_memory(src)
    a.register_memory(dst)
    path = str(tmp_path / "kv.bin")
    a.register_memory([(0, n, 0, "rw,create:" + path)], "FILE")
    file_descs = a.get_xfer_descs([(0, n, 0)], "FILE")
    for op, t in (("WRITE", src), ("READ", dst)):
        h = a.initialize_xfer(op, a.get_xfer_descs(t), file_descs, a.name)
        st = a.transfer(h)
        while st == "PROC":
            st = a.check_xfer_state(h)
        assert st == "DONE"
        a.release_xfer_handle(h)
    assert torch.equal(src, dst)

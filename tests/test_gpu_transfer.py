"""GPU transfers through the public API, checked against plain torch copies.

Scenarios follow the reference's test/gtest/test_transfer.cpp (VRAM and DRAM, WRITE and
READ, notifications, batches) plus what is new here: the table path for large batches,
odd sizes and offsets, the bulk (TMA) copy path and stream-ordered posting."""
import glob
import os

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
    a, b = _pair(f"vv_{path}_{op}", {"copy_path": path, "coalesce": "false"})  # rows are contiguous: keep them apart
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


def _poll_notifs(agent, who, seconds):
    import time
    got = []
    end = time.monotonic() + seconds
    while time.monotonic() < end and not got:
        got.extend(agent.get_new_notifs().get(who, []))
    return got


def test_notification_reaches_the_target_without_the_initiator_polling():
    """The copy kernel's tail releases the notification in the target's ring itself: the target learns of
    the finished WRITE although the initiator never looks at its request again.  Without the ring the
    datagram leaves only when the initiator's host has seen the completion word."""
    for ring in (True, False):
        before = set(glob.glob(f"/dev/shm/nixl_b200.{os.getpid()}.*"))
        a, b = _pair(f"nr{int(ring)}", {"notif_ring": "true" if ring else "false"})
        rings = set(glob.glob(f"/dev/shm/nixl_b200.{os.getpid()}.*")) - before
        if ring and len(rings) < 2:
            pytest.skip("this box gives the engines no shared-memory ring (no room in /dev/shm?): notifications use datagrams")
        assert ring or not rings
        src = torch.full((1 << 28,), 9, dtype=torch.uint8, device="cuda:0")
        dst = torch.zeros_like(src)
        a.register_memory(src)
        b.register_memory(dst)
        _connect(a, b)
        torch.cuda.synchronize()
        h = a.initialize_xfer("WRITE", src, dst, b.name, b"landed")
        # Posted on a stream that is busy for a few milliseconds: the copy cannot be complete when the post returns,
        # whatever the host does in between.
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            torch.cuda._sleep(20_000_000)
            assert a.transfer(h, custom_param=f"stream={stream.cuda_stream}") == "PROC"
        if ring:
            assert _poll_notifs(b, a.name, 5.0) == [b"landed"]
            assert int(dst[-4096:].min()) == 9 and int(dst[:4096].min()) == 9  # the data was complete before the notification
        else:
            assert _poll_notifs(b, a.name, 0.2) == []
        assert _wait(a, h) == "DONE"
        if not ring:
            assert _poll_notifs(b, a.name, 5.0) == [b"landed"]
        assert _poll_notifs(b, a.name, 0.05) == []  # delivered once
        torch.cuda.synchronize()
        assert int(dst.min()) == 9
        a.release_xfer_handle(h)
        del a, b


def test_bulk_path_deep_pipeline_is_byte_exact():
    """One descriptor, 256 KiB chunks: every CTA runs eight 32 KiB pieces through its four
    shared-memory stages, so each stage is refilled while the store that last used it may still
    be reading it.  The bytes must survive, on the same GPU and (when there is one) to a peer."""
    a, b = _pair("bulk_deep", {"copy_path": "bulk", "chunk_shift": "18", "ce_threshold": "0"})
    n = (24 << 20) + 4096 + 16
    src = torch.randint(0, 255, (n,), dtype=torch.uint8, device="cuda:0")
    targets = ["cuda:0"] + (["cuda:1"] if torch.cuda.device_count() > 1 else [])
    a.register_memory(src)
    for t in targets:
        dst = torch.zeros(n, dtype=torch.uint8, device=t)
        reg = b.register_memory(dst)
        _connect(a, b)
        for op in ("WRITE", "READ"):
            if op == "READ":
                dst.copy_(torch.randint(0, 255, (n,), dtype=torch.uint8, device=t))
                want = dst.clone()
            else:
                dst.zero_()
                want = src.clone()
            h = a.initialize_xfer(op, src, dst, b.name)
            for _ in range(3):
                assert a.transfer(h) in ("DONE", "PROC")
                assert _wait(a, h) == "DONE"
            torch.cuda.synchronize()
            assert torch.equal(dst.to("cuda:0"), want.to("cuda:0")) and torch.equal(src, want.to("cuda:0")), (t, op)
            a.release_xfer_handle(h)
            if op == "READ":
                src.copy_(torch.randint(0, 255, (n,), dtype=torch.uint8, device="cuda:0"))
        b.deregister_memory(reg)


def test_request_after_released_table_request_completes():
    """A request with a descriptor table is released; the next request, whose kernel runs several
    CTAs and therefore counts them, must not inherit the table's bytes as its counter."""
    a, b = _pair("recycle", {"coalesce": "false"})
    src = torch.randint(0, 255, (256, 4096), dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros_like(src)
    a.register_memory(src)
    b.register_memory(dst)
    _connect(a, b)
    for _ in range(4):
        hs = [a.initialize_xfer("WRITE", [src[i] for i in range(256)], [dst[i] for i in range(256)], b.name) for _ in range(3)]
        for h in hs:
            a.transfer(h)
            assert _wait(a, h) == "DONE"
        for h in hs:
            a.release_xfer_handle(h)
        flat_s, flat_d = src.view(-1), dst.view(-1)
        many = [a.initialize_xfer("READ", flat_s[i * 65536:(i + 1) * 65536], flat_d[i * 65536:(i + 1) * 65536], b.name) for i in range(8)]
        for h in many:
            a.transfer(h)
        for h in many:
            assert _wait(a, h, 20_000_000) == "DONE"
            a.release_xfer_handle(h)


def test_ten_thousand_prepared_requests():
    """A serving engine keeps many prepared handles: more than one page of completion words."""
    a, b = _pair("many")
    src = torch.randint(0, 255, (10000, 64), dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros_like(src)
    a.register_memory(src)
    b.register_memory(dst)
    _connect(a, b)
    handles = [a.initialize_xfer("WRITE", src[i], dst[i], b.name) for i in range(10000)]
    for h in handles[::7]:
        a.transfer(h)
    for h in handles[::7]:
        assert _wait(a, h) == "DONE"
    torch.cuda.synchronize()
    assert torch.equal(dst[::7], src[::7]) and int(dst[1::7].max()) == 0
    for h in handles:
        a.release_xfer_handle(h)


def test_independent_requests_use_several_streams():
    """Independent requests of one agent do not queue behind each other (each prepared request is
    bound to one of the engine's streams): a small request posted right after a multi-gigabyte
    one completes while the large one is still in progress."""
    a, b = _pair("streams", {"num_streams": "4"})
    big_src = torch.empty(3 << 30, dtype=torch.uint8, device="cuda:0")
    big_dst = torch.empty_like(big_src)
    small_src = torch.randint(0, 255, (4096,), dtype=torch.uint8, device="cuda:0")
    small_dst = torch.zeros_like(small_src)
    for t in (big_src, small_src):
        a.register_memory(t)
    for t in (big_dst, small_dst):
        b.register_memory(t)
    _connect(a, b)
    big = a.initialize_xfer("WRITE", big_src, big_dst, b.name)
    small = a.initialize_xfer("WRITE", small_src, small_dst, b.name)
    overlapped = 0
    for _ in range(5):
        torch.cuda.synchronize()
        assert a.transfer(big) in ("DONE", "PROC")
        assert a.transfer(small) in ("DONE", "PROC")
        assert _wait(a, small) == "DONE"
        overlapped += a.check_xfer_state(big) == "PROC"
        assert _wait(a, big) == "DONE"
    assert overlapped >= 3, overlapped
    torch.cuda.synchronize()
    assert torch.equal(small_src, small_dst)
    a.release_xfer_handle(big)
    a.release_xfer_handle(small)


def test_neighbouring_descriptors_are_merged_and_long_runs_use_the_copy_engines():
    """Contiguous blocks posted as many descriptors move as one run; a run between two GPUs that
    is long enough goes to the copy engines, with a short one in the same request left to the
    kernel.  Bytes are checked either way (one GPU: everything stays with the kernel)."""
    a, b = _pair("merge", {"ce_threshold": str(1 << 20)})
    peer = "cuda:1" if torch.cuda.device_count() > 1 else "cuda:0"
    blocks, size = 48, 1 << 18
    src = torch.randint(0, 255, (blocks, size), dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros(blocks, size, dtype=torch.uint8, device=peer)
    a.register_memory(src)
    b.register_memory(dst)
    _connect(a, b)
    # blocks 0..39 in order (one 10 MiB run), then 40..47 swapped pairwise (eight short pieces)
    order = list(range(40)) + [41, 40, 43, 42, 45, 44, 47, 46]
    for op in ("WRITE", "READ"):
        if op == "WRITE":
            dst.zero_()
        else:
            dst.copy_(torch.randint(0, 255, (blocks, size), dtype=torch.uint8, device=peer))
            src.zero_()
        h = a.initialize_xfer(op, [src[i] for i in range(blocks)], [dst[j] for j in order], b.name)
        for _ in range(2):
            assert a.transfer(h) in ("DONE", "PROC")
            assert _wait(a, h) == "DONE"
        torch.cuda.synchronize()
        assert torch.equal(dst[order].to("cuda:0"), src), op
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

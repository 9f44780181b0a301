"""File and object backends on host memory (the GPU side of GDS is covered by the gpu-marked test)."""
import os

import numpy as np
import pytest
import torch

from nixl_b200 import nixl_agent, nixl_agent_config


def _wait(agent, h):
    for _ in range(2_000_000):
        st = agent.check_xfer_state(h)
        if st != "PROC":
            return st
    raise TimeoutError


def test_obj_put_get_roundtrip(tmp_path):
    a = nixl_agent("obj_agent", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", {"bucket": str(tmp_path)})
    src = torch.arange(1 << 16, dtype=torch.int32)
    dst = torch.zeros_like(src)
    a.register_memory(src)
    a.register_memory(dst)
    nbytes = src.numel() * 4
    objs = [(0, nbytes, 7, "layer0.kv")]
    reg = a.register_memory(objs, "OBJ")
    assert reg is not None
    # the key does not exist yet
    assert a.query_memory(objs, "OBJ", "OBJ")[0] is None
    local_w = a.get_xfer_descs(src)
    remote = a.get_xfer_descs([(0, nbytes, 7)], "OBJ")
    h = a.initialize_xfer("WRITE", local_w, remote, "obj_agent")
    assert a.transfer(h) in ("DONE", "PROC")
    assert _wait(a, h) == "DONE"
    assert os.path.getsize(tmp_path / "layer0.kv") == nbytes
    assert a.query_memory(objs, "OBJ", "OBJ")[0] is not None
    h2 = a.initialize_xfer("READ", a.get_xfer_descs(dst), remote, "obj_agent")
    a.transfer(h2)
    assert _wait(a, h2) == "DONE"
    assert torch.equal(src, dst)
    a.release_xfer_handle(h)
    a.release_xfer_handle(h2)


def test_obj_missing_key_fails(tmp_path):
    a = nixl_agent("obj_agent2", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", {"bucket": str(tmp_path)})
    dst = torch.zeros(1024, dtype=torch.uint8)
    a.register_memory(dst)
    a.register_memory([(0, 1024, 1, "absent")], "OBJ")
    h = a.initialize_xfer("READ", a.get_xfer_descs(dst), a.get_xfer_descs([(0, 1024, 1)], "OBJ"), "obj_agent2")
    try:
        st = a.transfer(h)
        if st == "PROC":
            st = _wait(a, h)
    except Exception:
        st = "ERR"
    assert st == "ERR"


def test_obj_rejects_path_separators(tmp_path):
    a = nixl_agent("obj_agent3", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", {"bucket": str(tmp_path)})
    with pytest.raises(Exception):
        a.register_memory([(0, 16, 1, "../escape")], "OBJ")


@pytest.mark.parametrize("name", ["GDS", "GDS_MT"])
def test_gds_host_memory_file_roundtrip(tmp_path, name):
    a = nixl_agent("gds_agent_" + name, nixl_agent_config(backends=[]))
    a.create_backend(name, {"thread_count": "2"})
    path = str(tmp_path / "blocks.bin")
    src = torch.from_numpy(np.random.default_rng(0).integers(0, 255, 3 << 20, dtype=np.uint8))
    dst = torch.zeros_like(src)
    a.register_memory(src)
    a.register_memory(dst)
    a.register_memory([(0, src.numel(), 0, "rw,create:" + path)], "FILE")
    half = src.numel() // 2
    file_descs = a.get_xfer_descs([(0, half, 0), (half, half, 0)], "FILE")
    p = src.data_ptr()
    h = a.initialize_xfer("WRITE", a.get_xfer_descs([(p, half, 0), (p + half, half, 0)], "DRAM"), file_descs, a.name)
    a.transfer(h)
    assert _wait(a, h) == "DONE"
    q = dst.data_ptr()
    h2 = a.initialize_xfer("READ", a.get_xfer_descs([(q, half, 0), (q + half, half, 0)], "DRAM"), file_descs, a.name)
    a.transfer(h2)
    assert _wait(a, h2) == "DONE"
    assert torch.equal(src, dst)

"""File and object backends on host memory (the GPU side of GDS is covered by the gpu-marked test)."""
import os

import numpy as np
import pytest
import torch

import nixl_b200
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
    if name == "GDS_MT":
        nixl_b200.add_plugin_directory(nixl_b200.STANDIN_PLUGIN_DIR)
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


def _gusli_config(lines):
    return "# Config file\nversion=1\n" + "\n".join(lines) + "\n"


def test_block_backend_reads_and_writes_at_byte_offsets(tmp_path):
    """The GUSLI-named block backend: BLK descriptors address (device id, byte offset)."""
    store = tmp_path / "store0.bin"
    ro = tmp_path / "readonly.bin"
    ro.write_bytes(bytes(range(256)) * 16)
    a = nixl_agent("blk_agent", nixl_agent_config(backends=[]))
    a.create_backend("GUSLI", {"config_file": _gusli_config([f"11 F W N {store} sec=0x3", f"12 F R Y {ro} sec=0x3"]), "num_threads": "3"})
    src = torch.arange(1 << 14, dtype=torch.int32)
    dst = torch.zeros_like(src)
    a.register_memory(src)
    a.register_memory(dst)
    nbytes = src.numel() * 4
    a.register_memory([(0, 1 << 20, 11, ""), (0, 4096, 12, "")], "BLK")
    info = a.query_memory([(0, 0, 11, ""), (0, 0, 12, ""), (0, 0, 99, "")], "GUSLI", "BLK")
    assert info[0] is not None and info[0]["access"] == "W" and info[1]["size"] == "4096" and info[2] is None

    # Two halves written to swapped positions at offset 8192 of device 11, read back straight.
    half = nbytes // 2
    base = src.data_ptr()
    local = a.get_xfer_descs([(base, half, 0), (base + half, half, 0)], "DRAM")
    swapped = a.get_xfer_descs([(8192 + half, half, 11), (8192, half, 11)], "BLK")
    h = a.initialize_xfer("WRITE", local, swapped, "blk_agent")
    a.transfer(h)
    assert _wait(a, h) == "DONE"
    raw = np.frombuffer(store.read_bytes(), dtype=np.int32)
    assert raw.size == (8192 + nbytes) // 4
    assert np.array_equal(raw[2048 : 2048 + half // 4], src.numpy()[half // 4 :])
    h2 = a.initialize_xfer("READ", a.get_xfer_descs(dst), a.get_xfer_descs([(8192, nbytes, 11)], "BLK"), "blk_agent")
    a.transfer(h2)
    assert _wait(a, h2) == "DONE"
    assert torch.equal(dst, torch.cat([src[half // 4 :], src[: half // 4]]))

    # The read-only device serves reads and refuses writes when the request is built.
    small = torch.zeros(256, dtype=torch.uint8)
    a.register_memory(small)
    h3 = a.initialize_xfer("READ", a.get_xfer_descs(small), a.get_xfer_descs([(256, 256, 12)], "BLK"), "blk_agent")
    a.transfer(h3)
    assert _wait(a, h3) == "DONE"
    assert small.tolist() == list(range(256))
    with pytest.raises(Exception):
        a.initialize_xfer("WRITE", a.get_xfer_descs(small), a.get_xfer_descs([(0, 256, 12)], "BLK"), "blk_agent")
    for x in (h, h2, h3):
        a.release_xfer_handle(x)


def test_block_backend_rejects_bad_configurations(tmp_path):
    a = nixl_agent("blk_agent2", nixl_agent_config(backends=[]))
    for cfg in ("", _gusli_config([]), _gusli_config(["7 N W N t127.0.0.1 sec=0x1"]), _gusli_config(["7 F W"]),
                _gusli_config([f"7 F R N {tmp_path}/absent.bin sec=0"]), "version=2\n7 F W N /tmp/x sec=0\n"):
        with pytest.raises(Exception):
            a.create_backend("GUSLI", {"config_file": cfg})
    # A device that is not in the configuration cannot be registered.
    a.create_backend("GUSLI", {"config_file": _gusli_config([f"1 F W N {tmp_path}/d.bin sec=0"])})
    with pytest.raises(Exception):
        a.register_memory([(0, 4096, 2, "")], "BLK")


@pytest.mark.parametrize("name,param", [("AZURE_BLOB", "container_name"), ("INFINIA", "dataset")])
def test_object_engine_under_the_other_object_store_names(tmp_path, name, param):
    nixl_b200.add_plugin_directory(nixl_b200.STANDIN_PLUGIN_DIR)
    a = nixl_agent(f"obj_{name}", nixl_agent_config(backends=[]))
    assert name in a.get_plugin_list()
    a.create_backend(name, {param: str(tmp_path), "account_url": "https://example.invalid", "tenant": "t"})
    src = torch.arange(4096, dtype=torch.int16)
    dst = torch.zeros_like(src)
    a.register_memory(src)
    a.register_memory(dst)
    a.register_memory([(0, 8192, 3, "blob.bin")], "OBJ")
    remote = a.get_xfer_descs([(0, 8192, 3)], "OBJ")
    h = a.initialize_xfer("WRITE", a.get_xfer_descs(src), remote, f"obj_{name}")
    a.transfer(h)
    assert _wait(a, h) == "DONE"
    assert (tmp_path / "blob.bin").stat().st_size == 8192
    h2 = a.initialize_xfer("READ", a.get_xfer_descs(dst), remote, f"obj_{name}")
    a.transfer(h2)
    assert _wait(a, h2) == "DONE"
    assert torch.equal(src, dst)


def test_file_engine_under_the_hf3fs_name(tmp_path):
    nixl_b200.add_plugin_directory(nixl_b200.STANDIN_PLUGIN_DIR)
    a = nixl_agent("hf3fs_agent", nixl_agent_config(backends=[]))
    a.create_backend("HF3FS", {"mem_config": "auto", "iopool_size": "2"})
    src = torch.arange(1 << 15, dtype=torch.uint8)
    dst = torch.zeros_like(src)
    a.register_memory(src)
    a.register_memory(dst)
    fd = os.open(tmp_path / "f.bin", os.O_RDWR | os.O_CREAT, 0o644)
    try:
        a.register_memory([(0, 4096 + src.numel(), fd, "")], "FILE")
        remote = a.get_xfer_descs([(4096, src.numel(), fd)], "FILE")
        h = a.initialize_xfer("WRITE", a.get_xfer_descs(src), remote, "hf3fs_agent")
        a.transfer(h)
        assert _wait(a, h) == "DONE"
        h2 = a.initialize_xfer("READ", a.get_xfer_descs(dst), remote, "hf3fs_agent")
        a.transfer(h2)
        assert _wait(a, h2) == "DONE"
        assert torch.equal(src, dst) and os.fstat(fd).st_size == 4096 + src.numel()
    finally:
        os.close(fd)

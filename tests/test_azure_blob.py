"""The AZURE_BLOB backend against a blob service: `tests/fake_azure_blob_server.py` keeps containers in memory and
checks the Shared Key signature of every request with hashlib / hmac / base64.  Covered: put, ranged get, properties
through `query_memory`, names with separators and characters that need escaping, a wrong key, a missing blob, block
upload and ranged download of a large blob, a shared access signature instead of a key, and the fall-back to a directory
when no connection string is given."""
import base64
import json
import os
import subprocess
import sys
import time
import urllib.request

import pytest
import torch

from nixl_b200 import nixl_agent, nixl_agent_config

HERE = os.path.dirname(os.path.abspath(__file__))
KEY = base64.b64encode(b"an account key for the tests, long enough").decode()


def _wait(agent, handle, seconds=60):
    deadline = time.time() + seconds
    state = agent.check_xfer_state(handle)
    while state == "PROC" and time.time() < deadline:
        state = agent.check_xfer_state(handle)
    return state


class _Server:
    def __init__(self, *flags):
        self.proc = subprocess.Popen([sys.executable, os.path.join(HERE, "fake_azure_blob_server.py"), "--account", "teststore", "--key", KEY, *flags],
                                     stdout=subprocess.PIPE, text=True)
        self.port = int(self.proc.stdout.readline())

    def connection_string(self, key=KEY, extra=""):
        auth = f"AccountKey={key};" if key else ""
        return f"DefaultEndpointsProtocol=http;AccountName=teststore;{auth}BlobEndpoint=http://127.0.0.1:{self.port}/teststore;{extra}"

    def admin(self, what):
        return json.loads(urllib.request.urlopen(f"http://127.0.0.1:{self.port}/_admin/{what}", timeout=5).read())

    def close(self):
        self.proc.kill()
        self.proc.wait()


@pytest.fixture
def blob():
    server = _Server()
    yield server
    server.close()


def _roundtrip(agent, name, key, src, dev_id=1):
    n = src.numel() * src.element_size()
    agent.register_memory([(0, n, dev_id, key)], "OBJ")
    remote = agent.get_xfer_descs([(0, n, dev_id)], "OBJ")
    h = agent.initialize_xfer("WRITE", agent.get_xfer_descs(src), remote, name)
    agent.transfer(h)
    assert _wait(agent, h) == "DONE"
    dst = torch.zeros_like(src)
    agent.register_memory(dst)
    h2 = agent.initialize_xfer("READ", agent.get_xfer_descs(dst), remote, name)
    agent.transfer(h2)
    assert _wait(agent, h2) == "DONE"
    agent.release_xfer_handle(h)
    agent.release_xfer_handle(h2)
    return dst


def test_put_get_properties_and_ranges_with_shared_key(blob):
    a = nixl_agent("az_a", nixl_agent_config(backends=[]))
    assert "AZURE_BLOB" in a.get_plugin_list()  # on the regular plug-in path
    a.create_backend("AZURE_BLOB", {"connection_string": blob.connection_string(), "container_name": "kv-cache"})
    src = torch.arange(1 << 15, dtype=torch.int32)
    a.register_memory(src)
    name = "layers/3/kv block #2+b.bin"
    objs = [(0, src.numel() * 4, 1, name)]
    assert a.query_memory(objs, "AZURE_BLOB", "OBJ")[0] is None
    assert torch.equal(_roundtrip(a, "az_a", name, src), src)
    info = a.query_memory(objs, "AZURE_BLOB", "OBJ")[0]
    assert info is not None and int(info["size"]) == src.numel() * 4
    assert blob.admin("blobs") == {"kv-cache": {name: src.numel() * 4}}
    part = torch.zeros(500, dtype=torch.int32)
    a.register_memory(part)
    h = a.initialize_xfer("READ", a.get_xfer_descs(part), a.get_xfer_descs([(8000, 2000, 1)], "OBJ"), "az_a")
    a.transfer(h)
    assert _wait(a, h) == "DONE"
    assert torch.equal(part, src[2000:2500])
    stats = blob.admin("stats")
    assert stats["bad_signature"] == 0 and stats["put_blob"] == 1 and stats["get_blob"] == 2 and stats["head"] == 2


def test_a_wrong_key_and_a_missing_blob(blob):
    a = nixl_agent("az_b", nixl_agent_config(backends=[]))
    a.create_backend("AZURE_BLOB", {"connection_string": blob.connection_string(), "container_name": "kv-cache"})
    dst = torch.zeros(1024, dtype=torch.uint8)
    a.register_memory(dst)
    a.register_memory([(0, 1024, 1, "absent")], "OBJ")
    h = a.initialize_xfer("READ", a.get_xfer_descs(dst), a.get_xfer_descs([(0, 1024, 1)], "OBJ"), "az_b")
    st = a.transfer(h)
    assert (st if st != "PROC" else _wait(a, h)) == "ERR"
    assert blob.admin("stats")["bad_signature"] == 0
    b = nixl_agent("az_c", nixl_agent_config(backends=[]))
    b.create_backend("AZURE_BLOB", {"connection_string": blob.connection_string(key=base64.b64encode(b"some other key").decode()), "container_name": "kv-cache"})
    src = torch.ones(1024, dtype=torch.uint8)
    b.register_memory(src)
    b.register_memory([(0, 1024, 1, "forbidden")], "OBJ")
    h = b.initialize_xfer("WRITE", b.get_xfer_descs(src), b.get_xfer_descs([(0, 1024, 1)], "OBJ"), "az_c")
    st = b.transfer(h)
    assert (st if st != "PROC" else _wait(b, h)) == "ERR"
    assert blob.admin("stats")["bad_signature"] == 1 and blob.admin("blobs") == {"kv-cache": {}}


def test_large_blobs_go_up_as_blocks_and_come_down_as_ranges(blob):
    a = nixl_agent("az_d", nixl_agent_config(backends=[]))
    a.create_backend("AZURE_BLOB", {"connection_string": blob.connection_string(), "container_name": "kv-cache", "crtMinLimit": str(1 << 20), "num_threads": "5"})
    src = torch.randint(0, 255, ((4 << 20) + 777,), dtype=torch.uint8)
    a.register_memory(src)
    assert torch.equal(_roundtrip(a, "az_d", "big.bin", src), src)
    stats = blob.admin("stats")
    assert stats["put_block"] == 5 and stats["put_block_list"] == 1 and stats["put_blob"] == 0 and stats["get_blob"] == 5
    assert stats["staged"] == 0 and stats["bad_signature"] == 0


def test_a_shared_access_signature_instead_of_a_key():
    server = _Server("--sas", "abc123")
    try:
        a = nixl_agent("az_e", nixl_agent_config(backends=[]))
        a.create_backend("AZURE_BLOB", {"connection_string": server.connection_string(key="", extra="SharedAccessSignature=sv=2021-08-06&sp=rw&sig=abc123"),
                                        "container_name": "kv-cache"})
        src = torch.arange(3000, dtype=torch.int16)
        a.register_memory(src)
        assert torch.equal(_roundtrip(a, "az_e", "sas.bin", src), src)
        assert server.admin("stats")["sas"] >= 2 and server.admin("stats")["bad_signature"] == 0
    finally:
        server.close()


def test_the_environment_names_the_account_and_no_account_means_a_directory(monkeypatch, tmp_path, blob):
    monkeypatch.setenv("AZURE_STORAGE_CONNECTION_STRING", blob.connection_string())
    monkeypatch.setenv("AZURE_STORAGE_CONTAINER_NAME", "kv-cache")
    a = nixl_agent("az_f", nixl_agent_config(backends=[]))
    a.create_backend("AZURE_BLOB", {})
    src = torch.arange(1000, dtype=torch.float32)
    a.register_memory(src)
    assert torch.equal(_roundtrip(a, "az_f", "env.bin", src), src)
    assert "env.bin" in blob.admin("blobs")["kv-cache"]
    monkeypatch.delenv("AZURE_STORAGE_CONNECTION_STRING")
    b = nixl_agent("az_g", nixl_agent_config(backends=[]))
    b.create_backend("AZURE_BLOB", {"container_name": str(tmp_path), "account_url": "https://example.invalid"})
    b.register_memory(src)
    assert torch.equal(_roundtrip(b, "az_g", "dir.bin", src), src)
    assert (tmp_path / "dir.bin").stat().st_size == 4000
    # a connection string that cannot be used is an error, not a silent fall-back
    c = nixl_agent("az_h", nixl_agent_config(backends=[]))
    with pytest.raises(Exception):
        c.create_backend("AZURE_BLOB", {"connection_string": "AccountName=x", "container_name": "kv-cache"})


def test_nixlbench_against_the_blob_service(blob):
    exe = os.path.join(os.path.dirname(HERE), "nixl_b200", "bin", "nixlbench")
    env = dict(os.environ, NIXL_PLUGIN_DIR=os.path.join(os.path.dirname(HERE), "nixl_b200", "lib", "plugins"), NIXL_LOG_LEVEL="ERROR")
    res = subprocess.run([exe, "--backend", "AZURE_BLOB", "--mem", "DRAM", "--azure_blob_connection_string=" + blob.connection_string(),
                          "--azure_blob_container_name=kv-cache", "--min", "8192", "--max", "131072", "--batch", "2", "--iters", "5", "--warmup", "1", "--check"],
                         env=env, capture_output=True, text=True, timeout=180)
    assert res.returncode == 0, res.stdout + res.stderr
    assert blob.admin("blobs")["kv-cache"] == {"nixlbench-0": 131072, "nixlbench-1": 131072}
    assert blob.admin("stats")["bad_signature"] == 0


def test_an_account_url_with_a_key_beside_it(monkeypatch, blob):
    """`account_url` plus the account's key (parameter or AZURE_STORAGE_KEY) is as good as a connection string."""
    a = nixl_agent("az_url", nixl_agent_config(backends=[]))
    a.create_backend("AZURE_BLOB", {"account_url": f"http://127.0.0.1:{blob.port}/teststore", "account_key": KEY, "container_name": "kv-cache"})
    src = torch.arange(777, dtype=torch.int32)
    a.register_memory(src)
    assert torch.equal(_roundtrip(a, "az_url", "by-url.bin", src), src)
    monkeypatch.setenv("AZURE_STORAGE_ACCOUNT_URL", f"http://127.0.0.1:{blob.port}/teststore")
    monkeypatch.setenv("AZURE_STORAGE_KEY", KEY)
    b = nixl_agent("az_url2", nixl_agent_config(backends=[]))
    b.create_backend("AZURE_BLOB", {"container_name": "kv-cache"})
    b.register_memory(src)
    assert torch.equal(_roundtrip(b, "az_url2", "by-env.bin", src), src)
    assert set(blob.admin("blobs")["kv-cache"]) == {"by-url.bin", "by-env.bin"} and blob.admin("stats")["bad_signature"] == 0


def test_any_blob_name_round_trips(blob):
    """Names drawn by hypothesis: the escaped path is what goes on the wire and what the Shared Key signs."""
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st

    a = nixl_agent("az_names", nixl_agent_config(backends=[]))
    a.create_backend("AZURE_BLOB", {"connection_string": blob.connection_string(), "container_name": "kv-cache"})
    src = torch.arange(48, dtype=torch.uint8)
    dst = torch.zeros_like(src)
    a.register_memory(src)
    a.register_memory(dst)
    seen = []
    alphabet = st.one_of(st.characters(min_codepoint=0x20, max_codepoint=0x7E), st.sampled_from(list("äßçñ漢字ключ🙂")))

    @settings(max_examples=30, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
    @given(st.text(alphabet, min_size=1, max_size=40).filter(lambda k: k.strip("/") == k and "//" not in k and k not in (".", "..") and "\\" not in k))
    def check(name):
        if name in seen:
            return
        seen.append(name)
        dev = len(seen)
        src.fill_(dev % 251)
        a.register_memory([(0, 48, dev, name)], "OBJ")
        remote = a.get_xfer_descs([(0, 48, dev)], "OBJ")
        for op, buf in (("WRITE", src), ("READ", dst)):
            h = a.initialize_xfer(op, a.get_xfer_descs(buf), remote, "az_names")
            a.transfer(h)
            assert _wait(a, h) == "DONE", name
            a.release_xfer_handle(h)
        assert torch.equal(src, dst), name

    check()
    assert sorted(blob.admin("blobs")["kv-cache"]) == sorted(seen) and blob.admin("stats")["bad_signature"] == 0

"""The host-side examples run to completion (the GPU ones are exercised by the gpu-marked suites)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,args", [
    ("basic_two_peers.py", []),
    ("expanded_two_peers.py", []),
    ("partial_md_example.py", []),
    ("query_mem_example.py", []),
    ("nixl_gds_example.py", ["--mib", "2"]),
    ("metadata_store_example.py", []),
])
def test_example_runs(script, args):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), *args], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]


def test_cpp_example_builds_with_the_pkg_config_file_and_runs(tmp_path):
    """A C++ user's build line: flags from the pkg-config file the build writes next to the library."""
    import shutil

    exe = str(tmp_path / "two_agents")
    lib = os.path.join(ROOT, "nixl_b200", "lib")
    flags = ["-I" + os.path.join(ROOT, "csrc", "include"), "-L" + lib, "-lnixl", "-Wl,-rpath," + lib]
    pc = os.path.join(lib, "pkgconfig", "nixl.pc")
    if shutil.which("pkg-config") and os.path.exists(pc):
        out = subprocess.run(["pkg-config", "--cflags", "--libs", "nixl"], env=dict(os.environ, PKG_CONFIG_PATH=os.path.dirname(pc)), capture_output=True, text=True)
        assert out.returncode == 0, out.stderr
        flags = out.stdout.split()
        assert any(f.startswith("-I") for f in flags) and "-lnixl" in flags
    build = subprocess.run(["g++", "-std=c++20", "-O1", os.path.join(ROOT, "examples", "cpp", "two_agents.cpp"), "-o", exe, *flags, "-pthread"],
                           capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, NIXL_PLUGIN_DIR=os.path.join(lib, "plugins"))
    for backend in ("NVLINK", "TCP"):
        res = subprocess.run([exe, backend], env=env, capture_output=True, text=True, timeout=120)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
        assert f"backend {backend}: moved 1048576 bytes" in res.stdout and "identical" in res.stdout


def test_cpp_telemetry_reader_drains_a_ring_written_by_an_agent(tmp_path):
    exe = str(tmp_path / "telemetry_reader")
    build = subprocess.run(["g++", "-std=c++20", "-O1", "-I" + os.path.join(ROOT, "csrc", "include"),
                            os.path.join(ROOT, "examples", "cpp", "telemetry_reader.cpp"), "-o", exe, "-pthread"], capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    tdir = tmp_path / "telemetry"
    tdir.mkdir()
    env = dict(os.environ, NIXL_TELEMETRY_ENABLE="1", NIXL_TELEMETRY_DIR=str(tdir), NIXL_TELEMETRY_RUN_INTERVAL="20", PYTHONPATH=ROOT)
    # The ring lives as long as its agent: the writer moves 4 MiB, says so, and waits for a line on stdin.
    code = (
        "import sys, time, torch\n"
        "from nixl_b200 import nixl_agent, nixl_agent_config\n"
        "a = nixl_agent('initiator', nixl_agent_config(backends=['NVLINK']))\n"
        "b = nixl_agent('target', nixl_agent_config(backends=['NVLINK']))\n"
        "s, d = torch.ones(1 << 20), torch.zeros(1 << 20)\n"
        "a.register_memory(s); b.register_memory(d)\n"
        "a.add_remote_agent(b.get_agent_metadata())\n"
        "h = a.initialize_xfer('WRITE', s, d, 'target')\n"
        "st = a.transfer(h)\n"
        "while st == 'PROC': st = a.check_xfer_state(h)\n"
        "time.sleep(0.3)\n"
        "print('moved', flush=True)\n"
        "sys.stdin.readline()\n"
    )
    writer = subprocess.Popen([sys.executable, "-c", code], env=env, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        assert writer.stdout.readline().strip() == "moved", writer.stderr.read()[-2000:]
        res = subprocess.run([exe, str(tdir / "initiator")], capture_output=True, text=True, timeout=60)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "agent_tx_bytes 4194304" in res.stdout and "agent_memory_registered" in res.stdout
        # The ring was consumed: a second pass finds nothing new.
        again = subprocess.run([exe, str(tdir / "initiator")], capture_output=True, text=True, timeout=60)
        assert "# 0 events" in again.stdout
    finally:
        writer.stdin.write("\n")
        writer.stdin.close()
        writer.wait(timeout=60)


def test_remote_storage_example_between_a_server_and_a_client(tmp_path):
    """examples/remote_storage_example.py: a client stores its blocks on a storage server and loads them back; the server
    moves every block over the network backend and the storage backend, one stage behind the other."""
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = os.path.join(ROOT, "examples", "remote_storage_example.py")
    (tmp_path / "agents.txt").write_text(f"# storage servers\nstore0 127.0.0.1 {port}\n")
    common = ["--buf_size", str(256 << 10), "--batch_size", "6"]
    server = subprocess.Popen([sys.executable, script, "--role", "server", "--agent_name", "store0", "--port", str(port), "--fileprefix", str(tmp_path / "srv"),
                               "--requests", "2", *common], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        assert "serving" in server.stdout.readline()
        client = subprocess.run([sys.executable, script, "--role", "client", "--agent_name", "kv_client", "--agents_file", str(tmp_path / "agents.txt"),
                                 "--fileprefix", str(tmp_path / "cli"), *common], capture_output=True, text=True, timeout=240)
        assert client.returncode == 0, client.stdout[-2000:] + client.stderr[-2000:]
        assert "all blocks verified" in client.stdout
        assert server.wait(timeout=60) == 0, server.stderr.read()[-2000:]
        # what the server keeps is what the client sent: block i is filled with (17 + i) % 251
        for i in range(6):
            data = (tmp_path / f"srv_store0_{i}.bin").read_bytes()
            assert len(data) == 256 << 10 and set(data) == {(17 + i) % 251}
    finally:
        if server.poll() is None:
            server.kill()
        server.wait()


def test_cpp_etcd_example_against_the_stand_in_gateway(tmp_path):
    """examples/cpp/etcd_metadata.cpp: full metadata, partial metadata under a label, invalidation, all through the store."""
    exe = str(tmp_path / "etcd_metadata")
    lib = os.path.join(ROOT, "nixl_b200", "lib")
    build = subprocess.run(["g++", "-std=c++20", "-O1", "-I" + os.path.join(ROOT, "csrc", "include"), "-I/usr/local/cuda/include",
                            os.path.join(ROOT, "examples", "cpp", "etcd_metadata.cpp"), "-o", exe, "-L" + lib, "-lnixl", "-Wl,-rpath," + lib, "-pthread"],
                           capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    gateway = subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "fake_etcd_gateway.py")], stdout=subprocess.PIPE, text=True)
    try:
        port = int(gateway.stdout.readline())
        env = dict(os.environ, NIXL_ETCD_ENDPOINTS=f"http://127.0.0.1:{port}", NIXL_PLUGIN_DIR=os.path.join(lib, "plugins"))
        env.pop("NIXL_TCPSTORE_ENDPOINT", None)
        res = subprocess.run([exe], env=env, capture_output=True, text=True, timeout=120)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
        assert "label 'extra_buffers'" in res.stdout and "prefill dropped it" in res.stdout
    finally:
        gateway.kill()
        gateway.wait()


@pytest.mark.parametrize("backends", ["NVLINK,TCP", "TCP"])
def test_kv_blocks_between_a_prefill_and_a_decode_process(backends):
    """examples/kv_blocks_between_hosts.py: prepared lists on both sides, block numbers per request, over the sockets
    when only TCP is created (what two hosts would use) and over whatever the agent prefers otherwise."""
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = os.path.join(ROOT, "examples", "kv_blocks_between_hosts.py")
    dec = subprocess.Popen([sys.executable, script, "--role", "decode", "--port", str(port), "--backends", backends], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        assert "listening" in dec.stdout.readline()
        pre = subprocess.run([sys.executable, script, "--role", "prefill", "--peer-port", str(port), "--backends", backends], capture_output=True, text=True, timeout=240)
        assert pre.returncode == 0, pre.stdout[-2000:] + pre.stderr[-2000:]
        assert "has verified the blocks" in pre.stdout
        if backends == "TCP":
            assert "over TCP" in pre.stdout
        assert dec.wait(timeout=60) == 0, dec.stderr.read()[-2000:]
        assert "20 blocks arrived" in dec.stdout.read()
    finally:
        if dec.poll() is None:
            dec.kill()
        dec.wait()

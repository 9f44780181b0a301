"""The Prometheus telemetry exporters: single process, and the multi-process one where whichever
process holds the lock serves everybody's metrics and a survivor takes over when it dies."""
import os
import socket
import subprocess
import sys
import time
import urllib.request

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import sys, time, torch
sys.path.insert(0, %r)
from nixl_b200 import nixl_agent, nixl_agent_config
name = sys.argv[1]
a = nixl_agent(name, nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"], capture_telemetry=True))
b = nixl_agent(name + "_peer", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
src, dst = torch.arange(4096, dtype=torch.uint8), torch.zeros(4096, dtype=torch.uint8)
a.register_memory(src); b.register_memory(dst)
a.add_remote_agent(b.get_agent_metadata())
h = a.initialize_xfer("WRITE", src, dst, name + "_peer")
for _ in range(3):
    a.transfer(h)
    while a.check_xfer_state(h) == "PROC":
        pass
print("ready", flush=True)
sys.stdin.readline()  # stay alive until the test says otherwise
""" % ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _scrape(port, want, timeout=15.0):
    deadline = time.time() + timeout
    last = ""
    while time.time() < deadline:
        try:
            last = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=2).read().decode()
            if all(w in last for w in want):
                return last
        except OSError:
            pass
        time.sleep(0.2)
    raise AssertionError(f"metrics never showed {want}; last scrape:\n{last[-1500:]}")


def _spawn(name, env):
    p = subprocess.Popen([sys.executable, "-c", WORKER, name], env=env, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    assert p.stdout.readline().strip() == "ready"
    return p


def test_single_process_exporter_serves_counters_and_histograms():
    port = _free_port()
    env = dict(os.environ, NIXL_TELEMETRY_EXPORTER="PROMETHEUS", NIXL_TELEMETRY_PROMETHEUS_PORT=str(port), NIXL_TELEMETRY_PROMETHEUS_LOCAL="y",
               NIXL_TELEMETRY_RUN_INTERVAL="20")
    p = _spawn("prom_solo", env)
    try:
        text = _scrape(port, ['agent_tx_bytes_total{agent="prom_solo"} 12288', 'agent_xfer_time_us_bucket{agent="prom_solo",le="+Inf"} 3'])
        assert 'agent_errors_total{agent="prom_solo",status=' in text and "# TYPE agent_xfer_time_us histogram" in text
    finally:
        p.stdin.close()
        p.wait(timeout=20)


def test_multi_process_exporter_one_endpoint_and_takeover(tmp_path):
    port = _free_port()
    env = dict(os.environ, NIXL_TELEMETRY_EXPORTER="PROMETHEUS_MP", NIXL_TELEMETRY_PROMETHEUS_PORT=str(port), NIXL_TELEMETRY_PROMETHEUS_LOCAL="y",
               NIXL_TELEMETRY_PROMETHEUS_MP_DIR=str(tmp_path), NIXL_TELEMETRY_RUN_INTERVAL="20")
    first = _spawn("mp_first", env)
    second = _spawn("mp_second", env)
    try:
        text = _scrape(port, ['agent_tx_bytes_total{agent="mp_first"', 'agent_tx_bytes_total{agent="mp_second"'])
        assert text.count("agent_tx_requests_num_total{") == 2  # the peers capture nothing
        assert len([f for f in os.listdir(tmp_path) if f.endswith(".prom")]) == 2
        # The owner of the endpoint goes away without cleaning up: the other process takes the lock and the port,
        # keeps serving its own metrics and removes the dead process's file.
        first.kill()
        first.wait(timeout=20)
        text = _scrape(port, ['agent_tx_bytes_total{agent="mp_second"'], timeout=20)
        deadline = time.time() + 10
        while 'agent="mp_first"' in text and time.time() < deadline:
            time.sleep(0.3)
            text = _scrape(port, ['agent="mp_second"'])
        assert 'agent="mp_first"' not in text
    finally:
        for p in (first, second):
            if p.poll() is None:
                p.stdin.close()
                p.wait(timeout=20)

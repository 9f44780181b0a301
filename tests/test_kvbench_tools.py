"""kvbench tools on CPU: size parsing, traffic patterns, workload generation, plans, and a
two-rank custom-traffic run over host memory (gloo + the agent API)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from benchmarks.kvbench import matgen, plan, traffic  # noqa: E402
from nixl_b200.models import ParallelConfig  # noqa: E402


def test_size_cells():
    assert traffic.parse_size("4096") == 4096
    assert traffic.parse_size("5K") == 5 << 10
    assert traffic.parse_size("1.5M") == 3 << 19
    assert traffic.parse_size("2GB") == 2 << 30
    assert traffic.format_size(3 << 20) == "3M" and traffic.format_size(1000) == "1000" and traffic.format_size(0) == "0"
    with pytest.raises(ValueError):
        traffic.parse_size("lots")


def test_matrix_file_roundtrip_and_rank_sets(tmp_path):
    m = [[0, 0, 1 << 20, 1 << 20], [0, 0, 1 << 20, 1 << 20], [0, 0, 0, 5 << 10], [0, 0, 0, 0]]
    path = tmp_path / "m.txt"
    traffic.save_matrix(str(path), m)
    assert path.read_text().splitlines()[2] == "0 0 0 5K"
    assert traffic.load_matrix(str(path)) == m
    tp = traffic.TrafficPattern(matrix=m, mem_type="cpu")
    assert tp.senders() == [0, 1, 2] and tp.receivers() == [2, 3] and tp.receivers([2]) == [3]
    assert tp.total_bytes() == (4 << 20) + (5 << 10) and tp.recv_bytes(3) == (2 << 20) + (5 << 10)
    with pytest.raises(ValueError):
        traffic.TrafficPattern(matrix=[[0, 1]], mem_type="cpu")


def test_workload_generation_is_reproducible_and_conserves_bytes(tmp_path):
    task = matgen.TaskConfig(isl_mean=8000, isl_scale=3000, batch_size=2)
    prefill, decode = ParallelConfig(tp=2), ParallelConfig(tp=4)
    a = matgen.generate("llama-3-8b", 6, task, prefill, decode, world_size=12, seed=7)
    b = matgen.generate("llama-3-8b", 6, task, prefill, decode, world_size=12, seed=7)
    assert [m.matrix for m in a] == [m.matrix for m in b] and len(a) == 3
    batches = matgen.gen_batches(6, task, "llama-3-8b", seed=7)
    for tm, batch in zip(a, batches):
        want = sum(matgen.kv_bytes_total("llama-3-8b", isl) for isl in batch.isls)
        assert abs(sum(map(sum, tm.matrix)) - want) <= 8  # integer division over 2 x 2 cells
        senders = [i for i, r in enumerate(tm.matrix) if any(r)]
        assert len(senders) == 2 and all(sum(1 for c in tm.matrix[s] if c) == 2 for s in senders)  # each prefill rank feeds two decode ranks
        assert tm.compute_time > 0
    # the two couples (6 ranks each) take turns
    assert [i for i, r in enumerate(a[0].matrix) if any(r)] == [0, 1] and [i for i, r in enumerate(a[1].matrix) if any(r)] == [6, 7]
    cfg = matgen.write_workload(a, str(tmp_path))
    import yaml

    doc = yaml.safe_load(open(cfg))
    assert len(doc["traffic_patterns"]) == 3 and os.path.exists(tmp_path / "matrices" / "matrix_2.txt")
    with pytest.raises(ValueError):
        matgen.generate("llama-3-8b", 1, task, ParallelConfig(tp=4), ParallelConfig(tp=2), world_size=6)


def test_plan_lines_follow_the_model_geometry():
    rep = plan.kvcache_report("llama-3-8b", 4096, 8, ParallelConfig(tp=4), 16)
    assert rep["io_size"] == 16 * 2 * 128 * 2 and rep["kv_bytes_per_request_per_gpu"] == 4096 * 32 * 2 * 2 * 128 * 2
    cmds = plan.plan_commands("llama-3-8b", 4096, 8, ParallelConfig(tp=4), 16)
    assert len(cmds) == 2 and "--min 8192 --max 8192" in cmds[0] and "--backend NVLINK" in cmds[0]
    assert "llama-3-8b" in plan.model_names()


@pytest.mark.parametrize("backend,port", [("NVLINK", "29631"), ("TCP", "29633")])
def test_ct_perftest_two_ranks_host_memory(tmp_path, backend, port):
    """The traffic-matrix test between two ranks on host memory; with the TCP backend it is the run one would start over
    several hosts (torchrun across nodes, the agents reaching each other over sockets)."""
    cfg = tmp_path / "ct.yaml"
    cfg.write_text("iters: 3\nwarmup_iters: 1\ntraffic_pattern:\n  matrix: [[0, 256K], [64K, 0]]\n  mem_type: cpu\n  shards: 4\n  xfer_op: WRITE\n")
    out = tmp_path / "report.json"
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", port, "-m", "benchmarks.kvbench", "ct-perftest", str(cfg), "--backend", backend, "--json-output-path", str(out)],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rep = json.loads(out.read_text())
    assert rep["verified"] is True and rep["num_senders"] == 2 and rep["ranks"] == 2 and rep["avg_ms"] > 0


def test_sequential_ct_perftest_two_ranks_read(tmp_path):
    cfg = tmp_path / "seq.yaml"
    cfg.write_text("traffic_patterns:\n- matrix: [[0, 1M], [0, 0]]\n  mem_type: cpu\n  xfer_op: READ\n  sleep_before_launch_sec: 0.01\n"
                   "- matrix: [[0, 0], [128K, 0]]\n  mem_type: cpu\n")
    out = tmp_path / "rows.json"
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29632", "-m", "benchmarks.kvbench", "sequential-ct-perftest", str(cfg), "--json-output-path", str(out)],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rows = json.loads(out.read_text())
    assert len(rows) == 2 and rows[0]["num_senders"] == 1 and rows[0]["isolated_latency_ms"] > 0
    assert "Isolated Latency" in r.stdout


def test_storage_backend_reads_and_writes_file_regions(tmp_path):
    import torch

    from benchmarks.kvbench.storage import FilesystemBackend, StorageOp, storage_perftest
    from nixl_b200 import nixl_agent, nixl_agent_config

    rep = storage_perftest(str(tmp_path / "bench"), 1 << 20, iters=2, mem="cpu", chunk_bytes=1 << 18)
    assert rep["verified"] and rep["read_GBps"] > 0 and rep["chunk_bytes"] == 1 << 18

    agent = nixl_agent("kvb_store_test", nixl_agent_config(backends=["POSIX"]))
    fs = FilesystemBackend(agent, str(tmp_path / "ops"))
    op = StorageOp(str(tmp_path / "ops" / "custom.bin"), file_size=12288, read_offset=4096, read_size=4096, write_offset=8192, write_size=2048)
    h = fs.prepare(3, 5, op=op)
    buf = torch.zeros(4096, dtype=torch.uint8)
    agent.register_memory(buf)
    rh = fs.get_read_handle(h, buf)
    assert agent.transfer(rh) in ("DONE", "PROC")
    while agent.check_xfer_state(rh) == "PROC":
        pass
    assert buf[:256].tolist() == [(5 * 31 + i) & 0xFF for i in range(256)]
    buf[:2048] = 7
    wh = fs.get_write_handle(h, buf)
    agent.transfer(wh)
    while agent.check_xfer_state(wh) == "PROC":
        pass
    raw = (tmp_path / "ops" / "custom.bin").read_bytes()
    assert len(raw) == 12288 and raw[8192:10240] == bytes([7]) * 2048 and raw[:4096] == bytes(4096)
    import pytest

    with pytest.raises(ValueError):
        StorageOp("x", 100, read_offset=90, read_size=20)
    fs.close(remove_files=True)
    assert not (tmp_path / "ops" / "custom.bin").exists()


def test_storage_perftest_against_object_stores(tmp_path):
    """kvbench's storage test with objects instead of file regions: a directory as the bucket, then an S3 service (the
    stand-in of tests/fake_s3_server.py) through the CLI, with the region cut into several objects."""
    from benchmarks.kvbench.storage import storage_perftest

    bucket = tmp_path / "bucket"
    bucket.mkdir()
    rep = storage_perftest(str(bucket), 1 << 20, iters=2, store="obj", chunk_bytes=1 << 18, rank=3)
    assert rep["verified"] and rep["store"] == "obj" and rep["read_GBps"] > 0
    assert sorted(p.name for p in bucket.iterdir()) == [f"kvbench_tp0_rank3.{kind}.{k}" for kind in ("read", "write") for k in range(4)]

    server = subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "fake_s3_server.py"), "--bucket", "kv", "--access-key", "AK", "--secret-key", "SK"],
                              stdout=subprocess.PIPE, text=True)
    try:
        port = int(server.stdout.readline())
        out = subprocess.run([sys.executable, "-m", "benchmarks.kvbench", "storage-perftest", "--path", str(tmp_path), "--size", "512K", "--iters", "2",
                              "--store", "obj", "--store-param", f"endpoint_override=http://127.0.0.1:{port}", "--store-param", "bucket=kv",
                              "--store-param", "access_key=AK", "--store-param", "secret_key=SK"],
                             cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT), capture_output=True, text=True, timeout=180)
        assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
        rep = json.loads(out.stdout.strip().splitlines()[-1])
        assert rep["verified"] is True and rep["bytes"] == 512 << 10
        import urllib.request

        keys = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/_admin/keys", timeout=5).read())["kv"]
        assert keys == {"kvbench_tp0_rank0.read": 512 << 10, "kvbench_tp0_rank0.write": 512 << 10}
        stats = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/_admin/stats", timeout=5).read())
        assert stats["bad_signature"] == 0
    finally:
        server.kill()
        server.wait()

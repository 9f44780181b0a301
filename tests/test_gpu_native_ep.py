"""The C++ host classes of the fused paths (csrc/include/nixl_ep.h: nixlEpBuffer, nixlKvTransfer), through the
example program that is built from examples/cpp/ep_dispatch_combine.cpp: expert-parallel dispatch and
rank-reduced combine over up to four ranks (one per GPU) and a resharding KV transfer, both checked on the host."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_native_ep_and_kv_example():
    exe = os.path.join(ROOT, "nixl_b200", "bin", "ep_native_example")
    assert os.path.exists(exe), "run `make -C csrc` first"
    env = dict(os.environ, NIXL_PLUGIN_DIR=os.path.join(ROOT, "nixl_b200", "lib", "plugins"))
    res = subprocess.run([exe], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "combined output as expected" in res.stdout and "bytes as expected" in res.stdout

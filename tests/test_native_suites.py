"""Runs the native (C++) test programs built by `make -C csrc tests` and the native sweep
driver on DRAM.  The programs print one line per case and exit with the number of failures."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "csrc", "build", "tests")
ENV = dict(os.environ, NIXL_PLUGIN_DIR=os.path.join(ROOT, "nixl_b200", "lib", "plugins"),
           NIXL_TEST_PLUGIN_DIR=os.path.join(ROOT, "nixl_b200", "lib", "test_plugins"), NIXL_LOG_LEVEL="FATAL")


def _run(binary, *args, timeout=300):
    path = os.path.join(BUILD, binary)
    if not os.path.exists(path):
        subprocess.run(["make", "-C", os.path.join(ROOT, "csrc"), "-j8", "tests"], check=True, capture_output=True)
    return subprocess.run([path, *args], env=ENV, capture_output=True, text=True, timeout=timeout, cwd=os.path.join(ROOT, "csrc"))


@pytest.mark.parametrize("binary", ["test_plumbing", "test_core"])
def test_native_suite(binary):
    res = _run(binary)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-2000:]
    assert " 0 failed" in res.stdout


def test_native_nixlbench_dram_consistency():
    exe = os.path.join(ROOT, "nixl_b200", "bin", "nixlbench")
    res = subprocess.run([exe, "--mem", "DRAM", "--max", "262144", "--iters", "50", "--warmup", "5", "--batch", "4", "--depth", "2", "--check"],
                         env=ENV, capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert len(res.stdout.strip().splitlines()) >= 7

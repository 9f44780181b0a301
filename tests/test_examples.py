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
])
def test_example_runs(script, args):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), *args], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]


def test_cpp_example_builds_and_runs(tmp_path):
    exe = str(tmp_path / "two_agents")
    lib = os.path.join(ROOT, "nixl_b200", "lib")
    build = subprocess.run(["g++", "-std=c++20", "-O1", "-I" + os.path.join(ROOT, "csrc", "include"), "-I/usr/local/cuda/include",
                            os.path.join(ROOT, "examples", "cpp", "two_agents.cpp"), "-o", exe, "-L" + lib, "-lnixl", "-Wl,-rpath," + lib, "-pthread"],
                           capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    res = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]

"""GPU device API: put / get / atomic add / get-pointer from inside a kernel at THREAD, WARP
and BLOCK level, two agents in one process (second GPU when present).  Mirrors the reference's
test/gtest/device_api/single_write_test.cu."""
import pytest
import torch

from nixl_b200 import _bindings as nb
from nixl_b200 import nixl_agent, nixl_agent_config
from nixl_b200.ops import device_api

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("level", ["THREAD", "WARP", "BLOCK"])
@pytest.mark.parametrize("use_get", [False, True])
def test_put_get_signal(level, use_get):
    d0 = torch.device("cuda:0")
    d1 = torch.device("cuda:1" if torch.cuda.device_count() > 1 else "cuda:0")
    cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"])
    a, b = nixl_agent(f"da_{level}_{int(use_get)}_a", cfg), nixl_agent(f"da_{level}_{int(use_get)}_b", cfg)
    size, iters = (1 << 12) + 16, 5
    mine = torch.randint(0, 255, (size * iters,), dtype=torch.uint8, device=d0)
    theirs = torch.randint(0, 255, (size * iters,), dtype=torch.uint8, device=d1)
    signal = torch.zeros(8, dtype=torch.int64, device=d1)
    a.register_memory(mine)
    b.register_memory(theirs)
    b.register_memory(signal)
    a.add_remote_agent(b.get_agent_metadata())
    with torch.cuda.device(d0):
        local_view = a.prep_mem_view(a.get_xfer_descs(mine))
        remote_view = a.prep_mem_view(a.get_remote_descs([(theirs.data_ptr(), theirs.numel(), d1.index, b.name)], "VRAM"))
        signal_view = a.prep_mem_view(a.get_remote_descs([(signal.data_ptr(), 64, d1.index, b.name)], "VRAM"))
    want = theirs.clone() if use_get else mine.clone()
    status = device_api.put_test(level, local_view, remote_view, signal_view, size, iters, use_get, device=d0)
    torch.cuda.synchronize(d1)
    assert status == [nb.NIXL_SUCCESS, nb.NIXL_ERR_INVALID_PARAM, 1, 1]
    assert torch.equal(mine.cpu(), want.cpu()) and torch.equal(theirs.cpu(), want.cpu())
    assert int(signal[0]) == iters
    for v in (local_view, remote_view, signal_view):
        a.release_mem_view(v)


def test_null_agent_hole_gives_null_pointer():
    cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"])
    a, b = nixl_agent("da_hole_a", cfg), nixl_agent("da_hole_b", cfg)
    buf_a = torch.zeros(4096, dtype=torch.uint8, device="cuda:0")
    buf_b = torch.zeros(4096, dtype=torch.uint8, device="cuda:0")
    sig = torch.zeros(8, dtype=torch.int64, device="cuda:0")
    a.register_memory(buf_a)
    b.register_memory(buf_b)
    b.register_memory(sig)
    a.add_remote_agent(b.get_agent_metadata())
    # entry 0 is a hole, entry 1 is real: a put to entry 0 must be refused
    view = a.prep_mem_view(a.get_remote_descs([(0, 0, 0, nb.NIXL_NULL_AGENT), (buf_b.data_ptr(), 4096, 0, b.name)], "VRAM"))
    local = a.prep_mem_view(a.get_xfer_descs(buf_a))
    sview = a.prep_mem_view(a.get_remote_descs([(sig.data_ptr(), 64, 0, b.name)], "VRAM"))
    status = device_api.put_test("WARP", local, view, sview, 1024, 2)
    assert status[0] == nb.NIXL_ERR_INVALID_PARAM  # destination entry 0 is a hole
    assert status[2] == 0  # and its pointer is null
    assert int(sig[0]) == 0

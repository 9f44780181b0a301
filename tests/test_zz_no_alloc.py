"""The allocation-free KV transfer entry point (csrc/include/kernels/nixl_kv_xfer_static.h) gives the
same bytes as the regular entry point.

Some users of this library cannot allocate GPU memory when they need a transfer (a serving
engine's pool owns the device; an allocator lock is off-limits on their hot path), so they can
hand over neither device block tables nor a device scratch counter.  The entry point tested here
takes the block tables from host memory and keeps its scratch inside the library image.  The test
drives it through the exported C symbol, twice in a row on one stream (the scratch is shared and
keeps the previous call's contents), and compares the receiver's cache with what the regular
entry point produced for the same inputs; a bf16 copy must match bit for bit, and so must the
bf16 -> fp8 e4m3 cast (both entry points run the same conversion).  The receiver-side completion
counter (``done_signal``) must have advanced by ``done_value`` per call.  It also checks that a
request above the built-in capacity is refused instead of overrunning the scratch.
The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test."""
import ctypes

import pytest
import torch

from nixl_b200 import nixl_agent, nixl_agent_config
from nixl_b200.ops import KVLayout, KVTransfer, _lib
from nixl_b200.ops.kv_transfer import _Params

pytestmark = pytest.mark.gpu

ERR_TOO_LARGE = -1001


def _entry():
    lib = _lib.lib()
    fn = lib.nixl_kv_xfer_launch_static
    fn.argtypes = [ctypes.POINTER(_Params), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.nixl_kv_xfer_static_max_pairs.restype = ctypes.c_int
    return fn, lib.nixl_kv_xfer_static_max_pairs()


@pytest.mark.parametrize("cast_fp8", [False, True], ids=["bf16", "fp8"])
def test_static_entry_matches_regular_entry_twice(cast_fp8):
    dev = torch.device("cuda:0")
    cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"])
    tag = "fp8" if cast_fp8 else "bf16"
    a, b = nixl_agent(f"zz_prefill_{tag}", cfg), nixl_agent(f"zz_decode_{tag}", cfg)
    g = torch.Generator(device=dev).manual_seed(7)
    blocks, n_tensors = 64, 4
    src = [torch.randn(blocks, 16, 2, 128, device=dev, dtype=torch.bfloat16, generator=g) for _ in range(n_tensors)]
    dst_dtype, esz = (torch.uint8, 1) if cast_fp8 else (torch.bfloat16, 2)
    dst_regular = [torch.zeros(blocks, 16, 4, 128, device=dev, dtype=dst_dtype) for _ in range(n_tensors)]
    dst_static = [torch.zeros_like(t) for t in dst_regular]
    signal = torch.zeros(2, dtype=torch.int64, device=dev)  # [0]: bumped by the static entry point when all data landed
    a.register_memory(src)
    b.register_memory(dst_regular)
    b.register_memory(dst_static)
    a.add_remote_agent(b.get_agent_metadata())

    def path(dst):
        return KVTransfer(a, src, KVLayout(16, 2, 128), b.name, [(t.data_ptr(), t.numel() * esz, 0) for t in dst],
                          KVLayout(16, 4, 128, elem_bytes=esz), dst_head_offset=2, cast_fp8=cast_fp8, scale=0.5 if cast_fp8 else 1.0)

    regular, static_path = path(dst_regular), path(dst_static)
    fn, max_pairs = _entry()
    assert max_pairs >= blocks
    stream = torch.cuda.current_stream(dev)
    flag = torch.zeros(1, dtype=torch.int64).pin_memory()

    for round_no, n in enumerate((48, 17), start=1):  # the second call sees the first call's leftovers in the scratch
        sb = torch.randperm(blocks, generator=torch.Generator().manual_seed(round_no))[:n].int()
        db = torch.randperm(blocks, generator=torch.Generator().manual_seed(100 + round_no))[:n].int()
        for t in dst_regular + dst_static:
            t.zero_()
        regular.wait(regular.post(sb.to(dev), db.to(dev)))

        p = _Params()
        ctypes.memmove(ctypes.byref(p), ctypes.byref(static_path._p), ctypes.sizeof(_Params))
        p.n_pairs = n
        p.src_blocks = p.dst_blocks = p.done_counter = None  # ignored by the static entry point
        p.host_flag, p.host_seq = flag.data_ptr(), round_no
        p.done_signal, p.done_value = signal.data_ptr(), 5
        rc = fn(ctypes.byref(p), sb.data_ptr(), db.data_ptr(), ctypes.c_void_p(stream.cuda_stream))
        assert rc == 0, rc
        torch.cuda.synchronize(dev)
        assert int(flag[0]) == round_no
        assert signal.tolist() == [5 * round_no, 0]
        for want, got in zip(dst_regular, dst_static):
            assert torch.equal(want, got)
            assert bool(want.any())

    # Over capacity: refused, nothing launched, destination untouched.
    before = [t.clone() for t in dst_static]
    p.n_pairs = max_pairs + 1
    big = torch.zeros(max_pairs + 1, dtype=torch.int32)
    assert fn(ctypes.byref(p), big.data_ptr(), big.data_ptr(), ctypes.c_void_p(stream.cuda_stream)) == ERR_TOO_LARGE
    torch.cuda.synchronize(dev)
    for x, y in zip(before, dst_static):
        assert torch.equal(x, y)
    regular.close()
    static_path.close()

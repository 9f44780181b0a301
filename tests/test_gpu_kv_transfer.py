"""Fused KV transfer kernel against the plain PyTorch statement of the same operation.
Uses a second GPU for the receiver when one is present, else both caches live on cuda:0."""
import pytest
import torch

from nixl_b200 import nixl_agent, nixl_agent_config
from nixl_b200.ops import KVLayout, KVTransfer, reference_kv_transfer

pytestmark = pytest.mark.gpu


def _setup(tag, n_tensors, blocks, src_heads, dst_heads, fp8, dst_order="NHD"):
    src_dev = torch.device("cuda:0")
    dst_dev = torch.device("cuda:1" if torch.cuda.device_count() > 1 else "cuda:0")
    cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"])
    a, b = nixl_agent(f"{tag}_prefill", cfg), nixl_agent(f"{tag}_decode", cfg)
    g = torch.Generator(device=src_dev).manual_seed(0)
    src = [torch.randn(blocks, 16, src_heads, 128, device=src_dev, dtype=torch.bfloat16, generator=g) for _ in range(n_tensors)]
    shape = (blocks, 16, dst_heads, 128) if dst_order == "NHD" else (blocks, dst_heads, 16, 128)
    dst = [torch.zeros(shape, device=dst_dev, dtype=torch.uint8 if fp8 else torch.bfloat16) for _ in range(n_tensors)]
    a.register_memory(src)
    b.register_memory(dst)
    a.add_remote_agent(b.get_agent_metadata())
    remote = [(t.data_ptr(), t.numel() * t.element_size(), t.get_device()) for t in dst]
    return a, b, src, dst, remote


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("head_offset", [0, 2])
def test_gather_reshard_cast(fp8, head_offset):
    a, b, src, dst, remote = _setup(f"kv{int(fp8)}{head_offset}", 6, 96, 2, 4, fp8)
    xfer = KVTransfer(a, src, KVLayout(16, 2, 128), b.name, remote, KVLayout(16, 4, 128, elem_bytes=1 if fp8 else 2),
                      dst_head_offset=head_offset, cast_fp8=fp8, scale=0.5 if fp8 else 1.0)
    g = torch.Generator(device="cuda:0").manual_seed(1)
    sb = torch.randperm(96, device="cuda:0", generator=g)[:77].int()
    db = torch.randperm(96, device="cuda:0", generator=g)[:77].int()
    for _ in range(2):  # second round re-uses the prepared path
        for d in dst:
            d.zero_()
        torch.cuda.synchronize()
        xfer.wait(xfer.post(sb, db))
        torch.cuda.synchronize()
        for s, d in zip(src, dst):
            if fp8:
                want = reference_kv_transfer(s, torch.zeros(d.shape, dtype=torch.float8_e4m3fn, device=s.device), sb, db,
                                             head_offset, True, 0.5).view(torch.uint8)
            else:
                want = reference_kv_transfer(s, torch.zeros(d.shape, dtype=d.dtype, device=s.device), sb, db, head_offset)
            assert torch.equal(d.to(s.device), want)
    xfer.close()


def test_hnd_receiver_layout_and_signal():
    a, b, src, dst, remote = _setup("kvhnd", 3, 40, 2, 4, False, dst_order="HND")
    signal = torch.zeros(8, dtype=torch.int64, device=dst[0].device)
    b.register_memory(signal)
    a.add_remote_agent(b.get_agent_metadata())
    view = a.prep_mem_view(a.get_remote_descs([(signal.data_ptr(), 64, signal.get_device(), b.name)], "VRAM"))
    xfer = KVTransfer(a, src, KVLayout(16, 2, 128), b.name, remote, KVLayout(16, 4, 128, order="HND"), dst_head_offset=1)
    sb = torch.arange(40, device="cuda:0").int()
    db = torch.arange(39, -1, -1, device="cuda:0").int()
    # The signal address at the receiver is reachable from the sender GPU as a peer pointer; in
    # one process that is the pointer itself.
    xfer.wait(xfer.post(sb, db, done_signal_ptr=signal.data_ptr(), done_value=5))
    torch.cuda.synchronize()
    assert int(signal[0]) == 5
    for s, d in zip(src, dst):
        want = torch.zeros(40, 16, 4, 128, dtype=s.dtype, device=s.device)
        reference_kv_transfer(s, want, sb, db, 1)
        assert torch.equal(d.to(s.device), want.permute(0, 2, 1, 3).contiguous())
    a.release_mem_view(view)
    xfer.close()


def test_block_ids_outside_the_cache_are_skipped_and_reported():
    """Block tables are device data nobody validated: the kernel checks every id against the registered range of its
    cache tensor on both sides, skips a block that does not fit and reports it; the other blocks arrive.  The caches
    here are the first 8 blocks of 16-block allocations, so even an unchecked id would stay inside memory this test owns."""
    src_dev = torch.device("cuda:0")
    dst_dev = torch.device("cuda:1" if torch.cuda.device_count() > 1 else "cuda:0")
    cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"])
    a, b = nixl_agent("kvoob_prefill", cfg), nixl_agent("kvoob_decode", cfg)
    g = torch.Generator(device=src_dev).manual_seed(3)
    src_all = [torch.randn(16, 16, 2, 128, device=src_dev, dtype=torch.bfloat16, generator=g) for _ in range(2)]
    dst_all = [torch.zeros(16, 16, 4, 128, device=dst_dev, dtype=torch.bfloat16) for _ in range(2)]
    src, dst = [t[:8] for t in src_all], [t[:8] for t in dst_all]  # what is registered and put into the views
    a.register_memory(src)
    b.register_memory(dst)
    a.add_remote_agent(b.get_agent_metadata())
    remote = [(t.data_ptr(), t.numel() * t.element_size(), t.get_device()) for t in dst]
    xfer = KVTransfer(a, src, KVLayout(16, 2, 128), b.name, remote, KVLayout(16, 4, 128))
    good_s = torch.tensor([0, 3, 7], device="cuda:0", dtype=torch.int32)
    good_d = torch.tensor([7, 1, 0], device="cuda:0", dtype=torch.int32)
    xfer.wait(xfer.post(good_s, good_d))  # in range: no report
    for bad_s, bad_d in (([0, 8, 7], [7, 1, 0]), ([0, 3, 7], [7, 9, 0]), ([0, -1, 7], [7, 1, 0])):
        for d in dst_all:
            d.zero_()
        torch.cuda.synchronize()
        sb = torch.tensor(bad_s, device="cuda:0", dtype=torch.int32)
        db = torch.tensor(bad_d, device="cuda:0", dtype=torch.int32)
        with pytest.raises(IndexError):
            xfer.wait(xfer.post(sb, db))
        torch.cuda.synchronize()
        for s, d_all in zip(src_all, dst_all):
            assert torch.equal(d_all[7, :, :2].to(src_dev), s[0]) and torch.equal(d_all[0, :, :2].to(src_dev), s[7])  # the valid pairs arrived
            assert int(d_all[1].abs().sum()) == 0 and int(d_all[8:].abs().sum()) == 0  # the bad pair moved nothing, inside or outside the cache
    xfer.wait(xfer.post(good_s, good_d))  # the report was cleared
    xfer.close()


def test_rejects_bad_arguments():
    a, b, src, dst, remote = _setup("kvbad", 2, 8, 2, 4, False)
    with pytest.raises(ValueError):
        KVTransfer(a, src, KVLayout(16, 2, 128), b.name, remote, KVLayout(16, 4, 128), dst_head_offset=3)
    xfer = KVTransfer(a, src, KVLayout(16, 2, 128), b.name, remote, KVLayout(16, 4, 128))
    with pytest.raises(TypeError):
        xfer.post(torch.zeros(4, device="cuda:0"), torch.zeros(4, device="cuda:0"))
    xfer.close()

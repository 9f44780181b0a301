#!/usr/bin/env python
"""Small, self-terminating cases of each hot kernel, sized for a profiler capture.

Inputs are larger than L2 (126 MB) where DRAM figures matter, hold at most a few GB and launch
the kernel of interest a handful of times.  One GPU only.

    python benchmarks/profile_cases.py copy|kv|ep|ep_push|ep_rr|gemm|gemm_pair|gemm_mx
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from nixl_b200 import _bindings as nb  # noqa: E402
from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402


def _wait(agent, h):
    while agent.agent.getXferStatus(h) != nb.NIXL_SUCCESS:
        pass


def case_copy():
    a = nixl_agent("prof_a", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
    b = nixl_agent("prof_b", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
    src = torch.randint(0, 255, (512 << 20,), dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros_like(src)
    a.register_memory(src)
    b.register_memory(dst)
    a.add_remote_agent(b.get_agent_metadata())
    h = a.initialize_xfer("WRITE", src, dst, "prof_b")
    for _ in range(4):
        a.agent.postXferReq(h)
        _wait(a, h)
    torch.cuda.synchronize()
    assert torch.equal(src, dst)


def case_kv():
    from nixl_b200.ops import KVLayout, KVTransfer

    cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"])
    a, b = nixl_agent("prof_kp", cfg), nixl_agent("prof_kd", cfg)
    blocks, tensors = 2048, 16
    src = [torch.randn(blocks, 16, 2, 128, device="cuda:0", dtype=torch.bfloat16) for _ in range(tensors)]
    dst = [torch.zeros(blocks, 16, 4, 128, device="cuda:0", dtype=torch.bfloat16) for _ in range(tensors)]
    a.register_memory(src)
    b.register_memory(dst)
    a.add_remote_agent(b.get_agent_metadata())
    x = KVTransfer(a, src, KVLayout(16, 2, 128), "prof_kd", [(t.data_ptr(), t.numel() * 2, 0) for t in dst], KVLayout(16, 4, 128), dst_head_offset=2)
    sb = torch.randperm(blocks, device="cuda:0").int()
    db = torch.randperm(blocks, device="cuda:0").int()
    for _ in range(4):
        x.wait(x.post(sb, db))
    torch.cuda.synchronize()


def case_ep(pull=True, rank_reduce=False):
    """Throughput dispatch and combine on one rank; the combine reads the exposed buffer (pull, what a
    pipeline with the expert GEMM in between does) or, as `ep_push`, stores rows to the home rank first; as `ep_rr`
    dispatch is given the weights and the combine is the rank-reduced pair of kernels."""
    from nixl_b200.parallel import Buffer

    T, H, E, K = 1024, 7168, 32, 8
    buf = Buffer(0, 1, E, H, T, K, device=torch.device("cuda:0"))
    x = torch.randn(T, H, device="cuda:0", dtype=torch.bfloat16)
    w, idx = torch.topk(torch.softmax(torch.randn(T, E, device="cuda:0"), -1), K, -1)
    idx, w = idx.long().contiguous(), w.float().contiguous()
    for _ in range(3):
        rx, sc, h = buf.dispatch(x, idx, topk_weights=w if rank_reduce else None)
        y = buf.get_next_combine_buffer(h) if pull else torch.empty(rx.shape[0], H, device="cuda:0", dtype=torch.bfloat16)
        buf.combine(y, idx, w, h)
    torch.cuda.synchronize()
    assert buf.status == 0


def case_ep_push():
    case_ep(pull=False)


def case_ep_rr():
    case_ep(rank_reduce=True)


def _gemm_inputs(G=8, N=2048, K=7168, rows_per=1024, pow2=False):
    from nixl_b200.parallel import per_token_cast_to_fp8

    x = torch.randn(G * rows_per, K, device="cuda:0", dtype=torch.bfloat16)
    a, sa = per_token_cast_to_fp8(x, round_scale=pow2)
    rs = (torch.arange(G, device="cuda:0") * rows_per).int()
    rc = torch.full((G,), rows_per, device="cuda:0", dtype=torch.int32)
    return a.contiguous(), sa.contiguous(), rs, rc


def _case_gemm(tile_mode):
    from nixl_b200.ops import grouped_gemm_fp8, quantize_weights

    G, N, K = 8, 2048, 7168
    a, sa, rs, rc = _gemm_inputs(G, N, K)
    wq, sw = quantize_weights(torch.randn(G, N, K, device="cuda:0") * 0.02)
    for _ in range(3):
        out = grouped_gemm_fp8(a, sa, wq, sw, rs, rc, tile_mode=tile_mode)
    torch.cuda.synchronize()
    assert int(out._nixl_status.item()) == 0


def case_gemm():
    """128 x 128 tiles on single CTAs (groupedGemmKernel)."""
    _case_gemm(1)


def case_gemm_pair():
    """256 x 256 tiles on CTA pairs, fp32 block scales (groupedGemmPairKernel)."""
    _case_gemm(2)


def case_gemm_mx():
    """256 x 256 tiles on CTA pairs, power-of-two scales in the tensor core (groupedGemmMxPairKernel)."""
    from nixl_b200.ops import grouped_gemm_mxfp8, quantize_weights_ue8m0, to_ue8m0

    G, N, K = 8, 2048, 7168
    a, sa, rs, rc = _gemm_inputs(G, N, K, pow2=True)
    wq, swb = quantize_weights_ue8m0(torch.randn(G, N, K, device="cuda:0") * 0.02)
    sab = to_ue8m0(sa)
    for _ in range(3):
        out = grouped_gemm_mxfp8(a, sab, wq, swb, rs, rc)
    torch.cuda.synchronize()
    assert int(out._nixl_status.item()) == 0


if __name__ == "__main__":
    {"copy": case_copy, "kv": case_kv, "ep": case_ep, "ep_push": case_ep_push, "ep_rr": case_ep_rr, "gemm": case_gemm, "gemm_pair": case_gemm_pair, "gemm_mx": case_gemm_mx}[sys.argv[1]]()
    print("ok", sys.argv[1])

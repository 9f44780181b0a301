"""One tiny launch of each fused kernel on cuda:0, with a correctness check."""
import torch


def run() -> None:
    from nixl_b200 import nixl_agent, nixl_agent_config

    from .kv_transfer import KVLayout, KVTransfer, reference_kv_transfer

    dev = torch.device("cuda:0")
    cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"])
    a, b = nixl_agent("smoke_kv_p", cfg), nixl_agent("smoke_kv_d", cfg)
    src = [torch.randn(32, 16, 2, 128, device=dev, dtype=torch.bfloat16) for _ in range(4)]
    dst = [torch.zeros(32, 16, 4, 128, device=dev, dtype=torch.bfloat16) for _ in range(4)]
    a.register_memory(src)
    b.register_memory(dst)
    a.add_remote_agent(b.get_agent_metadata())
    xfer = KVTransfer(
        a, src, KVLayout(16, 2, 128), "smoke_kv_d", [(t.data_ptr(), t.numel() * 2, 0) for t in dst], KVLayout(16, 4, 128), dst_head_offset=2
    )
    sb = torch.randperm(32, device=dev)[:24].int()
    db = torch.randperm(32, device=dev)[:24].int()
    xfer.wait(xfer.post(sb, db))
    torch.cuda.synchronize()
    for s, d in zip(src, dst):
        want = reference_kv_transfer(s, torch.zeros_like(d), sb, db, 2)
        assert torch.equal(d, want), "fused KV transfer differs from the PyTorch reference"
    xfer.close()

    # Expert-parallel layer on one rank: dispatch (exponent-byte scales) -> block-scaled grouped GEMM writing
    # into the exposed combine buffer -> pull combine; then the fp32-scale GEMM kernels on the same rows.
    from ..parallel import Buffer, dequant_fp8, per_token_cast_to_fp8
    from .grouped_gemm import (
        from_ue8m0,
        grouped_gemm_fp8,
        grouped_gemm_mxfp8,
        quantize_weights,
        quantize_weights_ue8m0,
        reference_grouped_gemm,
    )

    T, H, E, K = 64, 1024, 4, 2
    buf = Buffer(0, 1, E, H, T, K, device=dev, low_latency_mode=False)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    wts, idx = torch.topk(torch.softmax(torch.randn(T, E, device=dev), -1), K, -1)
    idx, wts = idx.long().contiguous(), wts.float().contiguous()
    w = torch.randn(E, H, H, device=dev) * 0.05
    wq, swb = quantize_weights_ue8m0(w)
    rx, packed, handle = buf.dispatch(x, idx, use_fp8=True, use_ue8m0=True)
    y = buf.get_next_combine_buffer(handle)
    rows = buf.compact_rows
    grouped_gemm_mxfp8(rx[:rows], packed[:rows].contiguous(), wq, swb, handle.expert_offsets, handle.recv_count, out=y)
    out = buf.combine(y, idx, wts, handle)
    torch.cuda.synchronize()
    assert buf.status == 0, "EP kernels reported a timeout"
    q, s = per_token_cast_to_fp8(x, round_scale=True)
    xd = dequant_fp8(q, s)
    wd = (wq.float().view(E, H // 128, 128, H // 128, 128) * from_ue8m0(swb)[:, :, None, :, None]).view(E, H, H)
    want = torch.zeros(T, H, device=dev)
    for k in range(K):
        want += wts[:, k : k + 1] * torch.einsum("th,tnh->tn", xd, wd[idx[:, k]]).to(torch.bfloat16).float()
    torch.testing.assert_close(out.float(), want.to(torch.bfloat16).float(), rtol=3e-2, atol=3e-2)

    rx2, sc2, h2 = buf.dispatch(x, idx, use_fp8=True)
    wq2, sw2 = quantize_weights(w)
    torch.cuda.synchronize()
    ref = reference_grouped_gemm(rx2[:rows], sc2[:rows], wq2, sw2, h2.expert_offsets[:E], h2.recv_count)
    for mode in (1, 2):
        got = grouped_gemm_fp8(rx2[:rows], sc2[:rows], wq2, sw2, h2.expert_offsets[:E].contiguous(), h2.recv_count, tile_mode=mode)
        torch.cuda.synchronize()
        assert int(got._nixl_status.item()) == 0
        for e in range(E):
            s0, c = int(h2.expert_offsets[e]), int(h2.recv_count[e])
            if c:
                err = (got[s0 : s0 + c].float() - ref[s0 : s0 + c]).abs().max() / (ref[s0 : s0 + c].abs().max() + 1e-6)
                assert float(err) < 2e-2, f"grouped GEMM (tile mode {mode}) differs from the fp32 reference"
    buf.destroy()

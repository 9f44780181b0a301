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

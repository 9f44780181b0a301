#!/usr/bin/env python
"""Expert-parallel dispatch -> (grouped fp8 GEMM) -> combine.

Single process: ``python examples/ep_dispatch_combine.py``; several GPUs:
``python -m torch.distributed.run --nproc-per-node N examples/ep_dispatch_combine.py``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from nixl_b200.ops import grouped_gemm_fp8, quantize_weights  # noqa: E402
from nixl_b200.parallel import Buffer  # noqa: E402


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl")
    tokens, hidden, experts_per_rank, topk, inter = 128, 2048, 8, 4, 512
    experts = experts_per_rank * world
    buf = Buffer(rank, world, experts, hidden, tokens, topk)
    buf.connect_ranks()
    x = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    weights, idx = torch.topk(torch.softmax(torch.randn(tokens, experts, device="cuda"), -1), topk, -1)
    idx, weights = idx.long().contiguous(), weights.float().contiguous()

    (recv_x, recv_scales), recv_count, handle, _, _ = buf.low_latency_dispatch(x, idx, use_fp8=True)
    wq, sw = quantize_weights(torch.randn(experts_per_rank, inter, hidden, device="cuda") * 0.02)
    rows = recv_x.shape[0] * recv_x.shape[1]
    up = grouped_gemm_fp8(recv_x.view(rows, hidden), recv_scales.view(rows, -1), wq, sw, handle.expert_offsets, recv_count)
    # stand-in for the rest of the expert MLP: project back to `hidden` with plain torch
    down = torch.randn(inter, hidden, device="cuda", dtype=torch.bfloat16) * 0.02
    y = (up @ down).view(experts_per_rank, -1, hidden)
    out, _, _ = buf.low_latency_combine(y, idx, weights, handle)
    torch.cuda.synchronize()
    print(f"rank {rank}: received {int(recv_count.sum())} rows, combined {tuple(out.shape)}, status {buf.status}")
    buf.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

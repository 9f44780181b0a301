#!/usr/bin/env python
"""A whole expert layer without staging copies, with power-of-two scales end to end:

    throughput dispatch (e4m3 rows + exponent-byte scales)
      -> block-scaled grouped GEMM (the tensor core applies the scales; output written straight into the
         buffer the other ranks will read)
      -> pull combine (every token's home rank loads its rows from the expert ranks and reduces them)

Single process: ``python examples/ep_block_scaled_layer.py``; several GPUs:
``python -m torch.distributed.run --nproc-per-node N examples/ep_block_scaled_layer.py``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from nixl_b200.ops import grouped_gemm_mxfp8, quantize_weights_ue8m0  # noqa: E402
from nixl_b200.parallel import Buffer  # noqa: E402


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl")
    tokens, hidden, experts_per_rank, topk = 1024, 2048, 8, 4
    experts = experts_per_rank * world
    buf = Buffer(rank, world, experts, hidden, tokens, topk, low_latency_mode=False)
    buf.connect_ranks()
    x = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    weights, idx = torch.topk(torch.softmax(torch.randn(tokens, experts, device="cuda"), -1), topk, -1)
    idx, weights = idx.long().contiguous(), weights.float().contiguous()
    # hidden -> hidden so that the GEMM's output is what combine returns (a real layer has up / act / down here)
    wq, sw = quantize_weights_ue8m0(torch.randn(experts_per_rank, hidden, hidden, device="cuda") * 0.02)

    recv_x, recv_scales, handle = buf.dispatch(x, idx, use_fp8=True, use_ue8m0=True)
    y = buf.get_next_combine_buffer(handle)  # [rows, hidden] bf16 inside the symmetric buffer
    grouped_gemm_mxfp8(recv_x, recv_scales, wq, sw, handle.expert_offsets, handle.recv_count, out=y)
    out = buf.combine(y, idx, weights, handle)  # y lies in the exposed buffer: pull mode, no copy
    torch.cuda.synchronize()
    print(f"rank {rank}: {int(handle.recv_count.sum())} rows through the experts, combined {tuple(out.shape)}, status {buf.status}")
    buf.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

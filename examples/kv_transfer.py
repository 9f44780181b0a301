#!/usr/bin/env python
"""Fused paged-KV transfer from a prefill cache (2 KV heads per GPU) into a decode cache
(4 KV heads per GPU) with block-table gather/scatter and an optional fp8 cast.  Needs a GPU."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402
from nixl_b200.ops import KVLayout, KVTransfer  # noqa: E402


def main(fp8=False):
    src_dev = torch.device("cuda:0")
    dst_dev = torch.device("cuda:1" if torch.cuda.device_count() > 1 else "cuda:0")
    cfg = nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"])
    prefill, decode = nixl_agent("prefill0", cfg), nixl_agent("decode0", cfg)
    layers, blocks = 4, 512
    src = [torch.randn(blocks, 16, 2, 128, device=src_dev, dtype=torch.bfloat16) for _ in range(2 * layers)]
    dst = [torch.zeros(blocks, 16, 4, 128, device=dst_dev, dtype=torch.uint8 if fp8 else torch.bfloat16) for _ in range(2 * layers)]
    prefill.register_memory(src)
    decode.register_memory(dst)
    prefill.add_remote_agent(decode.get_agent_metadata())
    path = KVTransfer(prefill, src, KVLayout(16, 2, 128), "decode0",
                      [(t.data_ptr(), t.numel() * t.element_size(), t.get_device()) for t in dst],
                      KVLayout(16, 4, 128, elem_bytes=1 if fp8 else 2), dst_head_offset=2, cast_fp8=fp8)
    request_blocks = torch.randperm(blocks, device=src_dev)[:256].int()   # where the request lives in the prefill cache
    decode_blocks = torch.randperm(blocks, device=src_dev)[:256].int()    # where the decode side wants it
    ticket = path.post(request_blocks, decode_blocks)
    path.wait(ticket)
    print("moved", path.bytes_moved(256), "source bytes,", "fp8" if fp8 else "bf16", "on the wire")
    path.close()


if __name__ == "__main__":
    main(fp8="--fp8" in sys.argv)

#!/usr/bin/env python
"""Two agents exchange metadata and move a tensor with a completion notification.

Runs on CPU tensors by default (``--device cuda`` uses two GPUs when present).  Follows the
flow of the reference's examples/python/basic_two_peers.py in one process."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    args = ap.parse_args()
    d0 = "cuda:0" if args.device == "cuda" else "cpu"
    d1 = ("cuda:1" if torch.cuda.device_count() > 1 else "cuda:0") if args.device == "cuda" else "cpu"

    initiator = nixl_agent("initiator", nixl_agent_config(backends=["NVLINK"]))
    target = nixl_agent("target", nixl_agent_config(backends=["NVLINK"]))
    src = torch.arange(1 << 20, dtype=torch.float32, device=d0)
    dst = torch.zeros(1 << 20, dtype=torch.float32, device=d1)
    initiator.register_memory(src)
    target.register_memory(dst)

    # Metadata travels as an opaque blob (any side channel works).
    print("target is known as", initiator.add_remote_agent(target.get_agent_metadata()))

    handle = initiator.initialize_xfer("WRITE", src, dst, "target", b"tensor-ready")
    state = initiator.transfer(handle)
    while state == "PROC":
        state = initiator.check_xfer_state(handle)
    assert state == "DONE"
    while not target.check_remote_xfer_done("initiator", b"tensor-ready"):
        pass
    assert torch.equal(src.cpu(), dst.cpu())
    print("moved", src.numel() * 4, "bytes with backend", initiator.query_xfer_backend(handle))
    initiator.release_xfer_handle(handle)


if __name__ == "__main__":
    main()

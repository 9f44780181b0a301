#!/usr/bin/env python
"""Storage round trip: buffer -> file -> buffer through a file backend.

The flow of the reference's examples/python/nixl_gds_example.py.  With ``--device cuda`` the
buffers are CUDA tensors and the GDS backend moves them (staged through pinned host memory on
machines without GPUDirect Storage); on the host the POSIX backend does the same for DRAM."""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402


def run(agent, handle):
    state = agent.transfer(handle)
    while state == "PROC":
        state = agent.check_xfer_state(handle)
    assert state == "DONE", state


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--path", default="")
    ap.add_argument("--mib", type=int, default=16)
    args = ap.parse_args()
    backend = "GDS" if args.device == "cuda" else "POSIX"
    agent = nixl_agent("storage_agent", nixl_agent_config(backends=[]))
    agent.create_backend(backend, {})
    n = args.mib << 20
    src = torch.randint(0, 255, (n,), dtype=torch.uint8, device=args.device)
    back = torch.zeros_like(src)
    agent.register_memory(src)
    agent.register_memory(back)
    path = args.path or os.path.join(tempfile.mkdtemp(), "nixl_storage_example.bin")
    fd = os.open(path, os.O_RDWR | os.O_CREAT, 0o644)
    try:
        reg = agent.register_memory([(0, n, fd, "")], "FILE")
        file_descs = agent.get_xfer_descs([(0, n, fd)], "FILE")
        w = agent.initialize_xfer("WRITE", src, file_descs, "storage_agent", backends=[backend])
        run(agent, w)
        r = agent.initialize_xfer("READ", back, file_descs, "storage_agent", backends=[backend])
        run(agent, r)
        assert torch.equal(src.cpu(), back.cpu()) and os.fstat(fd).st_size == n
        print(f"{n} bytes went to {path} and back through {backend}")
        agent.release_xfer_handle(w)
        agent.release_xfer_handle(r)
        agent.deregister_memory(reg)
    finally:
        os.close(fd)
        if not args.path:
            os.unlink(path)


if __name__ == "__main__":
    main()

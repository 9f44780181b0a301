#!/usr/bin/env python
"""Prepared descriptor lists: prepare both sides once, then build many transfers by index.

The flow of the reference's examples/python/expanded_two_peers.py in one process: a paged buffer is
registered on each side, both sides are prepared block by block, and transfers are made from index
selections (a different subset of blocks each time), in both directions, with notifications."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402

BLOCK, BLOCKS = 4096, 32


def wait(agent, handle):
    state = agent.transfer(handle)
    while state == "PROC":
        state = agent.check_xfer_state(handle)
    assert state == "DONE", state


def main():
    target = nixl_agent("target", nixl_agent_config(backends=["NVLINK"]))
    initiator = nixl_agent("initiator", nixl_agent_config(backends=["NVLINK"]))
    print("NVLINK parameters:", initiator.get_backend_params("NVLINK"), "memory kinds:", initiator.get_backend_mem_types("NVLINK"))

    t_buf = torch.zeros(BLOCKS * BLOCK, dtype=torch.uint8)
    i_buf = (torch.arange(BLOCKS * BLOCK) % 251).to(torch.uint8)
    target.register_memory(t_buf)
    initiator.register_memory(i_buf)
    initiator.add_remote_agent(target.get_agent_metadata())

    # The target tells the initiator where its blocks are: descriptors serialise to bytes.
    t_blocks = [(t_buf.data_ptr() + b * BLOCK, BLOCK, 0) for b in range(BLOCKS)]
    wire = target.get_serialized_descs(target.get_xfer_descs(t_blocks, "DRAM"))
    remote_descs = initiator.deserialize_descs(wire)

    i_blocks = [(i_buf.data_ptr() + b * BLOCK, BLOCK, 0) for b in range(BLOCKS)]
    local_side = initiator.prep_xfer_dlist("NIXL_INIT_AGENT", i_blocks, "DRAM")
    remote_side = initiator.prep_xfer_dlist("target", remote_descs)

    # WRITE the even blocks into the odd slots of the target, then READ two of them back elsewhere.
    evens, odds = list(range(0, BLOCKS, 2)), list(range(1, BLOCKS, 2))
    w = initiator.make_prepped_xfer("WRITE", local_side, evens, remote_side, odds, b"evens-written")
    wait(initiator, w)
    while not target.check_remote_xfer_done("initiator", b"evens-written"):
        pass
    assert torch.equal(t_buf.view(BLOCKS, BLOCK)[odds], i_buf.view(BLOCKS, BLOCK)[evens])

    r = initiator.make_prepped_xfer("READ", local_side, [1, 3], remote_side, [5, 7])
    wait(initiator, r)
    assert torch.equal(i_buf.view(BLOCKS, BLOCK)[[1, 3]], t_buf.view(BLOCKS, BLOCK)[[5, 7]])
    print("estimated cost of the read (us, margin, method):", initiator.estimate_xfer_cost(r))

    for h in (w, r):
        initiator.release_xfer_handle(h)
    for side in (local_side, remote_side):
        initiator.release_dlist_handle(side)
    initiator.remove_remote_agent("target")
    print("prepared transfers done")


if __name__ == "__main__":
    main()

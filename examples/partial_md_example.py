#!/usr/bin/env python
"""Partial metadata: hand a peer only the registrations it needs, and take them back again.

The flow of the reference's examples/python/partial_md_example.py in one process: the target
registers two buffers, first ships connection information plus buffer A only, later buffer B, and
finally invalidates what it published."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402


def run(agent, handle):
    state = agent.transfer(handle)
    while state == "PROC":
        state = agent.check_xfer_state(handle)
    return state


def main():
    target = nixl_agent("target", nixl_agent_config(backends=["NVLINK"]))
    initiator = nixl_agent("initiator", nixl_agent_config(backends=["NVLINK"]))
    a, b = torch.zeros(4096, dtype=torch.uint8), torch.zeros(4096, dtype=torch.uint8)
    src = torch.full((4096,), 7, dtype=torch.uint8)
    reg_a, reg_b = target.register_memory(a), target.register_memory(b)
    initiator.register_memory(src)

    # Connection information and buffer A only.
    blob = target.get_partial_agent_metadata(reg_a, True, ["NVLINK"])
    assert initiator.add_remote_agent(blob) == "target"
    assert initiator.check_remote_metadata("target", target.get_xfer_descs(a))
    assert not initiator.check_remote_metadata("target", target.get_xfer_descs(b))
    h = initiator.initialize_xfer("WRITE", src, target.get_xfer_descs(a), "target")
    assert run(initiator, h) == "DONE" and int(a.sum()) == 7 * 4096
    initiator.release_xfer_handle(h)
    try:
        initiator.initialize_xfer("WRITE", src, target.get_xfer_descs(b), "target")
        raise SystemExit("buffer B should not be reachable yet")
    except Exception as e:
        print("buffer B is not known to the initiator yet:", type(e).__name__)

    # Buffer B follows, without connection information this time.
    initiator.add_remote_agent(target.get_partial_agent_metadata(reg_b, False, ["NVLINK"]))
    h = initiator.initialize_xfer("WRITE", src, target.get_xfer_descs(b), "target")
    assert run(initiator, h) == "DONE" and int(b.sum()) == 7 * 4096
    initiator.release_xfer_handle(h)

    # The initiator drops what it knows about the target.
    initiator.remove_remote_agent("target")
    assert not initiator.check_remote_metadata("target")
    print("partial metadata example done")


if __name__ == "__main__":
    main()

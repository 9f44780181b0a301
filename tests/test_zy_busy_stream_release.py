"""Release of a request whose copy kernel is still queued behind other work of the caller's stream.

Kept in a file of its own, late in the collection order: the scenario holds the GPU for a tenth of a second per
round and depends on how the runtime schedules three streams against each other, so a hiccup here should not keep
the rest of the GPU suite from running."""
import time

import pytest
import torch

from nixl_b200 import nixl_agent, nixl_agent_config

pytestmark = pytest.mark.gpu


def _wait(agent, handle, seconds=30.0):
    end = time.monotonic() + seconds
    state = "PROC"
    while time.monotonic() < end:
        state = agent.check_xfer_state(handle)
        if state != "PROC":
            break
    return state


def _pair(tag, params=None):
    cfg = nixl_agent_config(enable_prog_thread=False, backends=[])
    a, b = nixl_agent(f"{tag}_a", cfg), nixl_agent(f"{tag}_b", cfg)
    a.create_backend("NVLINK", params or {})
    b.create_backend("NVLINK", params or {})
    return a, b


def _connect(a, b):
    a.add_remote_agent(b.get_agent_metadata())
    b.add_remote_agent(a.get_agent_metadata())


def test_release_right_after_post_on_a_busy_caller_stream():
    """The request is posted on the caller's stream behind a long-running kernel and released at
    once: the release must wait for the copy kernel (it reads the request's descriptor table and
    writes its completion word), and the bytes must be intact afterwards."""
    a, b = _pair("rel_stream", {"coalesce": "false"})
    n_desc, size = 64, 1 << 16  # more than 32 descriptors: the table lives in device memory
    src = torch.randint(0, 255, (n_desc, size), dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros_like(src)
    a.register_memory(src)
    b.register_memory(dst)
    _connect(a, b)
    stream = torch.cuda.Stream()
    for _ in range(3):
        dst.zero_()
        torch.cuda.synchronize()
        h = a.initialize_xfer("WRITE", [src[i] for i in range(n_desc)], [dst[i] for i in range(n_desc)], b.name)
        with torch.cuda.stream(stream):
            torch.cuda._sleep(200_000_000)  # ~0.1 s of device time in front of the copy
            state = a.transfer(h, custom_param=f"stream={stream.cuda_stream}")
            assert state in ("DONE", "PROC"), f"post on the busy stream: {state}"
        a.release_xfer_handle(h)
        # another request right away: it must not be handed a completion word that the first kernel still writes
        h2 = a.initialize_xfer("WRITE", src[0], dst[0], b.name)
        state = a.transfer(h2)
        assert state in ("DONE", "PROC"), f"post of the second request: {state}"
        state = _wait(a, h2)
        assert state == "DONE", f"second request: {state}"
        a.release_xfer_handle(h2)
        torch.cuda.synchronize()
        wrong = (src != dst).any(dim=1).nonzero().flatten().tolist()
        assert not wrong, f"rows that differ after both requests: {wrong[:8]} (of {len(wrong)})"

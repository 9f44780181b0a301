#!/usr/bin/env python
"""Metadata through a central store instead of a side channel.

The flow of the reference's examples/cpp/nixl_etcd_example.cpp: agents publish their metadata under
their name (``send_local_metadata``), fetch a peer's by name (``fetch_remote_metadata``), transfer,
and withdraw it again (``invalidate_local_metadata``).  The store is chosen by the environment:
``NIXL_ETCD_ENDPOINTS=http://host:2379`` for etcd (v3 JSON gateway) or
``NIXL_TCPSTORE_ENDPOINT=host:port`` for a torch TCPStore.  With neither set this script starts a
TCPStore in-process so that it runs anywhere."""
import datetime
import os
import socket
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    server = None
    if not os.environ.get("NIXL_ETCD_ENDPOINTS") and not os.environ.get("NIXL_TCPSTORE_ENDPOINT"):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        server = dist.TCPStore("127.0.0.1", port, is_master=True, wait_for_workers=False, timeout=datetime.timedelta(seconds=20))
        os.environ["NIXL_TCPSTORE_ENDPOINT"] = f"127.0.0.1:{port}"
    from nixl_b200 import nixl_agent, nixl_agent_config

    prefill = nixl_agent("store_prefill", nixl_agent_config(backends=["NVLINK"]))
    decode = nixl_agent("store_decode", nixl_agent_config(backends=["NVLINK"]))
    src, dst = torch.arange(1 << 16, dtype=torch.int32), torch.zeros(1 << 16, dtype=torch.int32)
    prefill.register_memory(src)
    decode.register_memory(dst)

    decode.send_local_metadata()                     # "store_decode" is now in the store
    prefill.fetch_remote_metadata("store_decode")    # asynchronous: poll until it is loaded
    deadline = time.time() + 20
    while not prefill.check_remote_metadata("store_decode"):
        if time.time() > deadline:
            raise SystemExit("metadata did not arrive")
        time.sleep(0.01)

    h = prefill.initialize_xfer("WRITE", src, dst, "store_decode", b"done")
    state = prefill.transfer(h)
    while state == "PROC":
        state = prefill.check_xfer_state(h)
    assert state == "DONE" and torch.equal(src, dst)
    prefill.release_xfer_handle(h)

    decode.invalidate_local_metadata()               # withdrawn: new fetches no longer find it
    print("metadata went through", "etcd" if os.environ.get("NIXL_ETCD_ENDPOINTS") else "the TCPStore", "and", src.numel() * 4, "bytes moved")
    del server


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Prefill worker on one host, decode worker on another: KV blocks cross over the TCP backend.

    decode host:   python kv_blocks_between_hosts.py --role decode  --port 5801
    prefill host:  python kv_blocks_between_hosts.py --role prefill --peer-ip <decode host> --peer-port 5801

Both create the NVLINK and the TCP backend; the agent uses NVLINK when the two sit in one box and TCP otherwise.  The
decode worker publishes where its cache blocks are (`describe_blocks`, sent as a notification once it knows the prefill
worker); the prefill worker prepares both sides once (`KVBlockTransfer`) and then names block numbers only.  Every
request carries a notification ("<i>/<n>:<blocks>"), so the decode worker learns of finished blocks without polling
anything but its agent; requests finish in any order.
Run both on one machine with --peer-ip 127.0.0.1 to try it.
"""
import argparse
import os
import socket
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402
from nixl_b200.ops import KVBlockTransfer, describe_blocks  # noqa: E402

LAYERS, BLOCKS, TOKENS, HEADS, DIM = 4, 64, 16, 8, 128


def caches(device, fill):
    """K and V of every layer: [blocks, tokens, heads, dim] bf16."""
    out = []
    for layer in range(LAYERS):
        for kv in range(2):
            t = torch.zeros(BLOCKS, TOKENS, HEADS, DIM, dtype=torch.bfloat16, device=device)
            if fill:
                t += (torch.arange(BLOCKS, device=device, dtype=torch.float32).view(-1, 1, 1, 1) + 100 * layer + 1000 * kv).to(torch.bfloat16)
            out.append(t)
    return out


def wait_for(what, ready, seconds=60):
    deadline = time.time() + seconds
    while not ready():
        if time.time() > deadline:
            raise TimeoutError(what)
        time.sleep(0.001)


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def decode(args):
    agent = nixl_agent("decode", nixl_agent_config(enable_prog_thread=False, enable_listen_thread=True, listen_port=args.port, backends=args.backends.split(",")))
    kv = caches(args.device, fill=False)
    for t in kv:
        agent.register_memory(t)
    print(f"decode: {len(kv)} cache tensors of {BLOCKS} blocks registered, listening on {args.port}", flush=True)
    wait_for("the prefill worker's metadata", lambda: agent.check_remote_metadata("prefill"), 600)
    agent.send_notif("prefill", b"BLOCKS|" + describe_blocks(agent, kv))
    # Requests finish in any order: every notification says "<i>/<n>:<blocks>", and all n have to be in.
    got = []
    wait_for("the blocks", lambda: got.extend(agent.get_new_notifs().get("prefill", [])) or (got and len(got) == int(got[0].split(b":")[0].split(b"/")[1])), 600)
    landed = sorted(int(x) for m in got for x in m.split(b":")[1].split(b","))
    # block b of the prefill worker went to block BLOCKS - 1 - b here
    for t_index, t in enumerate(kv):
        layer, is_v = divmod(t_index, 2)
        for dst in landed:
            want = float(torch.tensor((BLOCKS - 1 - dst) + 100 * layer + 1000 * is_v, dtype=torch.float32).to(torch.bfloat16))
            assert float(t[dst, 0, 0, 0]) == want and float(t[dst, -1, -1, -1]) == want, (t_index, dst)
    untouched = [b for b in range(BLOCKS) if b not in landed]
    assert all(float(t[b].float().abs().sum()) == 0 for t in kv for b in untouched)
    print(f"decode: {len(landed)} blocks arrived and hold what the prefill worker computed", flush=True)
    agent.send_notif("prefill", b"VERIFIED")


def prefill(args):
    agent = nixl_agent("prefill", nixl_agent_config(enable_prog_thread=False, enable_listen_thread=True, listen_port=free_port(), backends=args.backends.split(",")))
    kv = caches(args.device, fill=True)
    for t in kv:
        agent.register_memory(t)
    agent.fetch_remote_metadata("decode", args.peer_ip, args.peer_port)
    agent.send_local_metadata(args.peer_ip, args.peer_port)
    wait_for("the decode worker's metadata", lambda: agent.check_remote_metadata("decode"))
    got = []
    wait_for("the decode worker's blocks", lambda: got.extend(agent.get_new_notifs().get("decode", [])) or got)
    mover = KVBlockTransfer(agent, kv, "decode", got[0].split(b"|", 1)[1])
    # three requests of scattered blocks, all in flight at once
    requests = [list(range(0, 20, 2)), list(range(21, 41, 3)), [63, 50, 47]]
    t0 = time.time()
    handles = []
    for i, blocks in enumerate(requests):
        there = [BLOCKS - 1 - b for b in blocks]
        tag = f"{i + 1}/{len(requests)}:".encode() + b",".join(str(b).encode() for b in there)
        handles.append(mover.post(blocks, there, "WRITE", tag))
    backend = agent.query_xfer_backend(handles[0])
    for h in handles:
        mover.wait(h)
    n = sum(len(r) for r in requests)
    print(f"prefill: {n} blocks ({mover.bytes_moved(n)} bytes) over {backend} in {time.time() - t0:.3f} s", flush=True)
    wait_for("the decode worker's answer", lambda: agent.check_remote_xfer_done("decode", b"VERIFIED"), 120)
    mover.close()
    print("prefill: the decode worker has verified the blocks", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", required=True, choices=["prefill", "decode"])
    ap.add_argument("--port", type=int, default=5801, help="decode: the port of its metadata listener")
    ap.add_argument("--peer-ip", default="127.0.0.1")
    ap.add_argument("--peer-port", type=int, default=5801)
    ap.add_argument("--device", default="cpu", help="cpu, or cuda:N for caches in GPU memory")
    ap.add_argument("--backends", default="NVLINK,TCP", help="the same list on both sides; \"TCP\" alone forces the sockets inside one box too")
    args = ap.parse_args()
    (decode if args.role == "decode" else prefill)(args)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""A storage server that other agents store blocks on and load blocks from, over two backends at once.

The server owns files; a client owns buffers.  A client asks by notification; the server moves the bytes itself:

    store:  client buffers --(network: TCP or NVLINK, the server READs)--> server buffers --(POSIX WRITE)--> files
    load:   files --(POSIX READ)--> server buffers --(network, the server WRITEs)--> client buffers

Every block goes through the two stages on its own, so block i + 1 is on the network while block i is on the disk.
The client also runs the storage backend locally (its buffers to its own files and back).

    python remote_storage_example.py --role server --agent_name store0 --port 5701 --fileprefix /tmp/store0
    python remote_storage_example.py --role client --agent_name me --agents_file agents.txt --fileprefix /tmp/me

The agents file holds one server per line: "<agent name> <ip address> <port>".  `--buf_size` and `--batch_size` must be
the same on both sides.  Same roles and options as the reference's
examples/python/remote_storage_example/nixl_p2p_storage_example.py; the peers here talk over the TCP backend when they
sit on different hosts and over NVLINK inside one box.
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402


def make_agent(name, port):
    agent = nixl_agent(name, nixl_agent_config(enable_prog_thread=False, enable_listen_thread=True, listen_port=port, backends=["NVLINK", "TCP"]))
    storage = "POSIX"
    agent.create_backend(storage)
    return agent, storage


def wait_done(agent, handles, what, seconds=120):
    """Polls every request of `handles` until none is running."""
    deadline = time.time() + seconds
    pending = list(handles)
    while pending:
        pending = [h for h in pending if _state(agent, h, what) == "PROC"]
        if time.time() > deadline:
            raise TimeoutError(what)


def _state(agent, handle, what):
    st = agent.check_xfer_state(handle)
    if st == "ERR":
        raise RuntimeError(what + " failed")
    return st


class Blocks:
    """`batch` buffers of `size` bytes and as many files, registered with the agent."""

    def __init__(self, agent, prefix, size, batch, fill=None):
        self.agent, self.size, self.batch = agent, size, batch
        self.buffers = [torch.zeros(size, dtype=torch.uint8) if fill is None else torch.full((size,), (fill + i) % 251, dtype=torch.uint8)
                        for i in range(batch)]
        for b in self.buffers:
            agent.register_memory(b)
        self.paths = [f"{prefix}_{i}.bin" for i in range(batch)]
        self.fds = [os.open(p, os.O_RDWR | os.O_CREAT, 0o644) for p in self.paths]
        self.file_regs = agent.register_memory([(0, size, fd, "") for fd in self.fds], "FILE")

    def mem_descs(self, i):
        return self.agent.get_xfer_descs([(self.buffers[i].data_ptr(), self.size, 0)], "DRAM")

    def file_descs(self, i):
        return self.agent.get_xfer_descs([(0, self.size, self.fds[i])], "FILE")

    def close(self):
        for fd in self.fds:
            os.close(fd)


def storage_pass(agent, blocks, op):
    """Every buffer to its file (op WRITE) or back (READ), all requests in flight at once."""
    handles = [agent.initialize_xfer(op, blocks.mem_descs(i), blocks.file_descs(i), agent.name) for i in range(blocks.batch)]
    for h in handles:
        agent.transfer(h)
    wait_done(agent, handles, "storage " + op)
    for h in handles:
        agent.release_xfer_handle(h)


# ---------------------------------------------------------------------------------------------- server
def serve(args):
    agent, _ = make_agent(args.agent_name, args.port)
    blocks = Blocks(agent, args.fileprefix + "_" + args.agent_name, args.buf_size, args.batch_size)
    print(f"{args.agent_name}: serving on port {args.port}", flush=True)
    served = 0
    while args.requests == 0 or served < args.requests:
        for client, msgs in agent.get_new_notifs().items():
            for msg in msgs:
                op, _, blob = msg.partition(b"|")
                if op not in (b"STORE", b"LOAD"):
                    continue
                handle_request(agent, blocks, client, op.decode(), agent.deserialize_descs(blob))
                agent.send_notif(client, op + b"-DONE")
                served += 1
        time.sleep(0.0005)
    blocks.close()


def handle_request(agent, blocks, client, op, client_descs):
    """The two-stage pipeline.  store: network READ then file WRITE; load: file READ then network WRITE."""
    n = blocks.batch
    if client_descs.descCount() != n:
        raise ValueError(f"{client} sent {client_descs.descCount()} blocks, this server works in batches of {n}")

    def theirs(i):
        return agent.get_xfer_descs([client_descs[i]], "DRAM")

    first = ("READ", lambda i: (blocks.mem_descs(i), theirs(i), client)) if op == "STORE" else \
            ("READ", lambda i: (blocks.mem_descs(i), blocks.file_descs(i), agent.name))
    second = ("WRITE", lambda i: (blocks.mem_descs(i), blocks.file_descs(i), agent.name)) if op == "STORE" else \
             ("WRITE", lambda i: (blocks.mem_descs(i), theirs(i), client))
    stage1 = {}
    stage2 = {}
    for i in range(n):
        local, remote, peer = first[1](i)
        stage1[i] = agent.initialize_xfer(first[0], local, remote, peer)
        agent.transfer(stage1[i])
    done = 0
    deadline = time.time() + 120
    while done < n:
        for i in list(stage1):
            if _state(agent, stage1[i], f"{op} block {i}, first stage") != "PROC":
                agent.release_xfer_handle(stage1.pop(i))
                local, remote, peer = second[1](i)
                stage2[i] = agent.initialize_xfer(second[0], local, remote, peer)
                agent.transfer(stage2[i])
        for i in list(stage2):
            if _state(agent, stage2[i], f"{op} block {i}, second stage") != "PROC":
                agent.release_xfer_handle(stage2.pop(i))
                done += 1
        if time.time() > deadline:
            raise TimeoutError(op)


# ---------------------------------------------------------------------------------------------- client
def run_client(args):
    agent, storage = make_agent(args.agent_name, args.port)
    blocks = Blocks(agent, args.fileprefix + "_" + args.agent_name, args.buf_size, args.batch_size, fill=17)
    expect = [b.clone() for b in blocks.buffers]

    # local: buffers -> own files -> buffers
    t0 = time.time()
    storage_pass(agent, blocks, "WRITE")
    for b in blocks.buffers:
        b.zero_()
    storage_pass(agent, blocks, "READ")
    assert all(torch.equal(a, b) for a, b in zip(blocks.buffers, expect)), "local storage round trip"
    total = 2 * args.buf_size * args.batch_size
    print(f"{args.agent_name}: local {storage} round trip of {total} bytes in {time.time() - t0:.3f} s", flush=True)

    servers = []
    with open(args.agents_file) as f:
        for line in f:
            if line.strip() and not line.startswith("#"):
                name, ip, port = line.split()
                servers.append((name, ip, int(port)))
    all_descs = agent.get_xfer_descs([(b.data_ptr(), args.buf_size, 0) for b in blocks.buffers], "DRAM")
    blob = agent.get_serialized_descs(all_descs)
    for name, ip, port in servers:
        agent.fetch_remote_metadata(name, ip, port)
        agent.send_local_metadata(ip, port)
        deadline = time.time() + 30
        while not agent.check_remote_metadata(name):
            if time.time() > deadline:
                raise TimeoutError("metadata of " + name)
            time.sleep(0.01)
        for op in (b"STORE", b"LOAD"):
            if op == b"LOAD":
                for b in blocks.buffers:
                    b.zero_()
            t0 = time.time()
            agent.send_notif(name, op + b"|" + blob)
            deadline = time.time() + 120
            while not agent.check_remote_xfer_done(name, op + b"-DONE"):
                if time.time() > deadline:
                    raise TimeoutError(op.decode() + " at " + name)
                time.sleep(0.0005)
            print(f"{args.agent_name}: {op.decode()} of {args.buf_size * args.batch_size} bytes at {name} in {time.time() - t0:.3f} s", flush=True)
        assert all(torch.equal(a, b) for a, b in zip(blocks.buffers, expect)), "blocks loaded from " + name
    blocks.close()
    print(f"{args.agent_name}: all blocks verified", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", required=True, choices=["client", "server"])
    ap.add_argument("--agent_name", required=True)
    ap.add_argument("--fileprefix", required=True)
    ap.add_argument("--agents_file", help="client: the servers, one '<name> <ip> <port>' per line")
    ap.add_argument("--port", type=int, default=0, help="port of this agent's metadata listener (server: the one in the agents file)")
    ap.add_argument("--buf_size", type=int, default=1 << 20)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--requests", type=int, default=0, help="server: leave after this many requests (0: serve until killed)")
    args = ap.parse_args()
    if args.role == "server":
        if not args.port:
            ap.error("a server needs --port")
        serve(args)
    else:
        if not args.agents_file:
            ap.error("a client needs --agents_file")
        if not args.port:
            import socket

            s = socket.socket()
            s.bind(("127.0.0.1", 0))
            args.port = s.getsockname()[1]
            s.close()
        run_client(args)


if __name__ == "__main__":
    main()

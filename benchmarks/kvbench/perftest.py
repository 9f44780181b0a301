"""Custom-traffic performance tests over the agent API (ct-perftest and sequential-ct-perftest).

One process per rank (``torchrun``); metadata and descriptors travel over torch.distributed
(gloo for host memory, nccl for GPUs), transfers go through ``nixl_agent``.  Follows the
reference's benchmark/kvbench/test/custom_traffic_perftest.py and
sequential_custom_traffic_perftest.py: a pattern is prepared once (buffers, registration, one
transfer handle per destination), then timed between barriers; the sequential test runs a list
of patterns back to back and also reports each pattern's isolated time."""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from nixl_b200 import nixl_agent, nixl_agent_config

from .traffic import TrafficPattern


class Runtime:
    """The few collectives the tests need, over an initialised torch.distributed group."""

    def __init__(self, device: Optional[torch.device]):
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.device = device

    def barrier(self) -> None:
        if self.device is not None and self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier()

    def allgather(self, obj):
        out = [None] * self.world
        dist.all_gather_object(out, obj)
        return out

    def max(self, value: float) -> float:
        dev = self.device if (self.device is not None and dist.get_backend() == "nccl") else torch.device("cpu")
        t = torch.tensor([value], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())


class PreparedPattern:
    """Buffers and transfer handles of one pattern on one rank."""

    def __init__(self, agent, rt: Runtime, tp: TrafficPattern):
        """Allocates and registers this rank's buffers; ``connect`` builds the handles once every
        rank's metadata (which must include these registrations) has been exchanged."""
        self.tp, self.agent, self.rt = tp, agent, rt
        rank = rt.rank
        dev = rt.device if tp.on_gpu else torch.device("cpu")
        self.send = {j: torch.full((n,), rank % 127, dtype=torch.int8, device=dev) for j, n in enumerate(tp.matrix[rank]) if n > 0}
        self.recv = {i: torch.zeros(tp.matrix[i][rank], dtype=torch.int8, device=dev) for i in range(tp.world_size) if tp.matrix[i][rank] > 0}
        self.regs = []
        bufs = list(self.send.values()) + list(self.recv.values())
        if bufs:
            self.regs.append(agent.register_memory(bufs))
        self.handles, self.expect, self.peer_names = [], [], []

    def connect(self, peer_names: Sequence[str]) -> None:
        tp, rt, agent, rank = self.tp, self.rt, self.agent, self.rt.rank
        # Everybody learns where everybody else's landing (WRITE) or source (READ) buffers are.
        exposed = self.recv if tp.xfer_op == "WRITE" else self.send
        table = rt.allgather({peer: (t.data_ptr(), t.numel(), t.get_device() if t.is_cuda else 0) for peer, t in exposed.items()})
        mem = "VRAM" if tp.on_gpu else "DRAM"
        local_side = self.send if tp.xfer_op == "WRITE" else self.recv
        for peer, buf in local_side.items():
            addr, size, devid = table[peer][rank]
            local_descs = agent.get_xfer_descs(self._shards(buf.data_ptr(), buf.numel(), buf.get_device() if buf.is_cuda else 0), mem)
            remote_descs = agent.get_xfer_descs(self._shards(addr, size, devid), mem)
            note = f"tp{tp.id}:{rank}".encode()
            self.handles.append((peer, agent.initialize_xfer(tp.xfer_op, local_descs, remote_descs, peer_names[peer], note)))
        # Whom this rank expects a completion note from: its senders (WRITE) or its readers (READ).
        self.expect = sorted(self.recv) if tp.xfer_op == "WRITE" else sorted(self.send)
        self.peer_names = peer_names

    def _shards(self, addr: int, size: int, dev: int):
        n = max(1, min(self.tp.shards, size))
        step = -(-size // n)
        return [(addr + o, min(step, size - o), dev) for o in range(0, size, step)]

    def run_once(self) -> float:
        """Posts everything, waits for local completion and for the peers' notes; returns seconds."""
        t0 = time.perf_counter()
        pending = []
        for peer, h in self.handles:
            st = self.agent.transfer(h)
            if st == "ERR":
                raise RuntimeError(f"transfer to rank {peer} failed")
            if st != "DONE":
                pending.append((peer, h))
        while pending:
            nxt = []
            for peer, h in pending:
                st = self.agent.check_xfer_state(h)
                if st == "ERR":
                    raise RuntimeError(f"transfer to rank {peer} failed")
                if st != "DONE":
                    nxt.append((peer, h))
            pending = nxt
        waiting = {p: f"tp{self.tp.id}:{p}".encode() for p in self.expect}
        deadline = time.perf_counter() + 60
        while waiting:
            for p in list(waiting):
                if self.agent.check_remote_xfer_done(self.peer_names[p], waiting[p]):
                    del waiting[p]
            if time.perf_counter() > deadline:
                raise TimeoutError(f"no completion note from ranks {sorted(waiting)}")
        return time.perf_counter() - t0

    def verify(self) -> bool:
        ok = True
        for peer, buf in (self.recv if self.tp.xfer_op == "WRITE" else {}).items():
            ok = ok and bool((buf == peer % 127).all().item())
        return ok

    def release(self) -> None:
        for _, h in self.handles:
            self.agent.release_xfer_handle(h)
        for r in self.regs:
            self.agent.deregister_memory(r)
        self.handles, self.regs = [], []


def _setup(backend: str, use_gpu: bool):
    if not dist.is_initialized():
        dist.init_process_group("nccl" if use_gpu else "gloo")
    rank = dist.get_rank()
    device = None
    if use_gpu:
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank % max(1, torch.cuda.device_count()))))
        torch.cuda.set_device(device)
    rt = Runtime(device)
    agent = nixl_agent(f"ct{rank}", nixl_agent_config(enable_prog_thread=False, backends=[backend]))
    return rt, agent


def _exchange_metadata(rt: Runtime, agent) -> List[str]:
    """After all registrations: every rank loads every other rank's metadata; returns agent names by rank."""
    mds = rt.allgather((agent.name, agent.get_agent_metadata()))
    for name, md in mds:
        if name != agent.name:
            agent.add_remote_agent(md)
    return [m[0] for m in mds]


def _time_pattern(rt: Runtime, prep: PreparedPattern, iters: int, warmup: int) -> Dict[str, float]:
    times = []
    for i in range(warmup + iters):
        rt.barrier()
        t = prep.run_once()
        if prep.tp.on_gpu:
            torch.cuda.synchronize(rt.device)
        if i >= warmup:
            times.append(rt.max(t))
    times.sort()
    return {"avg_ms": 1e3 * sum(times) / len(times), "min_ms": 1e3 * times[0], "p50_ms": 1e3 * times[len(times) // 2], "max_ms": 1e3 * times[-1]}


def ct_perftest(tp: TrafficPattern, iters: int = 50, warmup: int = 10, backend: str = "NVLINK", json_output_path: Optional[str] = None) -> dict:
    """Times one traffic pattern; rank 0 returns (and prints) the report."""
    rt, agent = _setup(backend, tp.on_gpu)
    if tp.world_size != rt.world:
        raise ValueError(f"matrix is {tp.world_size} x {tp.world_size} but the job has {rt.world} ranks")
    prep = PreparedPattern(agent, rt, tp)
    prep.connect(_exchange_metadata(rt, agent))
    stats = _time_pattern(rt, prep, iters, warmup)
    ok = all(rt.allgather(prep.verify()))
    prep.release()
    gb = tp.total_bytes() / 1e9
    report = {"bench": "ct-perftest", "ranks": rt.world, "total_GB": round(gb, 6), "num_senders": len(tp.senders()), "xfer_op": tp.xfer_op,
              "mem_type": tp.mem_type, "shards": tp.shards, "verified": ok, "GBps": round(gb / (stats["avg_ms"] / 1e3), 3) if stats["avg_ms"] else 0.0,
              **{k: round(v, 4) for k, v in stats.items()}}
    if rt.rank == 0:
        print(json.dumps(report), flush=True)
        if json_output_path:
            with open(json_output_path, "w") as f:
                json.dump(report, f, indent=1)
    return report


def sequential_ct_perftest(patterns: List[TrafficPattern], backend: str = "NVLINK", json_output_path: Optional[str] = None,
                           isolation_iters: int = 5, honor_sleep: bool = True) -> List[dict]:
    """Runs the patterns one after the other (optionally sleeping before each, as a stand-in for
    compute), then times each pattern alone; reports both latencies per pattern."""
    if not patterns:
        return []
    rt, agent = _setup(backend, patterns[0].on_gpu)
    preps = [PreparedPattern(agent, rt, tp) for tp in patterns]
    names = _exchange_metadata(rt, agent)
    for prep in preps:
        prep.connect(names)
    rows = []
    rt.barrier()
    for tp, prep in zip(patterns, preps):
        if honor_sleep and tp.sleep_before_launch_sec:
            time.sleep(tp.sleep_before_launch_sec)
        rt.barrier()
        t = rt.max(prep.run_once())
        if honor_sleep and tp.sleep_after_launch_sec:
            time.sleep(tp.sleep_after_launch_sec)
        rows.append({"id": tp.id, "size_GB": round(tp.total_bytes() / 1e9, 6), "latency_ms": round(1e3 * t, 4), "num_senders": len(tp.senders()),
                     "metadata": tp.metadata})
    for row, prep in zip(rows, preps):
        row["isolated_latency_ms"] = round(_time_pattern(rt, prep, isolation_iters, 1)["avg_ms"], 4)
    for prep in preps:
        prep.release()
    if rt.rank == 0:
        print(f"{'Transfer size (GB)':>20}{'Latency (ms)':>16}{'Isolated Latency (ms)':>25}{'Num Senders':>15}")
        for r in rows:
            print(f"{r['size_GB']:>20.3f}{r['latency_ms']:>16.3f}{r['isolated_latency_ms']:>25.3f}{r['num_senders']:>15d}")
        if json_output_path:
            with open(json_output_path, "w") as f:
                json.dump(rows, f, indent=1)
    return rows

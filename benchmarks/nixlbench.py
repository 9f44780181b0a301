#!/usr/bin/env python
"""nixlbench-style VRAM<->VRAM sweep through the agent API.

WRITE and READ, block sizes 4 KiB - 1 GiB (powers of two, x4 steps by default), batch 1 / 16 / 256
descriptors of uniform random bytes from a seed; patterns: pairwise (rank 0 <-> rank 1), ring
(rank -> rank+1) and all-to-all (every rank posts one request per peer).  For every point:
aggregate GB/s (device-timed with CUDA events over back-to-back requests, max over ranks) and
host-timed p50 / p99 latency of a single request.  Baselines on the same buffers: NCCL send/recv
(ring) and, in one process, ``cudaMemcpyPeerAsync`` per descriptor (torch ``copy_``).
Structure follows the reference's benchmark/nixlbench (sweep loops ``src/main.cpp:107,:220``,
statistics ``src/utils/utils.cpp:1336``); ``--check-consistency`` verifies the bytes.

Launch: ``python benchmarks/nixlbench.py`` (1 GPU, loopback) or under torch.distributed.run.
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from nixl_b200 import _bindings as nb  # noqa: E402
from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-block", "--start_block_size", dest="min_block", type=int, default=4096)
    ap.add_argument("--max-block", "--max_block_size", dest="max_block", type=int, default=1 << 30)
    ap.add_argument("--step", type=int, default=4, help="multiply the block size by this between points")
    ap.add_argument("--batches", default="1,16,256")
    ap.add_argument("--ops", "--op_type", dest="ops", default="WRITE,READ")
    ap.add_argument("--patterns", default="ring,alltoall,pairwise")
    ap.add_argument("--buffer", "--total_buffer_size", dest="buffer", type=int, default=4 << 30, help="bytes of source and of destination buffer per GPU")
    ap.add_argument("--iters", "--num_iter", dest="iters", type=int, default=0, help="0: chosen per point (more for small messages)")
    ap.add_argument("--copy-path", default="vector")
    ap.add_argument("--check-consistency", "--check_consistency", dest="check_consistency", action="store_true")
    ap.add_argument("--baselines", type=int, default=1)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    agent = nixl_agent(f"nb{rank}", nixl_agent_config(enable_prog_thread=False, backends=[]))
    agent.create_backend("NVLINK", {"copy_path": args.copy_path})
    src = torch.empty(args.buffer, dtype=torch.uint8, device=dev)
    dst = torch.zeros(args.buffer, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(42 + rank)
    src.view(torch.int64).random_(generator=g)
    agent.register_memory(src)
    agent.register_memory(dst)
    info = {"md": agent.get_agent_metadata(), "dst": (dst.data_ptr(), local), "src": (src.data_ptr(), local), "name": agent.name}
    infos = [None] * world
    if world > 1:
        dist.all_gather_object(infos, info)
    else:
        infos = [info]
    for r, i in enumerate(infos):
        if r != rank:
            agent.add_remote_agent(i["md"])

    stream = torch.cuda.Stream(device=dev)
    sparam = f"stream={stream.cuda_stream}"
    results = []

    def peers_for(pattern):
        if pattern == "ring":
            return [(rank + 1) % world]
        if pattern == "pairwise":
            if world == 1:
                return [0]
            return [1 - rank] if rank < 2 else []
        # staggered: rank r starts with r+1, so no receiver is hit by everybody at once
        return [(rank + 1 + i) % world for i in range(world - 1)] or [rank]

    def wait(h):
        while agent.agent.getXferStatus(h) != nb.NIXL_SUCCESS:
            pass

    for pattern in args.patterns.split(","):
        if pattern == "pairwise" and world > 2:
            pass  # ranks >= 2 idle but take part in the barriers
        peers = peers_for(pattern)
        for op in args.ops.split(","):
            for batch in [int(b) for b in args.batches.split(",")]:
                block = args.min_block
                while block <= args.max_block:
                    per_peer = block * batch
                    if per_peer * max(1, len(peers)) > args.buffer:
                        break
                    handles = []
                    for j, r in enumerate(peers):
                        base_l = src.data_ptr() + j * per_peer if op == "WRITE" else dst.data_ptr() + j * per_peer
                        # every source rank gets its own window of the target buffer
                        slot = (rank if pattern == "alltoall" else 0) * per_peer
                        if (slot + per_peer) > args.buffer:
                            slot = 0
                        base_r = (infos[r]["dst"][0] if op == "WRITE" else infos[r]["src"][0]) + slot
                        la = [(base_l + i * block, block, local) for i in range(batch)]
                        ra = [(base_r + i * block, block, infos[r]["dst"][1]) for i in range(batch)]
                        handles.append(agent.initialize_xfer(op, agent.get_xfer_descs(la, "VRAM"), agent.get_xfer_descs(ra, "VRAM"), infos[r]["name"]))
                    iters = args.iters or max(5, min(200, (1 << 31) // max(per_peer * max(1, len(peers)), 1)))
                    # latency: one request at a time, host clock
                    lat = []
                    if handles:
                        for i in range(min(iters, 100) + 5):
                            t0 = time.perf_counter()
                            st = agent.agent.postXferReq(handles[0])
                            if st != nb.NIXL_SUCCESS:
                                wait(handles[0])
                            if i >= 5:
                                lat.append((time.perf_counter() - t0) * 1e6)
                        lat.sort()
                    barrier()
                    # bandwidth: all peers' requests back to back, device clock
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    for _ in range(iters):
                        for h in handles:
                            agent.agent.postXferReq(h, None, sparam)
                        for h in handles:
                            wait(h)
                    e1.record(stream)
                    barrier()
                    ms = e0.elapsed_time(e1) if handles else 0.0
                    stat = torch.tensor([ms, float(len(handles) * per_peer * iters)], dtype=torch.float64, device=dev)
                    if world > 1:
                        mx = stat.clone()
                        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
                        sm = stat.clone()
                        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
                        ms, total = float(mx[0]), float(sm[1])
                    else:
                        total = float(stat[1])
                    ok = None
                    if args.check_consistency and handles and op == "WRITE" and world == 1:
                        ok = bool(torch.equal(dst[:per_peer], src[:per_peer]))
                    for h in handles:
                        agent.release_xfer_handle(h)
                    rec = {"bench": "nixlbench", "pattern": pattern, "op": op, "n_gpus": world, "block": block, "batch": batch,
                           "iters": iters, "GBps_total": round(total / (ms * 1e-3) / 1e9, 2) if ms else None,
                           "GBps_per_sender": round(total / (ms * 1e-3) / 1e9 / max(1, (world if pattern != "pairwise" else min(world, 2))), 2) if ms else None,
                           "p50_us": round(lat[len(lat) // 2], 2) if lat else None, "p99_us": round(lat[min(len(lat) - 1, int(len(lat) * 0.99))], 2) if lat else None}
                    if ok is not None:
                        rec["consistent"] = ok
                    results.append(rec)
                    if rank == 0:
                        print(json.dumps(rec), flush=True)
                    block *= args.step

    if args.baselines:
        # NCCL ring send/recv and (single process) cudaMemcpyPeerAsync-style copies on the same sizes
        block = args.min_block
        while block <= min(args.max_block, args.buffer):
            iters = max(5, min(200, (1 << 31) // block))
            view_s, view_d = src[:block], dst[:block]
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                if world > 1:
                    ops = [dist.P2POp(dist.isend, view_s, (rank + 1) % world), dist.P2POp(dist.irecv, view_d, (rank - 1) % world)]
                    for w in dist.batch_isend_irecv(ops):
                        w.wait()
                else:
                    view_d.copy_(view_s, non_blocking=True)
            e1.record()
            barrier()
            t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            rec = {"bench": "nixlbench-baseline", "what": "nccl_send_recv_ring" if world > 1 else "cudaMemcpyAsync_d2d", "n_gpus": world,
                   "block": block, "GBps_total": round(world * block * iters / (float(t) * 1e-3) / 1e9, 2)}
            if rank == 0:
                print(json.dumps(rec), flush=True)
            block *= args.step
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""GPU-initiated put-with-signal benchmark.

A persistent kernel on every GPU puts 256 KiB tiles to every peer from inside its compute
loop (1024 iterations per peer, ``--ctas-per-peer`` producer CTAs taking turns) with
``nixlPut<BLOCK>`` + ``nixlAtomicAdd`` (device API); the consumer side waits on the remote
per-slot counters and acknowledges.  Reported: microseconds per iteration, microseconds per put,
aggregate GB/s, and the same traffic posted from the host with ``postXferReq`` as baseline.
With one GPU the rank talks to itself.  Device-timed (CUDA events), max over ranks.

Launch: ``python benchmarks/device_put_bench.py`` or under torch.distributed.run.
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
from nixl_b200.ops import device_api  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=1024)
    ap.add_argument("--tile", type=int, default=256 << 10)
    ap.add_argument("--window", type=int, default=40)
    ap.add_argument("--compute-passes", type=int, default=1)
    ap.add_argument("--host-iters", type=int, default=128)
    ap.add_argument("--ctas-per-peer", type=int, default=20)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peers = [r for r in range(world) if r != rank] or [rank]
    P = len(peers)

    agent = nixl_agent(f"dput{rank}", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
    tiles = torch.randn(P * args.ctas_per_peer * args.tile // 4, dtype=torch.float32, device=dev)  # one source tile per producer CTA
    landing = torch.zeros(world * args.window * args.tile, dtype=torch.uint8, device=dev)
    signals = torch.zeros(2 * world * args.window, dtype=torch.int64, device=dev)  # arrival[rank][slot], then acknowledgement[rank][slot]
    for t in (tiles, landing, signals):
        agent.register_memory(t)
    info = {"md": agent.get_agent_metadata(), "landing": (landing.data_ptr(), landing.numel(), local),
            "signals": (signals.data_ptr(), signals.numel() * 8, local), "name": agent.name}
    infos = [None] * world
    if world > 1:
        dist.all_gather_object(infos, info)
    else:
        infos = [info]
    for r, i in enumerate(infos):
        if r != rank:
            agent.add_remote_agent(i["md"])
    local_tiles = agent.prep_mem_view(agent.get_xfer_descs(tiles))
    local_signals = agent.prep_mem_view(agent.get_xfer_descs(signals))
    remote_tiles = agent.prep_mem_view(agent.get_remote_descs([i["landing"] + (i["name"],) for i in infos], "VRAM"))
    remote_signals = agent.prep_mem_view(agent.get_remote_descs([i["signals"] + (i["name"],) for i in infos], "VRAM"))
    peer_ids = torch.tensor(peers, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def run(iters, passes):
        signals.zero_()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        p = device_api.DevPutParams()
        p.local_tiles, p.remote_tiles, p.local_signals, p.remote_signals = local_tiles, remote_tiles, local_signals, remote_signals
        p.peer_ids = peer_ids.data_ptr()
        p.peers, p.rank, p.iters, p.window, p.compute_passes = P, rank, iters, args.window, passes
        p.ctas_per_peer = args.ctas_per_peer
        p.tile_bytes, p.ack_offset, p.timeout_ns = args.tile, world * args.window * 8, 20_000_000_000
        p.status = status.data_ptr()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        device_api.put_signal_launch(p, dev)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t) * 1e3  # us

    run(64, args.compute_passes)  # warm-up
    t_full = run(args.iters, args.compute_passes)
    t_compute_only_proxy = run(args.iters, 0)  # communication only: the cost of the puts without the compute pass
    arrived = signals[: world * args.window].view(world, args.window).sum(dim=1)
    ok = int(status.item()) == 0 and all(int(arrived[r]) == args.iters for r in peers)
    # The tiles did not change during the communication-only run: every landing slot must hold the source tile of
    # the producer CTA that wrote it last.
    if world > 1:
        all_tiles = [torch.empty_like(tiles) for _ in range(world)]
        dist.all_gather(all_tiles, tiles)
        for r in peers:
            pi = [x for x in range(world) if x != r].index(rank)
            for slot in range(min(args.window, args.iters)):
                last_it = slot + 1 + ((args.iters - 1 - slot) // args.window) * args.window
                cta = pi * args.ctas_per_peer + (last_it - 1) % args.ctas_per_peer
                want = all_tiles[r].view(torch.uint8)[cta * args.tile:(cta + 1) * args.tile]
                got = landing[(r * args.window + slot) * args.tile:(r * args.window + slot + 1) * args.tile]
                ok = ok and bool(torch.equal(want, got))
        del all_tiles

    # Host-posted baseline: the same tile to every peer, posted and completed from the host.
    handles = []
    for j, r in enumerate(peers):
        la = [(tiles.data_ptr() + j * args.ctas_per_peer * args.tile, args.tile, local)]
        ra = [(infos[r]["landing"][0] + rank * args.window * args.tile, args.tile, infos[r]["landing"][2])]
        handles.append(agent.initialize_xfer("WRITE", agent.get_xfer_descs(la, "VRAM"), agent.get_xfer_descs(ra, "VRAM"), infos[r]["name"]))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.host_iters):
        for h in handles:
            agent.agent.postXferReq(h)
        for h in handles:
            while agent.agent.getXferStatus(h) != nb.NIXL_SUCCESS:
                pass
    host_us = (time.perf_counter() - t0) * 1e6 / args.host_iters
    hv = torch.tensor([host_us], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(hv, op=dist.ReduceOp.MAX)
    host_us = float(hv)

    if rank == 0:
        bytes_per_iter = P * args.tile
        print(json.dumps({
            "bench": "device_put_signal", "n_gpus": world, "peers_per_gpu": P, "tile_bytes": args.tile, "iters": args.iters, "window": args.window, "ctas_per_peer": args.ctas_per_peer,
            "us_per_iter": round(t_full / args.iters, 2), "us_per_put": round(t_full / args.iters / P, 2),
            "us_per_iter_comm_only": round(t_compute_only_proxy / args.iters, 2),
            "GBps_per_gpu": round(bytes_per_iter * args.iters / t_full / 1e3, 1),
            "GBps_per_gpu_comm_only": round(bytes_per_iter * args.iters / t_compute_only_proxy / 1e3, 1),
            "host_posted_us_per_iter": round(host_us, 2), "host_posted_GBps_per_gpu": round(bytes_per_iter / host_us / 1e3, 1),
            "speedup_vs_host_posted": round(host_us / (t_full / args.iters), 2), "verified": ok,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Headline benchmark: nixlbench-style VRAM->VRAM WRITE through the agent API, plus the rest of
the metric family (size sweep, KV-cache transfer, MoE dispatch/combine) and in-run baselines.

Headline step: every rank posts one transfer request (BATCH descriptors of BLOCK bytes) to its
ring neighbour (rank+1) % N through ``nixl_agent`` and polls it to completion; two identical
requests take turns (a request is posted again only once it has completed), so the next step is
queued on the stream while the current one runs.  With N = 1 the target is a second buffer on the
same GPU.  The reported value is the whole-job aggregate:
N x bytes per step x steps / (max over ranks of the device time).

Timing: CUDA events recorded on the stream the copies are launched on (stream-ordered posting),
bracketed by barrier + synchronize; buffers (1 GiB per step) are larger than L2, so no flush is
needed between iterations.  ``e2e`` repeats the measurement through the same public API with,
every step, a host->device copy of the step's payload from pinned host memory into the
registered source buffer and a device->host read of a digest of the buffer this rank received.

``extras`` (outside the timed regions, every figure device-timed and the max over ranks):
  baselines  the same ring step through (a) the copy engines, one cudaMemcpyAsync per descriptor
             (what a descriptor-at-a-time transport such as UCX cuda_ipc does), (b) the copy
             kernel only, (c) the same request with its destination blocks in reverse order (nothing
             to merge), (d) the headline once more, (e) NCCL send/recv; ``vs_baseline`` divides the
             headline by (a)
  sweep      WRITE and READ, 4 KiB - 1 GiB, 1/16/256 descriptors per request, ring and
             all-to-all (pairwise at N = 2): GB/s per GPU and host-timed p50/p99 latency
  kv         paged KV-cache transfer, Llama-3-8B shape, prefill ranks -> decode ranks with TP
             reshard, bf16 and bf16->fp8, ms/request, checked against the PyTorch statement
  ep         MoE dispatch + combine, DeepSeek-V3 shape, 128 and 4096 tokens per GPU, checked on
             every rank against an fp32 PyTorch statement of the routing
  dput       GPU-initiated put with signal: a persistent kernel puts 256 KiB tiles to every peer from
             inside its loop (device API), the consumer waits on the remote per-slot counters and
             acknowledges; µs per put, landed tiles compared with their sources

Launch: ``python bench.py`` (1 GPU) or
``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
``--impl reference`` runs the same ring step through the reference library when one is installed
under ``baseline/_ref`` and otherwise reports why it is not.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
GIB = 1 << 30


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--block", type=int, default=64 << 20, help="descriptor size in bytes")
    p.add_argument("--batch", type=int, default=16, help="descriptors per request")
    p.add_argument("--extras", default="baselines,sweep,kv,ep,dput", help="comma list of extras to run ('' or 'none': headline only)")
    p.add_argument("--extras-budget", type=float, default=120.0, help="seconds the extras may take in all; sections that do not fit are skipped")
    return p.parse_args()


# ====================================================================== clocks


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while running."""

    FIELDS = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL,
                text=True,
            )
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, max_clocks, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                clocks.append(float(r[1]))
                max_clocks.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max(max_clocks) if max_clocks else None,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


# ====================================================================== reference arm

REFERENCE_INSTALL = (
    "python -m pip install --no-index --no-build-isolation --find-links <wheelhouse> --target baseline/_ref <reference source tree>"
)


def reference_arm(args):
    """Runs the ring step through the reference's own Python API (``nixl._api.nixl_agent`` with its UCX
    backend) when the reference is installed under baseline/_ref; otherwise prints why it is not.
    The probe imports in a child process whose module path does not contain this repository, so the
    ``nixl`` compatibility package of this repository can never answer for the reference."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(ref_dir) or not os.listdir(ref_dir):
        why = (f"baseline/_ref is absent: `{REFERENCE_INSTALL}` fails with \"ModuleNotFoundError: No module named 'mesonpy'\" "
               "(the build backend meson-python is neither in the image nor in the wheelhouse; UCX, abseil, asio, etcd-cpp-api, which the "
               "build links, are absent too)")
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    probe = (
        "import os, sys\n"
        f"root = {ROOT!r}\n"
        "sys.path = [p for p in sys.path if os.path.abspath(p or os.getcwd()) != root]\n"
        f"sys.path.insert(0, {ref_dir!r})\n"
        "import nixl._api as api\n"
        "assert os.path.abspath(api.__file__).startswith(os.path.abspath(sys.path[0])), api.__file__\n"
        "print(api.__file__)\n"
    )
    r = subprocess.run([sys.executable, "-c", probe], capture_output=True, text=True, cwd="/")
    if r.returncode != 0:
        tail = (r.stderr.strip().splitlines() or ["no output"])[-1]
        print(json.dumps({"impl": "reference", "unavailable": f"baseline/_ref exists but the reference does not import: {tail}"}))
        return 0
    return reference_ring(args, ref_dir)


def reference_ring(args, ref_dir):
    """The headline ring step with the reference's agent (stock UCX path).  Wall-clock timed between
    barrier + synchronize pairs, since the reference posts on streams of its own."""
    sys.path = [p for p in sys.path if os.path.abspath(p or os.getcwd()) != ROOT]
    sys.path.insert(0, ref_dir)
    import torch
    import torch.distributed as dist
    from nixl._api import nixl_agent, nixl_agent_config

    rank, world, local_rank = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    step_bytes = args.block * args.batch
    agent = nixl_agent(f"ref{rank}", nixl_agent_config(backends=["UCX"]))
    src = torch.randint(0, 256, (step_bytes,), dtype=torch.uint8, device=dev)
    dst = torch.zeros(step_bytes, dtype=torch.uint8, device=dev)
    agent.register_memory(src)
    agent.register_memory(dst)
    info = (agent.get_agent_metadata(), dst.data_ptr(), local_rank)
    infos = [info]
    if world > 1:
        infos = [None] * world
        dist.all_gather_object(infos, info)
    peer = (rank + 1) % world
    peer_name = f"ref{peer}"
    if peer != rank:
        agent.add_remote_agent(infos[peer][0])
    local = [(src.data_ptr() + i * args.block, args.block, local_rank) for i in range(args.batch)]
    remote = [(infos[peer][1] + i * args.block, args.block, infos[peer][2]) for i in range(args.batch)]
    h = agent.initialize_xfer("WRITE", agent.get_xfer_descs(local, "VRAM"), agent.get_xfer_descs(remote, "VRAM"), peer_name)

    def step():
        st = agent.transfer(h)
        while st == "PROC":
            st = agent.check_xfer_state(h)
        if st != "DONE":
            raise RuntimeError(f"reference transfer ended in state {st}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    barrier()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": round(world * step_bytes * args.steps / float(t) / 1e9, 2), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(float(t) * 1e3 / args.steps, 4),
            "higher_is_better": True, "scaling": "weak", "dtype": "uint8 payload", "data": "synthetic: uniform random bytes",
            "config": {"model": CONFIG_MODEL, "block_bytes": args.block, "batch_descs": args.batch, "timing": "wall clock between barriers, max over ranks"},
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


METRIC = ("P2P VRAM->VRAM WRITE GB/s through the agent API (nixlbench ring, aggregate over all GPUs); extras: GB/s + p50 us vs size, "
          "KV xfer ms/request, EP dispatch+combine us")
CONFIG_MODEL = "nixlbench-style VRAM sweep point (VRAM to VRAM WRITE, 16 x 64 MiB per request)"


# ====================================================================== helpers


class Env:
    """Everything a section needs: ranks, device, torch / dist modules, agents, the two 1 GiB buffers."""


def wait_done(env, agent, handle, limit_s=30.0, where=""):
    nb = env.nb
    t_end = None
    spins = 0
    while True:
        st = agent.agent.getXferStatus(handle)  # raises on a negative status
        if st == nb.NIXL_SUCCESS:
            return
        spins += 1
        if (spins & 0xFFF) == 0:
            now = time.perf_counter()
            if t_end is None:
                t_end = now + limit_s
            elif now > t_end:
                raise TimeoutError(f"transfer still in progress after {limit_s:.0f} s {where}")


def post(env, agent, handle, stream_param=""):
    """Posts and returns True when the request completed inside the call."""
    if stream_param:
        return agent.agent.postXferReq(handle, None, stream_param) == env.nb.NIXL_SUCCESS
    return agent.agent.postXferReq(handle) == env.nb.NIXL_SUCCESS


def barrier(env):
    if env.world > 1:
        env.dist.barrier()
    env.torch.cuda.synchronize()


def max_over_ranks(env, values):
    t = env.torch.tensor(list(values), dtype=env.torch.float64, device=env.dev)
    if env.world > 1:
        env.dist.all_reduce(t, op=env.dist.ReduceOp.MAX)
    return t.tolist()


def min_over_ranks(env, values):
    t = env.torch.tensor(list(values), dtype=env.torch.float64, device=env.dev)
    if env.world > 1:
        env.dist.all_reduce(t, op=env.dist.ReduceOp.MIN)
    return t.tolist()


def all_agree(env, flag):
    return min_over_ranks(env, [1.0 if flag else 0.0])[0] > 0.5


def fill_src(env, rank, out=None):
    """The bytes rank `rank` holds in its source buffer (any rank can regenerate them)."""
    torch = env.torch
    g = torch.Generator(device=env.dev)
    g.manual_seed(1234 + rank)
    if out is None:
        out = torch.empty(GIB, dtype=torch.uint8, device=env.dev)
    return out.random_(0, 256, generator=g)


def make_agent(env, tag, params):
    from nixl_b200 import nixl_agent, nixl_agent_config

    a = nixl_agent(f"{tag}{env.rank}", nixl_agent_config(enable_prog_thread=False, backends=[]))
    a.create_backend("NVLINK", params)
    a.register_memory(env.src)
    a.register_memory(env.dst)
    md = a.get_agent_metadata()
    mds = [md]
    if env.world > 1:
        mds = [None] * env.world
        env.dist.all_gather_object(mds, md)
    for r in range(env.world):
        if r != env.rank:
            a.add_remote_agent(mds[r])
    return a


def ring_handle(env, agent, tag, block, batch, scattered=False):
    """WRITE of `batch` blocks to the ring neighbour; `scattered` lands block i in slot batch-1-i."""
    peer = (env.rank + 1) % env.world
    pdev = env.devs[peer]
    local = [(env.src.data_ptr() + i * block, block, env.local_rank) for i in range(batch)]
    remote = [(env.dst_ptrs[peer] + (batch - 1 - i if scattered else i) * block, block, pdev) for i in range(batch)]
    return agent.initialize_xfer("WRITE", agent.get_xfer_descs(local, "VRAM"), agent.get_xfer_descs(remote, "VRAM"), f"{tag}{peer}")


def time_ring(env, agent, handles, steps, warm, warm_seconds=0.0):
    """Device time of `steps` posts on env.stream; returns (ms, wall_s).  `handles`: one request, or two identical
    ones posted alternately (a pipeline of depth two: the next launch is queued while the current one runs, so the
    stream never waits for the host; a request is posted again only once it has completed).  Warm-up: `warm` steps,
    and further steps until `warm_seconds` have passed."""
    torch = env.torch
    if not isinstance(handles, (list, tuple)):
        handles = [handles]
    pending = [False] * len(handles)

    def step(i):
        k = i % len(handles)
        if pending[k]:
            wait_done(env, agent, handles[k])
        pending[k] = not post(env, agent, handles[k], env.stream_param)

    def drain():
        for k, h in enumerate(handles):
            if pending[k]:
                wait_done(env, agent, h)
                pending[k] = False

    t_warm = time.perf_counter() + warm_seconds
    i = 0
    while i < warm or time.perf_counter() < t_warm:
        step(i)
        i += 1
    drain()
    barrier(env)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    ev0.record(env.stream)
    for i in range(steps):
        step(i)
    ev1.record(env.stream)
    drain()
    barrier(env)
    wall = time.perf_counter() - wall0
    return ev0.elapsed_time(ev1), wall


def roofline(env, aggregate_gbs):
    """What bounds the step and how close the run came.  One GPU copies inside its own HBM (bound: the
    measured copy bandwidth, read + write counted, halved for one-way bytes).  Two or more GPUs write to
    a neighbour over NVLink: the bound is the nominal 900 GB/s per direction per GPU; the measured
    ceilings of the link are given beside it (copy engine 779 / 774 GB/s one way / both ways busy,
    SM-issued stores 714 / 703: a store's 256 payload bytes carry 48 protocol bytes on the wire,
    a copy-engine write 32)."""
    hbm, source = 6650.0, "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            hbm = float(json.load(f)["hbm_gbs"])
            source = "measured"
    except Exception:
        pass
    per_gpu = aggregate_gbs / env.world
    if env.world == 1:
        bound = hbm / 2
        return {"bound": f"HBM copy, one-way bytes ({source} {hbm:.0f} GB/s read + write)", "bound_GBps_per_gpu": round(bound, 1),
                "GBps_per_gpu": round(per_gpu, 1), "fraction_of_bound": round(per_gpu / bound, 3)}
    return {"bound": "NVLink 5, 900 GB/s per direction per GPU (nominal)", "bound_GBps_per_gpu": 900.0, "GBps_per_gpu": round(per_gpu, 1),
            "fraction_of_bound": round(per_gpu / 900.0, 3), "fraction_of_measured_copy_engine_774": round(per_gpu / 774.0, 3),
            "wire_note": "payload ceiling at 100 % wire occupancy: 800 GB/s for copy-engine writes and loads (1/8 protocol bytes), 758 GB/s for SM stores (3/16)"}


# ====================================================================== main


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    t_start = time.perf_counter()

    import torch
    import torch.distributed as dist

    from nixl_b200 import _bindings as nb

    env = Env()
    env.torch, env.dist, env.nb = torch, dist, nb
    env.rank = int(os.environ.get("RANK", "0"))
    env.world = int(os.environ.get("WORLD_SIZE", "1"))
    env.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if env.world != args.gpus and env.world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(env.local_rank)
    env.dev = torch.device("cuda", env.local_rank)
    if env.world > 1:
        dist.init_process_group("nccl", device_id=env.dev)

    block, batch = args.block, args.batch
    step_bytes = block * batch
    buf_bytes = max(GIB, step_bytes)
    env.src = torch.empty(buf_bytes, dtype=torch.uint8, device=env.dev)
    env.dst = torch.zeros(buf_bytes, dtype=torch.uint8, device=env.dev)
    fill_src(env, env.rank, env.src[:GIB])
    ptrs = [(env.src.data_ptr(), env.dst.data_ptr(), env.local_rank)]
    if env.world > 1:
        ptrs = [None] * env.world
        dist.all_gather_object(ptrs, (env.src.data_ptr(), env.dst.data_ptr(), env.local_rank))
    env.src_ptrs, env.dst_ptrs, env.devs = [p[0] for p in ptrs], [p[1] for p in ptrs], [p[2] for p in ptrs]
    env.stream = torch.cuda.Stream(device=env.dev)
    env.stream_param = f"stream={env.stream.cuda_stream}"

    # The product configuration: neighbouring descriptors that continue each other are merged; the copy
    # kernel moves small and batched descriptors, the copy engines descriptors of 96 MiB and more between GPUs.
    env.agent = make_agent(env, "bench", {})
    plugin = ctypes.CDLL(os.path.join(ROOT, "nixl_b200", "lib", "plugins", "libplugin_NVLINK.so"))
    plugin.nixl_nvlink_kernel_launches.restype = ctypes.c_uint64
    handle = ring_handle(env, env.agent, "bench", block, batch)
    handle_b = ring_handle(env, env.agent, "bench", block, batch)  # the same request once more: posted alternately (depth two)

    # ---------------------------------------------------------------- device-timed region
    # Warm-up: W steps, then more of the same while the clock sampler starts up (a GPU left idle for that quarter of
    # a second drops its clocks and the timed steps would begin on the ramp).
    warm = max(args.warmup, 3)
    sampler = ClockSampler(env.local_rank)
    sampler.start()
    time_ring(env, env.agent, [handle, handle_b], 0, warm, warm_seconds=0.25)
    launches0 = plugin.nixl_nvlink_kernel_launches()
    dev_ms, wall = time_ring(env, env.agent, [handle, handle_b], args.steps, 0)
    launches = plugin.nixl_nvlink_kernel_launches() - launches0
    clocks = sampler.stop()

    # correctness: what landed in my dst is my predecessor's src
    expect = fill_src(env, (env.rank - 1) % env.world)
    ok = bool(torch.equal(env.dst[:step_bytes], expect[:step_bytes]))
    del expect

    # ---------------------------------------------------------------- end-to-end region
    host_in = torch.empty(step_bytes, dtype=torch.uint8).pin_memory()
    host_in.random_(0, 256)
    digest_dev = torch.empty(batch, dtype=torch.int64, device=env.dev)
    digest_host = torch.empty(batch, dtype=torch.int64).pin_memory()
    dst64 = env.dst.view(torch.int64)
    stride64 = block // 8
    src_step = env.src[:step_bytes]

    def e2e_step():
        with torch.cuda.stream(env.stream):
            src_step.copy_(host_in, non_blocking=True)  # H2D of this step's payload
        if not post(env, env.agent, handle, env.stream_param):  # ordered after the copy on the same stream
            wait_done(env, env.agent, handle)
        with torch.cuda.stream(env.stream):
            digest_dev.copy_(dst64[::stride64][:batch])  # first word of every received block
            digest_host.copy_(digest_dev, non_blocking=True)  # D2H of the step's result
        env.stream.synchronize()
        return int(digest_host[0])

    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(3):
        e2e_step()
    barrier(env)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier(env)
    e2e_s = time.perf_counter() - t0
    del host_in
    fill_src(env, env.rank, env.src[:GIB])  # the e2e payload overwrote the seeded source

    # ---------------------------------------------------------------- reduce over ranks
    dev_ms, e2e_s, wall = max_over_ranks(env, [dev_ms, e2e_s, wall])
    ok = all_agree(env, ok)
    gbs = env.world * step_bytes * args.steps / (dev_ms * 1e-3) / 1e9
    e2e_gbs = env.world * step_bytes * e2e_steps / e2e_s / 1e9
    env.agent.release_xfer_handle(handle)
    env.agent.release_xfer_handle(handle_b)

    # ---------------------------------------------------------------- extras (outside timed regions)
    extras = {}
    wanted = [x for x in args.extras.split(",") if x and x != "none"]
    sections = {"baselines": extras_baselines, "sweep": extras_sweep, "kv": extras_kv, "ep": extras_ep, "dput": extras_dput}
    deadline = time.perf_counter() + args.extras_budget
    for name in wanted:
        fn = sections.get(name)
        if fn is None:
            continue
        # every rank must take the same decision: rank 0's clock decides
        left = deadline - time.perf_counter()
        if env.world > 1:
            t = torch.tensor([left], dtype=torch.float64, device=env.dev)
            dist.broadcast(t, 0)
            left = float(t)
        if left < 5.0:
            extras[name] = {"skipped": "the extras' time budget was spent"}
            continue
        t_sec = time.perf_counter()
        try:
            extras[name] = fn(env, args, gbs, left)
        except Exception as exc:  # extras never invalidate the headline
            extras[name] = {"error": repr(exc)[:400]}
        if isinstance(extras[name], dict):
            extras[name]["section_s"] = round(time.perf_counter() - t_sec, 1)

    base = extras.get("baselines", {}) if isinstance(extras.get("baselines"), dict) else {}
    ce_gbs = base.get("copy_engine_per_descriptor_GBps")
    if env.rank == 0:
        out = {
            "metric": METRIC,
            "value": round(gbs, 2),
            "unit": "GB/s",
            "n_gpus": env.world,
            "steps": args.steps,
            "warmup": warm,
            "ms_per_step": round(dev_ms / args.steps, 4),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": round(gbs / ce_gbs, 3) if ce_gbs else None,
            "vs_baseline_what": "headline / the same ring step done as one copy-engine cudaMemcpyAsync per descriptor in the same run (the "
                                "reference publishes no numbers and cannot be built here)",
            "dtype": "uint8 payload (bandwidth test; no arithmetic)",
            "data": "synthetic: uniform random bytes from a per-rank seed",
            "impl": "ours",
            "verified": ok,
            "wall_ms_per_step": round(wall * 1e3 / args.steps, 4),
            "config": {
                "model": CONFIG_MODEL,
                "block_bytes": block,
                "batch_descs": batch,
                "global_batch": env.world * batch,
                "seq_len": None,
                "bytes_per_step_per_gpu": step_bytes,
                "parallelism": f"ring{env.world}" if env.world > 1 else "loopback (second buffer on the same GPU)",
                "engine": "NVLINK backend defaults: descriptors that continue their predecessor are merged (the 16 blocks of this request are one "
                          "1 GiB run), copy kernel below 96 MiB per merged descriptor, copy engines from 96 MiB between GPUs; "
                          "extras.baselines.headline_scattered_GBps is the same request with the destination blocks in reverse order (nothing to merge)",
                "l2": "inputs larger than L2 (1 GiB source and destination per GPU); no flush needed",
                "timing": "CUDA events on the launching stream, max over ranks; two identical requests are posted alternately (depth two: "
                          "a request is posted again only after it completed) so the stream does not wait for the host between steps; "
                          "warm-up = W steps plus further steps for 0.25 s while the clock sampler starts",
                "roofline": roofline(env, gbs),
            },
            "clocks": clocks,
            "e2e": {
                "value": round(e2e_gbs, 2),
                "unit": "GB/s",
                "steps": e2e_steps,
                "h2d_bytes_per_step": step_bytes,
                "d2h_bytes_per_step": batch * 8,
                "what": "pinned host -> registered VRAM (H2D), agent WRITE to the neighbour, D2H of a digest of the received buffer; wall clock, max over ranks",
            },
            "gpu_launches": int(launches),
            "gpu_launches_what": "kernels the NVLINK backend launched inside the timed region, counted by the backend "
                                 "(one per step: the completion kernel behind the copy-engine copies, or the copy kernel itself)",
            "total_s": round(time.perf_counter() - t_start, 1),
            "extras": extras,
        }
        print(json.dumps(out))
    if env.world > 1:
        dist.destroy_process_group()
    return 0 if ok else 1


# ====================================================================== extras: baselines


def extras_baselines(env, args, headline_gbs, budget_s):
    """The headline ring step by other means, same buffers, same sizes, device-timed."""
    torch, dist = env.torch, env.dist
    block, batch = args.block, args.batch
    step_bytes = block * batch
    steps = max(5, min(args.steps, 20))
    out = {"steps": steps, "bytes_per_step_per_gpu": step_bytes}

    for key, tag, params, scattered in (("copy_engine_per_descriptor_GBps", "bce", {"copy_path": "ce", "coalesce": "false"}, False),
                                        ("copy_kernel_only_GBps", "bk", {"ce_threshold": "0"}, False),
                                        ("headline_scattered_GBps", "bench", None, True),
                                        ("headline_repeat_GBps", "bench", None, False)):  # the headline once more, timed like the other arms
        agent = make_agent(env, tag, params) if params is not None else env.agent
        h = [ring_handle(env, agent, tag, block, batch, scattered) for _ in range(2)]  # depth two, as the headline
        ms, _ = time_ring(env, agent, h, steps, 3)
        ms = max_over_ranks(env, [ms])[0]
        out[key] = round(env.world * step_bytes * steps / (ms * 1e-3) / 1e9, 2)
        for x in h:
            agent.release_xfer_handle(x)

    if env.world > 1:
        # NCCL send/recv ring: the whole step as one message each way.
        nxt, prv = (env.rank + 1) % env.world, (env.rank - 1) % env.world
        send, recv = env.src[:step_bytes], env.dst[:step_bytes]

        def nccl_step():
            ops = [dist.P2POp(dist.isend, send, nxt), dist.P2POp(dist.irecv, recv, prv)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()

        for _ in range(3):
            nccl_step()
        barrier(env)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            nccl_step()
        ev1.record()
        barrier(env)
        ms = max_over_ranks(env, [ev0.elapsed_time(ev1)])[0]
        out["nccl_send_recv_GBps"] = round(env.world * step_bytes * steps / (ms * 1e-3) / 1e9, 2)
    out["headline_GBps"] = round(headline_gbs, 2)
    for k in ("copy_engine_per_descriptor_GBps", "copy_kernel_only_GBps", "nccl_send_recv_GBps", "headline_scattered_GBps"):
        if out.get(k):
            out["headline_over_" + k[:-5]] = round(headline_gbs / out[k], 3)
    out["note"] = ("aggregate over all GPUs; the copy-engine arm is what a descriptor-at-a-time transport (UCX cuda_ipc) does for these sizes, "
                   "with merging switched off; the engine itself uses the copy engines from 96 MiB per (merged) descriptor; the copy kernel wins at small and batched descriptors (sweep)")
    return out


# ====================================================================== extras: sweep


def extras_sweep(env, args, headline_gbs, budget_s):
    """nixlbench-style sweep: WRITE and READ, 4 KiB .. 1 GiB (powers of 4), 1 / 16 / 256 descriptors per
    request; ring (loopback at N = 1, pairwise at N = 2) and all-to-all.  GB/s per GPU is device-timed
    with up to four requests in flight; p50 / p99 are host-timed post -> completion of one request."""
    import numpy as np

    torch = env.torch
    t_end = time.perf_counter() + min(budget_s - 3.0, 60.0)
    W, rank = env.world, env.rank
    if W == 1:
        patterns = ["loopback"]
    elif W == 2:
        patterns = ["pairwise"]
    else:
        patterns = ["ring", "all2all"]
    sizes = [4096 << (2 * i) for i in range(10)]  # 4 KiB .. 1 GiB
    side = [torch.cuda.Stream(device=env.dev) for _ in range(max(1, W - 1))]
    entries, pending = [], []
    verified = {}
    truncated = False

    def descs(base, n, size, dev, reverse=False):
        a = np.empty((n, 3), dtype=np.uint64)
        order = np.arange(n, dtype=np.uint64)
        a[:, 0] = base + (order[::-1] if reverse else order) * np.uint64(size)
        a[:, 1] = size
        a[:, 2] = dev
        return a

    for op in ("WRITE", "READ"):
        for pattern in patterns:
            peers = [(rank + 1 + j) % W for j in range(W - 1)] if pattern == "all2all" else [(rank + 1) % W]
            slot = GIB // (W if pattern == "all2all" else 1)
            for nbatch in (1, 16, 256):
                for size in sizes:
                    total = nbatch * size
                    if total > slot:
                        continue
                    stop = time.perf_counter() > t_end
                    if not all_agree(env, not stop):
                        truncated = True
                        break
                    depth = 8 if total <= (2 << 20) else (4 if total <= (4 << 20) else 1)
                    handles = []
                    for j, p in enumerate(peers):
                        if op == "WRITE":  # my src slice j -> slot `rank` of the peer's dst
                            loc = descs(env.src.data_ptr() + j * slot, nbatch, size, env.local_rank)
                            rem = descs(env.dst_ptrs[p] + (rank if pattern == "all2all" else 0) * slot, nbatch, size, env.devs[p], reverse=True)
                        else:              # the peer's src slice 0 -> slot j of my dst
                            loc = descs(env.dst.data_ptr() + j * slot, nbatch, size, env.local_rank)
                            rem = descs(env.src_ptrs[p], nbatch, size, env.devs[p], reverse=True)
                        hs = [env.agent.initialize_xfer(op, env.agent.get_xfer_descs(loc, "VRAM"), env.agent.get_xfer_descs(rem, "VRAM"), f"bench{p}")
                              for _ in range(depth)]
                        handles.append(hs)
                    est_us = max(12.0, total / 700e3)
                    iters = 400 if total <= (2 << 20) else int(min(64, max(3, 12000.0 / est_us)))
                    iters -= iters % depth if iters >= depth else 0
                    # warm-up: every handle once
                    tag = f"[{op} {pattern} batch {nbatch} size {size}"
                    for hs in handles:
                        for h in hs:
                            if not post(env, env.agent, h):
                                wait_done(env, env.agent, h, 10.0, tag + " warm-up]")
                    barrier(env)
                    # Requests of up to 2 MiB go through the engine's doorbell proxy, which runs outside any stream the
                    # caller could time: those are timed on the host (wall clock around the pipelined loop, no
                    # synchronisation inside); larger ones with CUDA events on the streams they are posted on.
                    host_timed = total <= (2 << 20)
                    if host_timed:
                        depth_now = depth
                        t0 = time.perf_counter()
                        for it in range(iters):
                            for j, hs in enumerate(handles):
                                h = hs[it % depth_now]
                                if it >= depth_now:
                                    wait_done(env, env.agent, h, 10.0, tag + f" timed loop it {it}]")
                                post(env, env.agent, h)
                        for hs in handles:
                            for h in hs:
                                wait_done(env, env.agent, h, 10.0, tag + " timed loop end]")
                        dev_ms = (time.perf_counter() - t0) * 1e3
                        barrier(env)
                    else:
                        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        ev0.record(env.stream)
                        for s in side[: len(peers)]:
                            s.wait_event(ev0)
                        for it in range(iters):
                            for j, hs in enumerate(handles):
                                h = hs[it % depth]
                                if it >= depth:
                                    wait_done(env, env.agent, h, 10.0, tag + f" timed loop it {it}]")
                                post(env, env.agent, h, f"stream={side[j].cuda_stream}")
                        for s in side[: len(peers)]:
                            e = torch.cuda.Event()
                            e.record(s)
                            env.stream.wait_event(e)
                        ev1.record(env.stream)
                        for hs in handles:
                            for h in hs:
                                wait_done(env, env.agent, h, 10.0, tag + " timed loop end]")
                        barrier(env)
                        dev_ms = ev0.elapsed_time(ev1)
                    # host-timed latency of one step (every peer's request posted, then all polled)
                    n_lat = 40 if total <= (16 << 20) else 6
                    lat = []
                    for i in range(n_lat + 3):
                        t0 = time.perf_counter()
                        done = [post(env, env.agent, hs[0]) for hs in handles]
                        for d, hs in zip(done, handles):
                            if not d:
                                wait_done(env, env.agent, hs[0], 10.0, tag + f" latency loop {i}]")
                        if i >= 3:
                            lat.append((time.perf_counter() - t0) * 1e6)
                    lat.sort()
                    p50, p99 = lat[len(lat) // 2], lat[min(len(lat) - 1, int(len(lat) * 0.99))]
                    pending.append((dev_ms, p50, p99))
                    entries.append({"op": op, "pattern": pattern, "batch": nbatch, "bytes": size, "iters": iters, "in_flight": depth,
                                    "timed": "host" if host_timed else "device",
                                    "_moved": len(peers) * total * iters})
                    # value check of the largest request of every (op, pattern, batch)
                    if size == max(s for s in sizes if nbatch * s <= slot):
                        torch.cuda.synchronize()
                        good = True
                        for j, p in enumerate(peers):
                            if op == "WRITE":
                                who = (rank - 1 - j) % W  # the rank whose j-th peer I am
                                got = env.dst[(who if pattern == "all2all" else 0) * slot:][:total]
                                want = fill_src(env, who)[j * slot:][:total]
                            else:
                                got = env.dst[j * slot:][:total]
                                want = fill_src(env, p)[:total]
                            # block i of one side pairs with block nbatch-1-i of the other
                            good = good and bool(torch.equal(got.view(nbatch, size).flip(0), want.view(nbatch, size)))
                            del want
                        key = f"{op}/{pattern}"
                        verified[key] = verified.get(key, True) and good
                    for hs in handles:
                        for h in hs:
                            env.agent.release_xfer_handle(h)
                if truncated:
                    break
            if truncated:
                break
        if truncated:
            break

    flat = [v for t in pending for v in t]
    flat = max_over_ranks(env, flat) if flat else []
    for i, e in enumerate(entries):
        dev_ms, p50, p99 = flat[3 * i: 3 * i + 3]
        moved = e.pop("_moved")
        e["GBps_per_gpu"] = round(moved / (dev_ms * 1e-3) / 1e9, 2)
        e["p50_us"], e["p99_us"] = round(p50, 1), round(p99, 1)
    ok_all = {k: all_agree(env, v) for k, v in sorted(verified.items())}
    return {"entries": entries, "verified": ok_all, "truncated": truncated,
            "note": "GB/s per GPU: bytes one GPU sent (WRITE) or fetched (READ) / time of the pipelined loop, max over ranks (requests of up to 2 MiB "
                    "run through the doorbell proxy outside any stream and are timed on the host, larger ones on the device); p50/p99: host-timed post -> completion "
                    "of one step (all2all: one request per peer), max over ranks; engine defaults; descriptors of one request are laid out so that none continues its predecessor (destination blocks in reverse order)"}


# ====================================================================== extras: KV transfer


def extras_kv(env, args, headline_gbs, budget_s):
    """Disaggregated KV-cache transfer, Llama-3-8B shape: 32 layers x (K, V), 8 KV heads, head_dim 128, bf16,
    blocks of 16 tokens, 8 requests x 4096-token prompts, block tables shuffled by a seeded permutation.
    The first half of the GPUs are prefill ranks sharing the 8 heads (TP = N/2), the second half decode
    ranks at half that TP degree, i.e. two decode replicas which take four requests each (8 GPUs: prefill
    TP4 with 2 heads per GPU -> decode TP2 with 4 heads per GPU on GPUs 4-5 and 6-7).  One launch per
    destination GPU; ms/request = device time of the whole batch (max over ranks) / 8."""
    from nixl_b200 import nixl_agent, nixl_agent_config
    from nixl_b200.ops import KVLayout, KVTransfer, reference_kv_transfer

    torch, dist = env.torch, env.dist
    W, rank, dev = env.world, env.rank, env.dev
    layers, requests, prompt, tokens, head_dim, total_heads = 32, 8, 4096, 16, 128, 8
    n_tensors = layers * 2
    blocks_per_req = prompt // tokens
    n_blocks = requests * blocks_per_req
    if W == 1:
        n_prefill, n_decode, replicas = 1, 1, 1
    else:
        n_prefill = W // 2
        n_decode = W - n_prefill
        replicas = 2 if n_decode >= 2 and n_decode % 2 == 0 else 1
    dec_tp = n_decode // replicas                      # decode ranks per replica
    src_heads = total_heads // n_prefill               # heads per prefill rank
    dst_heads = total_heads // dec_tp                  # heads per decode rank
    is_prefill = rank < n_prefill
    is_decode = rank >= n_prefill or W == 1
    first_decode = 0 if W == 1 else n_prefill

    def src_tensor(prank, t):
        g = torch.Generator(device=dev).manual_seed(70000 + prank * 1000 + t)
        return torch.randn(n_blocks, tokens, src_heads, head_dim, device=dev, dtype=torch.bfloat16, generator=g)

    agent = nixl_agent(f"kv{rank}", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
    src = dst = dst8 = None
    if is_prefill:
        src = [src_tensor(rank, t) for t in range(n_tensors)]
        agent.register_memory(src)
    if is_decode:
        dst = [torch.zeros(n_blocks, tokens, dst_heads, head_dim, device=dev, dtype=torch.bfloat16) for _ in range(n_tensors)]
        dst8 = [torch.zeros(n_blocks, tokens, dst_heads, head_dim, device=dev, dtype=torch.uint8) for _ in range(n_tensors)]
        agent.register_memory(dst)
        agent.register_memory(dst8)
    info = {"md": agent.get_agent_metadata(), "name": agent.name,
            "dst": [(t.data_ptr(), t.numel() * 2, env.local_rank) for t in dst] if is_decode else None,
            "dst8": [(t.data_ptr(), t.numel(), env.local_rank) for t in dst8] if is_decode else None}
    infos = [info]
    if W > 1:
        infos = [None] * W
        dist.all_gather_object(infos, info)

    # Which decode GPUs does prefill rank p feed, with which requests, at which head slot?
    def targets_of(p):
        heads_lo = p * src_heads
        tp_rank, head_off = heads_lo // dst_heads, heads_lo % dst_heads
        per = requests // replicas
        return [(first_decode + rep * dec_tp + tp_rank, range(rep * per, (rep + 1) * per), head_off) for rep in range(replicas)]

    perm = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(123)).int()
    dperm = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(321)).int()

    def tables(reqs):
        idx = torch.cat([torch.arange(r * blocks_per_req, (r + 1) * blocks_per_req) for r in reqs])
        return perm[idx].to(dev), dperm[idx].to(dev)

    out = {"n_gpus": W, "prefill_ranks": n_prefill, "decode_ranks": n_decode, "decode_replicas": replicas, "heads_per_prefill_rank": src_heads,
           "heads_per_decode_rank": dst_heads, "requests": requests, "prompt_tokens": prompt, "blocks": n_blocks,
           "bytes_per_prefill_rank_bf16": n_tensors * n_blocks * tokens * src_heads * head_dim * 2}
    my_targets = targets_of(rank) if is_prefill else []
    for t_rank, _, _ in my_targets:
        if t_rank != rank:
            agent.add_remote_agent(infos[t_rank]["md"])
    streams = [torch.cuda.Stream(device=dev) for _ in my_targets]
    iters = 5
    verified = True
    # Prefill rank p starts with replica p % replicas: the senders of one decode GPU do not all arrive at once.
    my_targets = my_targets[rank % len(my_targets):] + my_targets[:rank % len(my_targets)] if my_targets else []
    for fp8 in (False, True):
        xfers = []
        for t_rank, reqs, head_off in my_targets:
            x = KVTransfer(agent, src, KVLayout(tokens, src_heads, head_dim), infos[t_rank]["name"], infos[t_rank]["dst8" if fp8 else "dst"],
                           KVLayout(tokens, dst_heads, head_dim, elem_bytes=1 if fp8 else 2), dst_head_offset=head_off, cast_fp8=fp8)
            xfers.append((x, *tables(reqs)))
        times = []
        for i in range(iters + 2):
            barrier(env)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for (x, sb, db), s in zip(xfers, streams):
                s.wait_event(e0)
                x.post(sb, db, stream=s)
                e = torch.cuda.Event()
                e.record(s)
                torch.cuda.current_stream().wait_event(e)
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(e0.elapsed_time(e1))
        times.sort()
        ms = max_over_ranks(env, [times[len(times) // 2]])[0]
        key = "fp8" if fp8 else "bf16"
        out[f"fused_{key}_ms_per_batch"] = round(ms, 4)
        out[f"fused_{key}_ms_per_request"] = round(ms / requests, 4)
        out[f"fused_{key}_GBps_per_prefill_rank"] = round(out["bytes_per_prefill_rank_bf16"] / (ms * 1e-3) / 1e9, 1)
        barrier(env)
        # value check on every decode rank: four of the 64 cache tensors against the PyTorch statement
        if is_decode:
            for t in (0, 21, 42, n_tensors - 1):
                want = torch.zeros(n_blocks, tokens, dst_heads, head_dim, device=dev, dtype=torch.uint8 if fp8 else torch.bfloat16)
                if fp8:
                    want = want.view(torch.float8_e4m3fn)
                for p in range(n_prefill):
                    for t_rank, reqs, head_off in targets_of(p):
                        if t_rank != rank:
                            continue
                        idx = torch.cat([torch.arange(r * blocks_per_req, (r + 1) * blocks_per_req) for r in reqs])
                        reference_kv_transfer(src_tensor(p, t), want, perm[idx].to(dev), dperm[idx].to(dev), head_off, cast_fp8=fp8)
                got = dst8[t] if fp8 else dst[t]
                verified = verified and bool(torch.equal(got.view(torch.uint8), want.view(torch.uint8)))
        for x, _, _ in xfers:
            x.close()
    out["verified"] = all_agree(env, verified)
    out["launches_per_batch_per_prefill_rank"] = len(my_targets) if is_prefill else 0
    del src, dst, dst8
    torch.cuda.empty_cache()
    return out


# ====================================================================== extras: EP dispatch / combine


def extras_ep(env, args, headline_gbs, budget_s):
    """MoE expert-parallel dispatch + combine, DeepSeek-V3 shape: hidden 7168, 32 routed experts per GPU, top-8
    from seeded N(0,1) router logits with softmax weights, bf16 tokens N(0,1); dispatch carries e4m3 with 1x128
    fp32 scales, combine returns bf16 with the top-k weighted sum.  Low-latency mode 128 tokens per GPU,
    throughput mode 4096.  Device-timed, L2 flushed between iterations, max over ranks.  `verified`: on EVERY
    rank, the per-expert receive counts against all ranks' routing and the combined output against the fp32
    PyTorch statement  out[t] = sum_k w[t,k] * bf16(dequant(fp8(x[t])) * (1 + e[t,k]) / 100)  (tolerances in the code)."""
    from nixl_b200.parallel import Buffer, dequant_fp8, per_token_cast_to_fp8

    torch, dist = env.torch, env.dist
    W, rank, dev = env.world, env.rank, env.dev
    H, El, K = 7168, 32, 8
    E = El * W
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    out = {"n_gpus": W, "hidden": H, "experts": E, "topk": K}
    t_limit = time.perf_counter() + budget_s - 2.0

    def timed(fn, iters=8, warmup=3, pre=None):
        ts = []
        for i in range(warmup + iters):
            if pre is not None:
                pre()
            flush.add_(1)
            barrier(env)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(400_000)  # the GPU stays busy while the host queues fn(): the events see device time only
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= warmup:
                ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        return max_over_ranks(env, [ts[len(ts) // 2]])[0]

    for mode, T in (("low_latency", 128), ("throughput", 4096)):
        if not all_agree(env, time.perf_counter() < t_limit - (4.0 if mode == "low_latency" else 12.0)):
            out[mode] = {"skipped": "the extras' time budget was spent"}
            continue
        gen = torch.Generator(device=dev).manual_seed(1000 + rank)
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16, generator=gen)
        logits = torch.randn(T, E, device=dev, generator=gen)
        w, idx = torch.topk(torch.softmax(logits, dim=-1), K, dim=-1)
        idx, w = idx.to(torch.int64).contiguous(), w.float().contiguous()
        compact = mode == "throughput"
        buf = Buffer(rank, W, E, H, T, K, device=dev, timeout_ms=20000, low_latency_mode=not compact)
        buf.connect_ranks()
        state = {}

        def do_dispatch():
            if compact:
                # the weights go along: the expert ranks can then add a token's rows up before they return one row
                state["rx"], state["sc"], state["h"] = buf.dispatch(x, idx, use_fp8=True, topk_weights=w)
            else:
                (rx, sc), _, h, _, _ = buf.low_latency_dispatch(x, idx, use_fp8=True)
                state["rx"], state["sc"], state["h"] = rx.view(-1, H), sc.view(-1, H // 128), h

        def do_combine():
            # the expert GEMM writes into the exposed buffer; low-latency mode: the home ranks pull their rows from it;
            # throughput mode: each expert rank reduces a token's rows and stores one row at the token's home rank
            src = buf.get_next_combine_buffer(state["h"])
            if compact:
                state["o"] = buf.combine(src.view(-1, H), idx, w, state["h"])
            else:
                state["o"] = buf.low_latency_combine(src, idx, w, state["h"])[0]

        def both():
            do_dispatch()
            do_combine()

        # ---- value check on this rank (before timing)
        do_dispatch()
        torch.cuda.synchronize()
        h = state["h"]
        all_idx = [idx]
        if W > 1:
            all_idx = [torch.empty_like(idx) for _ in range(W)]
            dist.all_gather(all_idx, idx)
        flat = torch.cat([a.reshape(-1) for a in all_idx])
        want_counts = torch.bincount(flat[(flat >= rank * El) & (flat < (rank + 1) * El)] - rank * El, minlength=El)
        good = bool(torch.equal(h.recv_count.to(torch.int64), want_counts))
        y = buf.get_next_combine_buffer(h).view(-1, H)
        offs, cnts = h.expert_offsets.tolist(), h.recv_count.tolist()
        for le in range(El):
            s, c = offs[le], cnts[le]
            if c:
                y[s:s + c] = (dequant_fp8(state["rx"][s:s + c], state["sc"][s:s + c]) * ((1 + rank * El + le) * 0.01)).to(torch.bfloat16)
        do_combine()
        torch.cuda.synchronize()
        base = dequant_fp8(*per_token_cast_to_fp8(x))
        want = torch.zeros(T, H, device=dev)
        for k in range(K):
            yk = (base * ((1 + idx[:, k]).float() * 0.01).unsqueeze(1)).to(torch.bfloat16).float()
            want += w[:, k].unsqueeze(1) * yk
        err = (state["o"].float() - want.to(torch.bfloat16).float()).abs()
        # The kernel and PyTorch round x * (448 / amax) differently on exact ties, so a few e4m3 codes sit one
        # step apart (one step is up to 1/8 of the value, and the same x feeds all k terms of a token): nearly
        # all elements must agree to bf16 accuracy, every element to one fp8 step.
        wabs = want.to(torch.bfloat16).float().abs()
        tight = err <= 2e-2 + 2e-2 * wabs
        loose = err <= 2e-2 + 0.13 * wabs
        frac_tight = float(tight.float().mean())
        good = good and frac_tight >= 0.98 and bool(loose.all()) and buf.status == 0
        max_err = float(err.max())
        del base, want, err, wabs, tight, loose

        t_disp = timed(do_dispatch)
        t_comb = timed(do_combine, pre=do_dispatch)
        t_both = timed(both)
        recv_rows = int(state["h"].recv_count.sum())
        rec = {
            "tokens_per_gpu": T, "dispatch_us": round(t_disp, 1), "combine_us": round(t_comb, 1), "dispatch_plus_combine_us": round(t_both, 1),
            "recv_rows_rank0": recv_rows, "status": buf.status, "verified": all_agree(env, good), "max_abs_err": round(max_over_ranks(env, [max_err])[0], 4),
            "fraction_within_bf16_tolerance": round(min_over_ranks(env, [frac_tight])[0], 5),
            "combine": "rank-reduced (expert ranks add a token's rows up, one row per (token, rank) returns)" if compact else
                       "pull (home ranks load expert outputs from the exposed buffer)",
        }
        # wire bytes per GPU and the link-time bound (rows that leave this GPU; about (W-1)/W of the copies)
        remote_rows = int(((idx // El) != rank).sum())
        remote_pairs = int(sum(int((((idx // El) == r).any(dim=1)).sum()) for r in range(W) if r != rank))  # (token, remote rank) pairs
        wire = remote_rows * (H + H // 128 * 4) + (remote_pairs if compact else remote_rows) * H * 2
        rec["wire_bytes_per_gpu"] = wire
        if W > 1:
            rec["fraction_of_900GBps_link_bound"] = round((wire / 900e9 * 1e6) / t_both, 3)
        out[mode] = rec
        buf.destroy()
        del buf, x, logits, y
        state.clear()
        torch.cuda.empty_cache()
    return out


# ====================================================================== extras: GPU-initiated put with signal


def extras_dput(env, args, headline_gbs, budget_s):
    """A persistent kernel on every GPU puts 256 KiB tiles to every peer from inside its compute loop (1024 iterations
    per peer, 20 producer CTAs per peer taking turns, 40 landing slots) with nixlPut<BLOCK> + nixlAtomicAdd of the device API; a consumer
    CTA waits on the per-slot counters the peers bump and acknowledges, which gates the reuse of a landing slot.  One GPU:
    the rank puts to itself.  Device-timed, max over ranks.  `verified`: the kernel's status word is clean, every peer's
    counters add up to the iterations, and after the communication-only run every landing slot holds the source tile
    of the producer CTA that wrote it last."""
    from nixl_b200 import nixl_agent, nixl_agent_config
    from nixl_b200.ops import device_api

    torch, dist = env.torch, env.dist
    W, rank, dev, local = env.world, env.rank, env.dev, env.local_rank
    tile, window, cpp, iters = 256 << 10, 40, 20, 1024
    peers = [r for r in range(W) if r != rank] or [rank]
    P = len(peers)
    agent = nixl_agent(f"dput{rank}", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
    tiles = torch.randn(P * cpp * tile // 4, dtype=torch.float32, device=dev)  # one source tile per producer CTA
    landing = torch.zeros(W * window * tile, dtype=torch.uint8, device=dev)
    signals = torch.zeros(2 * W * window, dtype=torch.int64, device=dev)  # arrival[rank][slot], then acknowledgement[rank][slot]
    for t in (tiles, landing, signals):
        agent.register_memory(t)
    info = {"md": agent.get_agent_metadata(), "landing": (landing.data_ptr(), landing.numel(), local),
            "signals": (signals.data_ptr(), signals.numel() * 8, local), "name": agent.name}
    infos = [info]
    if W > 1:
        infos = [None] * W
        dist.all_gather_object(infos, info)
    for r, i in enumerate(infos):
        if r != rank:
            agent.add_remote_agent(i["md"])
    views = [agent.prep_mem_view(agent.get_xfer_descs(tiles)), agent.prep_mem_view(agent.get_xfer_descs(signals)),
             agent.prep_mem_view(agent.get_remote_descs([i["landing"] + (i["name"],) for i in infos], "VRAM")),
             agent.prep_mem_view(agent.get_remote_descs([i["signals"] + (i["name"],) for i in infos], "VRAM"))]
    peer_ids = torch.tensor(peers, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def run(n, passes):
        signals.zero_()
        barrier(env)
        p = device_api.DevPutParams()
        p.local_tiles, p.local_signals, p.remote_tiles, p.remote_signals = views
        p.peer_ids = peer_ids.data_ptr()
        p.peers, p.rank, p.iters, p.window, p.compute_passes, p.ctas_per_peer = P, rank, n, window, passes, cpp
        p.tile_bytes, p.ack_offset, p.timeout_ns = tile, W * window * 8, 10_000_000_000
        p.status = status.data_ptr()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        device_api.put_signal_launch(p, dev)
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(env, [e0.elapsed_time(e1) * 1e3])[0]

    run(64, 1)
    t_full = run(iters, 1)
    def arrived_all():
        arrived = signals[: W * window].view(W, window).sum(dim=1)
        return all(int(arrived[r]) == iters for r in peers)

    ok = int(status.item()) == 0 and arrived_all()
    t_comm = run(iters, 0)
    ok = ok and int(status.item()) == 0 and arrived_all()
    all_tiles = [tiles]
    if W > 1:
        all_tiles = [torch.empty_like(tiles) for _ in range(W)]
        dist.all_gather(all_tiles, tiles)
    for r in peers:
        pi = ([x for x in range(W) if x != r] or [r]).index(rank)
        for slot in range(window):
            last_it = slot + 1 + ((iters - 1 - slot) // window) * window
            cta = pi * cpp + (last_it - 1) % cpp
            want = all_tiles[r].view(torch.uint8)[cta * tile:(cta + 1) * tile]
            got = landing[(r * window + slot) * tile:(r * window + slot + 1) * tile]
            ok = ok and bool(torch.equal(want, got))
    del all_tiles
    out = {"n_gpus": W, "peers_per_gpu": P, "tile_bytes": tile, "iters": iters, "window": window, "ctas_per_peer": cpp,
           "us_per_iter": round(t_full / iters, 2), "us_per_put": round(t_full / iters / P, 2), "us_per_iter_comm_only": round(t_comm / iters, 2),
           "GBps_per_gpu": round(P * tile * iters / t_full / 1e3, 1), "GBps_per_gpu_comm_only": round(P * tile * iters / t_comm / 1e3, 1),
           "verified": all_agree(env, ok)}
    barrier(env)
    for v in views:
        agent.release_mem_view(v)
    return out


if __name__ == "__main__":
    sys.exit(main())

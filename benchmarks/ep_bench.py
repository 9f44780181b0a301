#!/usr/bin/env python
"""MoE expert-parallel dispatch/combine benchmark (DeepSeek-V3 shape).

hidden 7168, 32 routed experts per GPU, top-8 routing from seeded N(0,1) router logits with
softmax weights, bf16 tokens N(0,1); dispatch carries e4m3 with 1x128 fp32 scales, combine
returns bf16 with the top-k weighted sum.  Modes: low-latency (128 tokens/GPU, expert-major
layout) and throughput (4096 tokens/GPU, compact layout).  Also times the grouped expert
up-projection 7168 -> 2048 (fp8 weights, 128x128 block scales) stand-alone and fused behind
the dispatch, and an unfused baseline (torch quantise -> NCCL all_to_all_single -> permute ->
weighted sum).

Device-timed with CUDA events (max over ranks), L2 flushed between iterations by writing a
256 MiB buffer.  Launch: ``python benchmarks/ep_bench.py`` or under
``python -m torch.distributed.run --nproc-per-node N benchmarks/ep_bench.py``.
Prints one JSON object per line on rank 0.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from nixl_b200.ops import grouped_gemm_fp8, grouped_gemm_mxfp8, quantize_weights, quantize_weights_ue8m0  # noqa: E402
from nixl_b200.parallel import Buffer, per_token_cast_to_fp8  # noqa: E402


def timed(fn, iters, warmup, flush, world, dev, pre=None):
    """Median device time of fn() in microseconds, max over ranks."""
    times = []
    for i in range(warmup + iters):
        if pre is not None:
            pre()
        flush.add_(1)  # > L2: evicts what the previous iteration left behind
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(400_000)  # keeps the GPU busy while the host queues fn(): the events then see device time only
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(e0.elapsed_time(e1) * 1e3)
    times.sort()
    med = torch.tensor([times[len(times) // 2]], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(med, op=dist.ReduceOp.MAX)
    return float(med)


def baseline_dispatch_combine(x, topk_idx, topk_w, world, El):
    """Unfused reference pipeline on NCCL (what a framework does without an EP library)."""
    T, H = x.shape
    K = topk_idx.shape[1]
    q, s = per_token_cast_to_fp8(x)
    flat_e = topk_idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = order // K
    send_q = q.view(torch.uint8)[tok]
    send_s = s[tok]
    send_e = flat_e[order]
    dst = send_e // El
    send_counts = torch.bincount(dst, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    if world > 1:
        dist.all_to_all_single(recv_counts, send_counts)
    else:
        recv_counts.copy_(send_counts)
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    n_recv = sum(rc)
    recv_q = torch.empty(n_recv, H, dtype=torch.uint8, device=x.device)
    recv_s = torch.empty(n_recv, H // 128, dtype=torch.float32, device=x.device)
    recv_e = torch.empty(n_recv, dtype=torch.int64, device=x.device)
    if world > 1:
        dist.all_to_all_single(recv_q, send_q, rc, sc)
        dist.all_to_all_single(recv_s, send_s, rc, sc)
        dist.all_to_all_single(recv_e, send_e, rc, sc)
    else:
        recv_q.copy_(send_q), recv_s.copy_(send_s), recv_e.copy_(send_e)
    perm = torch.argsort(recv_e, stable=True)  # expert-major packing
    packed = recv_q[perm]
    # "experts": identity in bf16, then the way back
    y = (packed.view(torch.float8_e4m3fn).float().view(n_recv, H // 128, 128) * recv_s[perm].unsqueeze(2)).view(n_recv, H).to(torch.bfloat16)
    back = torch.empty_like(y)
    back[perm] = y
    ret = torch.empty(T * K, H, dtype=torch.bfloat16, device=x.device)
    if world > 1:
        dist.all_to_all_single(ret, back, sc, rc)
    else:
        ret.copy_(back)
    unsort = torch.empty_like(ret)
    unsort[order] = ret
    return (unsort.view(T, K, H).float() * topk_w.unsqueeze(2)).sum(1).to(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts-per-rank", type=int, default=32)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--modes", default="ll,tp")
    ap.add_argument("--num-sms", type=int, default=0, help="grid of the dispatch / combine kernels (0: one CTA per SM)")
    ap.add_argument("--skip-baseline", action="store_true")
    ap.add_argument("--skip-gemm", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    H, El, K = args.hidden, args.experts_per_rank, args.topk
    E = El * world
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    out = []

    for mode in args.modes.split(","):
        T = 128 if mode == "ll" else 4096
        gen = torch.Generator(device=dev).manual_seed(1000 + rank)
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16, generator=gen)
        logits = torch.randn(T, E, device=dev, generator=gen)
        w, idx = torch.topk(torch.softmax(logits, dim=-1), K, dim=-1)
        idx, w = idx.to(torch.int64).contiguous(), w.float().contiguous()
        compact = mode != "ll"
        buf = Buffer(rank, world, E, H, T, K, device=dev, timeout_ms=20000, low_latency_mode=not compact)
        buf.connect_ranks()
        if args.num_sms:
            buf.set_num_sms(args.num_sms)

        state = {}

        def do_dispatch():
            if compact:
                state["rx"], state["sc"], state["h"] = buf.dispatch(x, idx, use_fp8=True)
            else:
                (rx, sc), cnt, h, _, _ = buf.low_latency_dispatch(x, idx, use_fp8=True)
                state["rx"], state["sc"], state["h"] = rx.view(-1, H), sc.view(-1, H // 128), h

        do_dispatch()
        torch.cuda.synchronize()
        rows_total = state["rx"].shape[0]
        y = torch.randn(rows_total, H, device=dev, dtype=torch.bfloat16) if rows_total * H * 2 < (8 << 30) else torch.zeros(
            rows_total, H, device=dev, dtype=torch.bfloat16)

        variant = {"v": "default"}

        def do_combine():
            # push: expert ranks store rows into the home rank's landing zone, which then reduces;
            # pull: home ranks load rows from the expert ranks' exposed output buffer and reduce;
            # pull_copy: same, but the outputs first have to be copied into that buffer;
            # push_logfmt: push with rows in the logarithmic 10-bit format (0.66 of the bytes on the wire).
            v = variant["v"]
            if v == "default":  # what a pipeline does: the expert GEMM writes into the exposed buffer
                v = "pull"
            logfmt = v == "push_logfmt"
            buf.combine_pull = not v.startswith("push")
            src = buf.get_next_combine_buffer(state["h"]).view(-1, H) if v == "pull" else y
            if compact:
                state["o"] = buf.combine(src, idx, w, state["h"], use_logfmt=logfmt)
            else:
                state["o"] = buf.low_latency_combine(src.view(El, -1, H), idx, w, state["h"], use_logfmt=logfmt)[0]

        def both():
            do_dispatch()
            do_combine()

        t_disp = timed(do_dispatch, args.iters, args.warmup, flush, world, dev)
        per_variant = {}
        for v in ("push", "push_logfmt", "pull_copy", "pull") if H % 512 == 0 else ("push", "pull_copy", "pull"):
            variant["v"] = v
            per_variant[f"combine_us_{v}"] = round(timed(do_combine, args.iters, args.warmup, flush, world, dev, pre=do_dispatch), 1)
            per_variant[f"dispatch_plus_combine_us_{v}"] = round(timed(both, args.iters, args.warmup, flush, world, dev), 1)
        variant["v"] = "default"
        t_comb = timed(do_combine, args.iters, args.warmup, flush, world, dev, pre=do_dispatch)
        t_both = timed(both, args.iters, args.warmup, flush, world, dev)
        status = buf.status
        recv_rows = int(state["h"].recv_count.sum())
        disp_bytes = recv_rows * (H + H // 128 * 4 + 8)
        comb_bytes = recv_rows * H * 2
        rec = {
            "bench": "ep", "mode": mode, "n_gpus": world, "tokens_per_gpu": T, "hidden": H, "experts": E, "topk": K,
            "dispatch_us": round(t_disp, 1), "combine_us": round(t_comb, 1), "dispatch_plus_combine_us": round(t_both, 1),
            "recv_rows": recv_rows, "dispatch_GBps_in": round(disp_bytes / t_disp / 1e3, 1), "combine_GBps_out": round(comb_bytes / t_comb / 1e3, 1),
            "status": status, "combine_default": "pull",
        }
        rec.update(per_variant)

        if not args.skip_gemm:
            wt = torch.randn(El, args.inter, H, device=dev, generator=gen) * 0.02
            wq, sw = quantize_weights(wt)
            del wt
            h = state["h"]
            d = torch.empty(rows_total, args.inter, dtype=torch.bfloat16, device=dev)
            st = torch.zeros(1, dtype=torch.int32, device=dev)

            def gemm():
                grouped_gemm_fp8(state["rx"], state["sc"], wq, sw, state["h"].expert_offsets[:El].contiguous(), state["h"].recv_count, out=d, status=st,
                                 tile_mode=2 if compact and args.inter % 256 == 0 else 1)

            def fused():
                # dispatch on a side stream with a small grid; the GEMM consumes arrivals tile by tile
                _, hh, _, _ = buf.dispatch_gemm(x, idx, wq, sw, low_latency=not compact, out=d)
                state["h"] = hh

            def unfused():
                do_dispatch()
                gemm()

            t_gemm = timed(gemm, args.iters, args.warmup, flush, world, dev)
            t_mx = None
            if compact and args.inter % 256 == 0 and H % 512 == 0:
                # Power-of-two scales end to end: dispatch delivers exponent bytes, the tensor core applies them.
                wq2, swb = quantize_weights_ue8m0(torch.randn(El, args.inter, H, device=dev, generator=gen) * 0.02)
                mx = {}

                def dispatch_mx():
                    mx["rx"], mx["sc"], mx["h"] = buf.dispatch(x, idx, use_fp8=True, use_ue8m0=True)

                def gemm_mx():
                    grouped_gemm_mxfp8(mx["rx"], mx["sc"], wq2, swb, mx["h"].expert_offsets, mx["h"].recv_count, out=d, status=st)

                dispatch_mx()
                torch.cuda.synchronize()
                t_mx = timed(gemm_mx, args.iters, args.warmup, flush, world, dev)
                do_dispatch()  # back to the fp32-scale state the following measurements expect
                torch.cuda.synchronize()
                del wq2, swb
            t_unf = timed(unfused, args.iters, args.warmup, flush, world, dev)
            t_fus = timed(fused, args.iters, args.warmup, flush, world, dev)
            flops = 2.0 * recv_rows * args.inter * H
            rec.update({
                "gemm_us": round(t_gemm, 1), "gemm_TFLOPs": round(flops / t_gemm / 1e6, 1),
                "dispatch_then_gemm_us": round(t_unf, 1), "fused_dispatch_gemm_us": round(t_fus, 1),
                "gemm_status": int(st.item()) | int(buf._gemm_status.item()), "gemm_weight_GB": round(El * args.inter * H / 1e9, 3),
            })
            if t_mx is not None:
                rec.update({"gemm_block_scaled_us": round(t_mx, 1), "gemm_block_scaled_TFLOPs": round(flops / t_mx / 1e6, 1)})
            del wq, sw, d

        if not args.skip_baseline:
            t_base = timed(lambda: baseline_dispatch_combine(x, idx, w, world, El), max(5, args.iters // 2), 3, flush, world, dev)
            rec["baseline_unfused_nccl_us"] = round(t_base, 1)
            rec["speedup_vs_baseline"] = round(t_base / t_both, 2)
        out.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)
        buf.destroy()
        del buf, y
        torch.cuda.empty_cache()

    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""``python -m benchmarks.kvbench <command>``

    kvcache                 KV sizes of a model under a parallel layout
    plan                    nixlbench command lines for that geometry
    profile                 run them
    matgen                  traffic matrices + YAML of a prefill -> decode workload
    ct-perftest             time one traffic pattern       (under torchrun, one rank per matrix row)
    sequential-ct-perftest  run a list of patterns in order (under torchrun)
    kv-transfer             fused paged-KV transfer benchmark (under torchrun for more than one GPU)
    storage-perftest        file <-> buffer reads and writes through the POSIX (host) or GDS (CUDA) backend
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _parallel(ns):
    from nixl_b200.models import ParallelConfig

    return ParallelConfig(tp=ns.tp, pp=ns.pp, cp=ns.cp)


def _apply_model_config(ns):
    """Serving configuration file in the reference's layout (benchmark/kvbench/examples/block-tp8-pp2.yaml)."""
    import yaml

    with open(ns.model_config) as f:
        cfg = yaml.safe_load(f) or {}
    strategy, runtime, system = cfg.get("strategy") or {}, cfg.get("runtime") or {}, cfg.get("system") or {}
    ns.tp = int(strategy.get("tp_size", ns.tp))
    ns.pp = int(strategy.get("pp_size", ns.pp))
    ns.cp = int(strategy.get("cp_size", ns.cp))
    ns.kvcache_quant = str(strategy.get("kvcache_quant_mode", ns.kvcache_quant) or "")
    ns.isl = int(runtime.get("isl", ns.isl))
    ns.num_requests = int(runtime.get("num_requests", ns.num_requests))
    ns.page_size = int(system.get("page_size", ns.page_size))


def _add_model_args(p):
    p.add_argument("--model", default="llama-3-8b", help="built-in model name or architecture YAML (model_name, num_layers, num_query_heads, ...)")
    p.add_argument("--model_config", "--model-config", dest="model_config", default="",
                   help="YAML with strategy (tp_size, pp_size, kvcache_quant_mode), runtime (isl, num_requests) and system (page_size); overrides the flags")
    p.add_argument("--kvcache-quant", default="", help="fp8 | bf16 | fp16 | fp32 (bytes per cached element)")
    p.add_argument("--isl", type=int, default=4096, help="prompt length in tokens")
    p.add_argument("--num-requests", type=int, default=1)
    p.add_argument("--tp", type=int, default=1)
    p.add_argument("--pp", type=int, default=1)
    p.add_argument("--cp", type=int, default=1)
    p.add_argument("--page-size", type=int, default=16)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="kvbench", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)

    p = sub.add_parser("kvcache")
    _add_model_args(p)
    p = sub.add_parser("plan")
    _add_model_args(p)
    for q in (p, sub.add_parser("profile")):
        if q is not p:
            _add_model_args(q)
        q.add_argument("--backend", default="NVLINK")
        q.add_argument("--mem", default="VRAM")
        q.add_argument("--op", default="WRITE")
        q.add_argument("--src-dev", type=int, default=0)
        q.add_argument("--dst-dev", type=int, default=1)
        q.add_argument("--iters", type=int, default=200)
        q.add_argument("--extra", default="", help="appended to every nixlbench command")

    p = sub.add_parser("matgen")
    p.add_argument("--model", default="llama-3-8b")
    p.add_argument("--num-user-requests", type=int, default=16)
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--isl-mean", type=int, default=16000)
    p.add_argument("--isl-scale", type=int, default=10000)
    p.add_argument("--min-isl", type=int, default=1000)
    p.add_argument("--max-isl", type=int, default=128000)
    p.add_argument("--prefill-tp", type=int, default=4)
    p.add_argument("--prefill-cp", type=int, default=1)
    p.add_argument("--decode-tp", type=int, default=4)
    p.add_argument("--world-size", type=int, default=8)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--mem-type", default="cuda")
    p.add_argument("--xfer-op", default="WRITE")
    p.add_argument("--results-dir", required=True)

    for name in ("ct-perftest", "sequential-ct-perftest"):
        p = sub.add_parser(name)
        p.add_argument("config", help="YAML file (see benchmarks/kvbench/README.md)")
        p.add_argument("--backend", default="NVLINK")
        p.add_argument("--json-output-path")
        p.add_argument("--no-sleep", action="store_true", help="ignore sleep_before/after_launch_sec")

    sub.add_parser("kv-transfer", add_help=False)

    p = sub.add_parser("storage-perftest")
    p.add_argument("--path", required=True, help="directory for the benchmark files")
    p.add_argument("--size", default="64M")
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--mem", default="cpu", help="cpu / dram or cuda / vram")
    p.add_argument("--chunk", default="0", help="bytes per descriptor (0: one descriptor)")
    p.add_argument("--keep-files", action="store_true")
    p.add_argument("--store", default="file", choices=["file", "obj", "azure_blob"], help="file: POSIX / GDS on --path; obj / azure_blob: an object store")
    p.add_argument("--store-param", action="append", default=[], metavar="KEY=VALUE",
                   help="parameter of the object backend (endpoint_override, bucket, access_key, ...; connection_string, container_name)")

    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "kv-transfer":
        from . import kv_transfer

        sys.argv = ["kv-transfer"] + list(argv[1:])
        return kv_transfer.main()
    ns = ap.parse_args(argv)
    if getattr(ns, "model_config", ""):
        _apply_model_config(ns)

    if ns.cmd == "kvcache":
        from .plan import kvcache_report

        print(json.dumps(kvcache_report(ns.model, ns.isl, ns.num_requests, _parallel(ns), ns.page_size, ns.kvcache_quant), indent=1))
    elif ns.cmd in ("plan", "profile"):
        from .plan import plan_commands, profile

        cmds = plan_commands(ns.model, ns.isl, ns.num_requests, _parallel(ns), ns.page_size, ns.backend, ns.mem, ns.op, ns.src_dev, ns.dst_dev,
                             ns.iters, ns.extra, ns.kvcache_quant)
        if ns.cmd == "plan":
            print("\n".join(cmds))
        else:
            for r in profile(cmds):
                print("$", r["cmd"])
                print(r["stdout"] or r["stderr"])
    elif ns.cmd == "storage-perftest":
        from .storage import storage_perftest
        from .traffic import parse_size

        print(json.dumps(storage_perftest(ns.path, parse_size(ns.size), ns.iters, ns.mem, parse_size(ns.chunk), keep_files=ns.keep_files, store=ns.store,
                                          store_params=dict(kv.split("=", 1) for kv in ns.store_param))))
    elif ns.cmd == "matgen":
        from nixl_b200.models import ParallelConfig

        from .matgen import TaskConfig, generate, write_workload

        task = TaskConfig(ns.isl_mean, ns.isl_scale, ns.min_isl, ns.max_isl, ns.batch_size)
        mats = generate(ns.model, ns.num_user_requests, task, ParallelConfig(tp=ns.prefill_tp, cp=ns.prefill_cp), ParallelConfig(tp=ns.decode_tp),
                        ns.world_size, ns.seed)
        print(write_workload(mats, ns.results_dir, ns.mem_type, ns.xfer_op))
    else:
        import yaml

        from .perftest import ct_perftest, sequential_ct_perftest
        from .traffic import pattern_from_dict

        with open(ns.config) as f:
            cfg = yaml.safe_load(f)
        base = os.path.dirname(os.path.abspath(ns.config))
        if ns.cmd == "ct-perftest":
            tp = pattern_from_dict(cfg["traffic_pattern"], base)
            ct_perftest(tp, int(cfg.get("iters", 50)), int(cfg.get("warmup_iters", 10)), ns.backend, ns.json_output_path)
        else:
            tps = [pattern_from_dict(d, base) for d in cfg["traffic_patterns"]]
            sequential_ct_perftest(tps, ns.backend, ns.json_output_path, honor_sleep=not ns.no_sleep)
    return 0


if __name__ == "__main__":
    sys.exit(main())

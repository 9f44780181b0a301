"""nixlbench plans from a model's KV geometry (the reference's kvbench `plan` / `profile` / `kvcache` commands,
benchmark/kvbench/main.py and commands/nixlbench.py)."""
from __future__ import annotations

import os
import shlex
import subprocess
from typing import List

from nixl_b200.models import MODELS, ParallelConfig, batch_descriptor_count, get_model

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
NIXLBENCH = os.path.join(ROOT, "nixl_b200", "bin", "nixlbench")


def kvcache_report(model_name: str, isl: int, requests: int, par: ParallelConfig, page_size: int, kvcache_quant: str = "") -> dict:
    m = get_model(model_name, kvcache_quant)
    block = m.block_bytes(page_size, par)
    per_gpu = m.kv_bytes_per_gpu(isl, par)
    return {
        "model": model_name, "isl": isl, "num_requests": requests, "tp": par.tp, "pp": par.pp, "cp": par.cp, "page_size": page_size,
        "bytes_per_token_per_gpu": m.bytes_per_token_per_gpu(par),
        "kv_bytes_per_request_per_gpu": per_gpu,
        "kv_bytes_batch_per_gpu": per_gpu * requests,
        "io_size": block,
        "cache_tensors_per_gpu": m.cache_tensors_per_gpu(par),
        "descriptors_per_batch": batch_descriptor_count(m, isl, requests, par, block),
    }


def _pow2_floor(n: int) -> int:
    return 1 << (max(1, n).bit_length() - 1)


def plan_commands(model_name: str, isl: int, requests: int, par: ParallelConfig, page_size: int, backend: str = "NVLINK", mem: str = "VRAM",
                  op: str = "WRITE", src_dev: int = 0, dst_dev: int = 1, iters: int = 200, extra: str = "", kvcache_quant: str = "") -> List[str]:
    """One nixlbench line per access granularity of a KV transfer: block-sized descriptors batched
    per request (what a paged engine posts) and one contiguous layer-sized copy (the upper bound)."""
    rep = kvcache_report(model_name, isl, requests, par, page_size, kvcache_quant)
    block = rep["io_size"]
    blocks_per_request = -(-isl // page_size) * rep["cache_tensors_per_gpu"]
    cmds = []
    base = f"{NIXLBENCH} --backend {backend} --op {op} --mem {mem} --src-dev {src_dev} --dst-dev {dst_dev} --iters {iters} --warmup {max(10, iters // 10)}"
    cmds.append(f"{base} --min {block} --max {block} --batch {min(_pow2_floor(blocks_per_request), 4096)} {extra}".strip())
    layer_bytes = _pow2_floor(rep["kv_bytes_per_request_per_gpu"] // max(1, rep["cache_tensors_per_gpu"]))
    cmds.append(f"{base} --min {layer_bytes} --max {layer_bytes} --batch {min(rep['cache_tensors_per_gpu'], 256)} {extra}".strip())
    return cmds


def profile(cmds: List[str], timeout: int = 600) -> List[dict]:
    out = []
    for c in cmds:
        r = subprocess.run(shlex.split(c), capture_output=True, text=True, timeout=timeout)
        out.append({"cmd": c, "rc": r.returncode, "stdout": r.stdout[-4000:], "stderr": r.stderr[-2000:]})
    return out


def model_names() -> List[str]:
    return sorted(MODELS)

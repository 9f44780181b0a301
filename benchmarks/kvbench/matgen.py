"""Workload generator: traffic matrices of a disaggregated prefill -> decode deployment.

Same model as the reference's benchmark/kvbench/test/inference_workload_matgen.py: user requests
with normally distributed prompt lengths are packed into batches, each batch is prefilled by one
prefill worker (``tp x cp`` ranks) and its KV cache is sent to the decode worker coupled with it;
the matrix cell [prefill rank][decode rank] is the bytes that pair moves.  The prefill compute
time estimate becomes the pattern's ``sleep_before_launch_sec``."""
from __future__ import annotations

import os
import random
from dataclasses import dataclass
from typing import List, Sequence

from nixl_b200.models import ParallelConfig, get_model

from .traffic import save_matrix

# Dense bf16 throughput one B200 sustains through cuBLAS under its power cap (the reference assumes 36 TFLOP/s of an H100).
DEFAULT_FLOPS_PER_GPU = 1.4e15


@dataclass
class TaskConfig:
    isl_mean: int = 16000
    isl_scale: int = 10000
    min_isl: int = 1000
    max_isl: int = 128000
    batch_size: int = 1
    max_batch_mem: float = 100e9


@dataclass
class Batch:
    isls: List[int]

    @property
    def total_isl(self) -> int:
        return sum(self.isls)


@dataclass
class TransferMatrix:
    matrix: List[List[int]]
    compute_time: float
    isl: int


def sample_isl(rng: random.Random, task: TaskConfig) -> int:
    return int(min(max(task.min_isl, rng.gauss(task.isl_mean, task.isl_scale)), task.max_isl))


def kv_bytes_total(model_name: str, isl: int) -> int:
    """KV bytes of one request on an unsharded model."""
    return get_model(model_name).kv_bytes_per_gpu(isl, ParallelConfig())


def gen_batches(num_requests: int, task: TaskConfig, model_name: str, seed: int = 0) -> List[Batch]:
    rng = random.Random(seed)
    batches, cur, mem = [], [], 0
    for _ in range(num_requests):
        isl = sample_isl(rng, task)
        cur.append(isl)
        mem += kv_bytes_total(model_name, isl)
        if mem > task.max_batch_mem or len(cur) >= task.batch_size:
            batches.append(Batch(cur))
            cur, mem = [], 0
    if cur:
        batches.append(Batch(cur))
    return batches


def gen_matrix(batch: Batch, world_size: int, prefill_worker: Sequence[int], decode_worker: Sequence[int], model_name: str,
               prefill: ParallelConfig, decode: ParallelConfig) -> List[List[int]]:
    kv = sum(kv_bytes_total(model_name, isl) for isl in batch.isls)
    slice_bytes = kv / prefill.tp / prefill.pp / prefill.cp
    peers = decode.tp / (prefill.tp * prefill.cp)
    if peers != int(peers) or peers < 1:
        raise ValueError("prefill tp * cp must divide decode tp")
    peers = int(peers)
    if len(prefill_worker) * peers != len(decode_worker):
        raise ValueError("worker rank lists do not match the parallel configurations")
    mat = [[0] * world_size for _ in range(world_size)]
    dst = iter(decode_worker)
    for src in prefill_worker:
        for _ in range(peers):
            mat[src][next(dst)] = int(slice_bytes / peers)
    return mat


def estimate_compute_time(batch: Batch, model_name: str, worker: ParallelConfig, flops_per_gpu: float = DEFAULT_FLOPS_PER_GPU) -> float:
    """Prefill seconds of a batch: attention O(S^2 H) plus projections and a 4H MLP, O(S H^2), per layer, divided over TP."""
    cfg = get_model(model_name).cfg
    h, layers = cfg.hidden, cfg.num_layers
    flops = 0.0
    for s in batch.isls:
        attention = 4.0 * s * s * h
        linear = 2.0 * s * (4 * h * h + 8 * h * h)
        flops += layers * (attention + linear)
    return flops / (flops_per_gpu * worker.tp * worker.cp)


def generate(model_name: str, num_requests: int, task: TaskConfig, prefill: ParallelConfig, decode: ParallelConfig, world_size: int,
             seed: int = 0, flops_per_gpu: float = DEFAULT_FLOPS_PER_GPU) -> List[TransferMatrix]:
    """Splits ``world_size`` ranks into coupled (prefill worker, decode worker) groups and walks the batches round-robin."""
    p_ranks, d_ranks = prefill.tp * prefill.cp, decode.tp * decode.cp
    group = p_ranks + d_ranks
    if world_size < group or world_size % group:
        raise ValueError(f"world size must be a multiple of {group} (prefill {p_ranks} + decode {d_ranks} ranks)")
    couples = []
    for base in range(0, world_size, group):
        couples.append((list(range(base, base + p_ranks)), list(range(base + p_ranks, base + group))))
    out = []
    for i, batch in enumerate(gen_batches(num_requests, task, model_name, seed)):
        pw, dw = couples[i % len(couples)]
        out.append(TransferMatrix(gen_matrix(batch, world_size, pw, dw, model_name, prefill, decode),
                                  estimate_compute_time(batch, model_name, prefill, flops_per_gpu), batch.total_isl))
    return out


def write_workload(matrices: Sequence[TransferMatrix], out_dir: str, mem_type: str = "cuda", xfer_op: str = "WRITE") -> str:
    """Writes matrix_<i>.txt files and the sequential-ct-perftest YAML that references them; returns the YAML path."""
    import yaml

    os.makedirs(os.path.join(out_dir, "matrices"), exist_ok=True)
    patterns = []
    for i, m in enumerate(matrices):
        path = os.path.join(out_dir, "matrices", f"matrix_{i}.txt")
        save_matrix(path, m.matrix)
        patterns.append({"matrix_file": os.path.join("matrices", f"matrix_{i}.txt"), "metadata": {"isl": m.isl},
                         "sleep_before_launch_sec": m.compute_time, "mem_type": mem_type, "xfer_op": xfer_op})
    cfg = os.path.join(out_dir, "workload.yaml")
    with open(cfg, "w") as f:
        yaml.safe_dump({"traffic_patterns": patterns}, f, sort_keys=False)
    return cfg

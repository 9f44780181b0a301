"""Traffic patterns: "rank i sends matrix[i][j] bytes to rank j".

Matrix files hold one row per line, cells separated by blanks, each cell a byte count with an
optional K / M / G suffix (powers of 1024), as in the reference's ct-perftest documentation
(benchmark/kvbench/docs/ct-perftest.md)."""
from __future__ import annotations

import itertools
import re
from dataclasses import dataclass, field
from typing import Iterable, List, Optional

_UNITS = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30, "T": 1 << 40}


_SIZE_RE = re.compile(r"^(\d+(?:\.\d+)?)\s*([KMGT]?)(?:I?B)?$", re.IGNORECASE)


def parse_size(cell: str) -> int:
    """``"4096"``, ``"5K"``, ``"1.5M"``, ``"2GB"`` -> bytes (units are powers of 1024)."""
    m = _SIZE_RE.match(cell.strip())
    if not m:
        raise ValueError(f"not a size: {cell!r}")
    return int(float(m.group(1)) * _UNITS.get(m.group(2).upper(), 1))


def format_size(n: int) -> str:
    for unit in ("G", "M", "K"):
        if n and n % _UNITS[unit] == 0:
            return f"{n // _UNITS[unit]}{unit}"
    return str(n)


def load_matrix(path: str) -> List[List[int]]:
    rows = []
    with open(path) as f:
        for line in f:
            line = line.split("#", 1)[0].strip()
            if line:
                rows.append([parse_size(c) for c in line.split()])
    if not rows or any(len(r) != len(rows) for r in rows):
        raise ValueError(f"{path}: the matrix must be square")
    return rows


def save_matrix(path: str, matrix: Iterable[Iterable[int]]) -> None:
    with open(path, "w") as f:
        for row in matrix:
            f.write(" ".join(format_size(int(c)) for c in row) + "\n")


_ids = itertools.count()


@dataclass
class TrafficPattern:
    matrix: List[List[int]]
    mem_type: str = "cuda"            # cuda / vram or cpu / dram
    xfer_op: str = "WRITE"            # WRITE: senders push; READ: receivers pull
    shards: int = 1                   # every message is split into this many descriptors
    sleep_before_launch_sec: float = 0.0
    sleep_after_launch_sec: float = 0.0
    metadata: dict = field(default_factory=dict)
    id: int = field(default_factory=lambda: next(_ids))

    def __post_init__(self):
        if self.xfer_op not in ("WRITE", "READ"):
            raise ValueError("xfer_op must be WRITE or READ")
        if self.mem_type.lower() not in ("cuda", "vram", "cpu", "dram"):
            raise ValueError("mem_type must be cuda/vram or cpu/dram")
        n = len(self.matrix)
        if any(len(r) != n for r in self.matrix):
            raise ValueError("matrix must be square")

    @property
    def world_size(self) -> int:
        return len(self.matrix)

    @property
    def on_gpu(self) -> bool:
        return self.mem_type.lower() in ("cuda", "vram")

    def senders(self) -> List[int]:
        return [i for i, row in enumerate(self.matrix) if any(c > 0 for c in row)]

    def receivers(self, from_ranks: Optional[Iterable[int]] = None) -> List[int]:
        rows = range(self.world_size) if from_ranks is None else list(from_ranks)
        return sorted({j for i in rows for j, c in enumerate(self.matrix[i]) if c > 0})

    def ranks(self) -> List[int]:
        return sorted(set(self.senders()) | set(self.receivers()))

    def total_bytes(self) -> int:
        return sum(sum(r) for r in self.matrix)

    def send_bytes(self, rank: int) -> int:
        return sum(self.matrix[rank])

    def recv_bytes(self, rank: int) -> int:
        return sum(row[rank] for row in self.matrix)


def pattern_from_dict(d: dict, base_dir: str = ".") -> TrafficPattern:
    """One ``traffic_pattern`` entry of a YAML configuration."""
    import os

    if "matrix" in d:
        matrix = [[parse_size(str(c)) for c in row] for row in d["matrix"]]
    else:
        path = d["matrix_file"]
        matrix = load_matrix(path if os.path.isabs(path) else os.path.join(base_dir, path))
    return TrafficPattern(
        matrix=matrix,
        mem_type=d.get("mem_type", "cuda"),
        xfer_op=d.get("xfer_op", "WRITE"),
        shards=int(d.get("shards", 1)),
        sleep_before_launch_sec=float(d.get("sleep_before_launch_sec", 0) or 0),
        sleep_after_launch_sec=float(d.get("sleep_after_launch_sec", 0) or 0),
        metadata=dict(d.get("metadata", {}) or {}),
    )

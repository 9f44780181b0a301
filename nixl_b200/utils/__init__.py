"""Helpers that are not part of the agent API.

``measured_peaks()``: the measured copy bandwidth and GEMM throughput of the machine the benchmarks ran on
(``MEASURED_PEAKS.json`` beside the package, when present), for roofline fractions.
``device_timed()``: median CUDA-event time of a callable, with warm-up and an optional L2 flush between runs.
The raw-memory helpers of the reference's ``nixl._utils`` (``malloc_passthru`` and friends) are re-exported here."""
import json
import os
from typing import Callable, Optional

from .._utils import ba_buf, free_passthru, malloc_passthru, verify_transfer  # noqa: F401

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def measured_peaks(path: Optional[str] = None) -> dict:
    """``{"hbm_gbs": ..., "bf16_tflops": ..., ...}`` from MEASURED_PEAKS.json, or ``{}`` when there is none."""
    try:
        with open(path or os.path.join(_ROOT, "MEASURED_PEAKS.json")) as f:
            data = json.load(f)
        return data if isinstance(data, dict) else {}
    except (OSError, ValueError):
        return {}


def device_timed(fn: Callable[[], None], iters: int = 10, warmup: int = 3, flush=None) -> float:
    """Median device time of ``fn()`` in microseconds (CUDA events on the current stream).  ``flush``: a tensor
    larger than L2 that is written between runs so that no run finds the previous one's data on chip."""
    import torch

    times = []
    for i in range(warmup + iters):
        if flush is not None:
            flush.add_(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(e0.elapsed_time(e1) * 1e3)
    times.sort()
    return times[len(times) // 2]


def pci_topology(root: str = "") -> dict:
    """The host's GPUs and network devices as the PCI sysfs tree shows them, and per GPU the network devices nearest to
    it (bridges through the closest common ancestor; another root complex and another NUMA node cost 100 each).
    ``root`` defaults to ``$NIXL_SYSFS_PCI_ROOT`` or ``/sys/bus/pci/devices``.  ``python -m nixl_b200.utils`` prints it.
    The TCP backend uses the same order for the addresses it publishes when ``device_id`` names a GPU."""
    from .. import _bindings

    return _bindings.pci_topology(root)

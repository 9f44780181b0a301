"""Fused GPU operations of the library (hand-written sm_100a kernels behind a C ABI)."""
from .grouped_gemm import grouped_gemm_fp8, quantize_weights, reference_grouped_gemm  # noqa: F401
from .kv_transfer import KVLayout, KVTransfer, reference_kv_transfer  # noqa: F401


def smoke_kernels() -> None:
    """Tiny run of every fused kernel on cuda:0 (used by the repository's smoke entry point)."""
    from . import _smoke

    _smoke.run()

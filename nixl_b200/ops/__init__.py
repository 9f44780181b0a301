"""Fused GPU operations of the library (hand-written sm_100a kernels behind a C ABI), and the descriptor path for KV
blocks that reaches peers on other hosts."""
from .grouped_gemm import (  # noqa: F401
    from_ue8m0,
    grouped_gemm_fp8,
    grouped_gemm_mxfp8,
    quantize_weights,
    quantize_weights_ue8m0,
    reference_grouped_gemm,
    to_ue8m0,
)
from .kv_blocks import KVBlockTransfer, describe_blocks  # noqa: F401
from .kv_transfer import KVLayout, KVTransfer, reference_kv_transfer  # noqa: F401


def smoke_kernels() -> None:
    """Tiny run of every fused kernel on cuda:0 (used by the repository's smoke entry point)."""
    from . import _smoke

    _smoke.run()

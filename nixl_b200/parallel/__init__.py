"""Multi-GPU building blocks: expert-parallel dispatch/combine (``ep.Buffer``)."""
from .ep import Buffer, EPHandle, EventOverlap, dequant_fp8, dequant_ue8m0, per_token_cast_to_fp8  # noqa: F401

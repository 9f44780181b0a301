"""Reference model of the logarithmic 10-bit row format that combine can use on the wire.

The kernel side is ``logfmtEncode16`` / ``logfmtDecodeAdd16`` in ``csrc/src/kernels/ep_kernels.cu``
(role of the reference's LogFMT-10 codec, examples/device/ep/csrc/kernels/nixl_ep_ll.cu:459-616).
Per group of 128 channels the magnitudes are coded on a grid of 510 logarithmic steps between the
group's smallest non-zero and largest magnitude (at most 32 octaves below the largest); code 0 is an
exact zero and one more bit holds the sign.  This module states the same arithmetic in plain
PyTorch: it is the oracle of the kernel's tests and lets a model check offline what the format
does to its activations.
"""
from __future__ import annotations

import torch

GROUP = 128
STEPS = 510.0
MAX_OCTAVES = 32.0


def logfmt10_codes(x: torch.Tensor):
    """Encode ``x [..., H]`` (H % 128 == 0).  Returns ``(codes int32 [..., H] in 0..511,
    negative bool [..., H], log_min float32 [..., H // 128], step float32 [..., H // 128])``."""
    if x.shape[-1] % GROUP:
        raise ValueError("the last dimension must be a multiple of 128")
    xf = x.float()
    g = xf.reshape(*xf.shape[:-1], -1, GROUP)
    mag = g.abs()
    amax = mag.amax(dim=-1).clamp(max=3.0e38)
    amin = torch.where(mag > 0, mag, torch.full_like(mag, float("inf"))).amin(dim=-1)
    log_amax = torch.where(amax > 0, torch.log2(amax.clamp(min=1e-45)), torch.zeros_like(amax))
    log_amin = torch.where(amin <= amax, torch.maximum(torch.log2(amin), log_amax - MAX_OCTAVES), log_amax)
    step = (log_amax - log_amin) / STEPS
    pos = step > 0
    step_inv = torch.where(pos, 1.0 / step.clamp(min=1e-38), torch.zeros_like(step))
    # A value moves to the upper neighbour once it passes the arithmetic midpoint of the two.
    bias = torch.where(pos, 1.0 - torch.log2(0.5 + 0.5 * torch.exp2(step)) * step_inv, torch.full_like(step, 0.5))
    q = (torch.log2(mag.clamp(min=1e-45)) - log_amin[..., None]) * step_inv[..., None] + bias[..., None]
    codes = torch.where(mag > 0, 1 + q.clamp(0.0, STEPS).floor().to(torch.int32), torch.zeros_like(q, dtype=torch.int32))
    return codes.reshape(x.shape), (g < 0).reshape(x.shape), log_amin, step


def logfmt10_decode(codes: torch.Tensor, negative: torch.Tensor, log_min: torch.Tensor, step: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`logfmt10_codes`, in float32."""
    c = codes.reshape(*codes.shape[:-1], -1, GROUP)
    v = torch.exp2((c - 1).float() * step[..., None] + log_min[..., None])
    v = torch.where(c > 0, v, torch.zeros_like(v))
    v = torch.where(negative.reshape(c.shape), -v, v)
    return v.reshape(codes.shape)


def logfmt10_roundtrip(x: torch.Tensor) -> torch.Tensor:
    """What the receiver sees for ``x`` (float32)."""
    return logfmt10_decode(*logfmt10_codes(x))


def logfmt10_row_bytes(hidden: int) -> int:
    """Bytes of one row on the wire: ten bits per channel plus two floats per group."""
    return hidden * 10 // 8 + (hidden // GROUP) * 8

"""Reference model of the logarithmic 10-bit row format that combine can use on the wire.

The kernel side is ``logfmtEncode16`` / ``logfmtDecodeAdd16`` in ``csrc/src/kernels/ep_kernels.cu``
(role of the reference's LogFMT-10 codec, examples/device/ep/csrc/kernels/nixl_ep_ll.cu:459-616).
The 15-bit magnitude pattern of a bf16 (exponent and mantissa read as one integer) is a
piecewise-linear logarithm of the value.  Per group of 128 channels the patterns between the
smallest non-zero one (at most 32 octaves = 4096 patterns below the largest) and the largest are
mapped onto 510 steps; code 0 is an exact zero and one more bit holds the sign.  A group spanning at
most 510 patterns (four octaves) is coded exactly.  This module states the same arithmetic in
plain PyTorch, bit for bit: it is the oracle of the kernel's tests and lets a model check offline
what the format does to its activations.
"""
from __future__ import annotations

import torch

GROUP = 128
STEPS = 510
MAX_PATTERNS = 32 * 128
_LARGEST_FINITE = 0x7F7F


def logfmt10_codes(x: torch.Tensor):
    """Encode ``x [..., H]`` (H % 128 == 0; converted to bf16 first).  Returns ``(codes int32
    [..., H] in 0..511, negative bool [..., H], min_pattern int32 [..., H // 128],
    patterns_per_step float32 [..., H // 128])``."""
    if x.shape[-1] % GROUP:
        raise ValueError("the last dimension must be a multiple of 128")
    bits = x.to(torch.bfloat16).contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    negative = (bits >> 15).bool()
    pat = (bits & 0x7FFF).clamp(max=_LARGEST_FINITE).reshape(*x.shape[:-1], -1, GROUP)
    pmax = pat.amax(dim=-1)
    pmin = torch.where(pat > 0, pat, torch.full_like(pat, 0x7FFF)).amin(dim=-1)
    pmin = torch.where(pmax > 0, pmin, torch.zeros_like(pmin))
    pmin = torch.maximum(pmin, pmax - MAX_PATTERNS)
    span = pmax - pmin
    wide = span > STEPS
    spanf = span.clamp(min=1).float()
    scale = torch.where(wide, torch.tensor(float(STEPS)) / spanf, torch.ones_like(spanf))
    per_step = torch.where(wide, spanf / float(STEPS), torch.ones_like(spanf))
    above = (pat - pmin[..., None]).clamp(min=0).float()
    q = torch.round(above * scale[..., None]).to(torch.int32).clamp(max=STEPS)  # round half to even, as cvt.rni
    codes = torch.where(pat > 0, 1 + q, torch.zeros_like(q))
    return codes.reshape(x.shape), negative, pmin, per_step


def logfmt10_decode(codes: torch.Tensor, negative: torch.Tensor, min_pattern: torch.Tensor, per_step: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`logfmt10_codes`, in float32."""
    c = codes.reshape(*codes.shape[:-1], -1, GROUP)
    pat = min_pattern[..., None] + torch.round((c - 1).float() * per_step[..., None]).to(torch.int32)
    pat = torch.where(c > 0, pat, torch.zeros_like(pat)).reshape(codes.shape)
    word = (pat << 16) | (negative.to(torch.int32) << 31)
    word = torch.where(codes > 0, word, torch.zeros_like(word))
    return word.view(torch.float32)


def logfmt10_roundtrip(x: torch.Tensor) -> torch.Tensor:
    """What the receiver sees for ``x`` (float32)."""
    return logfmt10_decode(*logfmt10_codes(x))


def logfmt10_row_bytes(hidden: int) -> int:
    """Bytes of one row on the wire: ten bits per channel plus eight bytes per group."""
    return hidden * 10 // 8 + (hidden // GROUP) * 8

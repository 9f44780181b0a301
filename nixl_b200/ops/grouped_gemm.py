"""Grouped expert GEMM (fp8, 1x128 / 128x128 block scales) on tcgen05 tensor cores.

Wraps ``csrc/src/kernels/grouped_gemm_fp8.cu``.  Rows of group ``g`` are
``row_start[g] : row_start[g] + row_count[g]`` of ``a``; both index tensors stay on the device so
the GEMM can be queued right behind an EP dispatch.  ``fused_with`` accepts the handle of such a
dispatch: the kernel then waits, tile by tile, for the arrival flags of the sources whose rows the
tile contains instead of waiting for the whole all-to-all.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib


class _Params(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p), ("scale_a", ctypes.c_void_p), ("w", ctypes.c_void_p), ("scale_w", ctypes.c_void_p), ("d", ctypes.c_void_p),
        ("row_start", ctypes.c_void_p), ("row_count", ctypes.c_void_p),
        ("groups", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32), ("a_rows", ctypes.c_int32),
        ("grid", ctypes.c_int32), ("ranks", ctypes.c_int32), ("experts_total", ctypes.c_int32), ("expert_base", ctypes.c_int32),
        ("status", ctypes.c_void_p), ("disp_flag", ctypes.c_void_p), ("counts", ctypes.c_void_p),
        ("epoch", ctypes.c_uint64), ("timeout_ns", ctypes.c_uint64),
        ("counts_flag", ctypes.c_void_p), ("rows_per_expert", ctypes.c_int32), ("tile_mode", ctypes.c_int32),
    ]


def quantize_weights(w: torch.Tensor):
    """bf16/fp32 ``[G, N, K]`` -> (e4m3 ``[G, N, K]``, fp32 scales ``[G, N/128, K/128]``), 128x128 blocks."""
    G, N, K = w.shape
    blocks = w.float().view(G, N // 128, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(2, 4)).clamp(min=1e-4)
    scale = amax / 448.0
    q = (blocks / scale[:, :, None, :, None]).to(torch.float8_e4m3fn).view(G, N, K)
    return q.contiguous(), scale.contiguous()


def to_ue8m0(scale: torch.Tensor) -> torch.Tensor:
    """Power-of-two fp32 scales -> biased exponent bytes (uint8, same shape)."""
    bits = scale.contiguous().view(torch.int32)
    if bool(((bits & 0x7FFFFF) != 0).any()):
        raise ValueError("scales are not powers of two")
    return ((bits >> 23) & 0xFF).to(torch.uint8)


def from_ue8m0(exp: torch.Tensor) -> torch.Tensor:
    """Biased exponent bytes -> fp32 scales."""
    return torch.ldexp(torch.ones(exp.shape, dtype=torch.float32, device=exp.device), exp.to(torch.int32) - 127)


def quantize_weights_ue8m0(w: torch.Tensor):
    """bf16/fp32 ``[G, N, K]`` -> (e4m3 ``[G, N, K]``, uint8 exponents ``[G, N/128, K/128]``): 128x128 blocks whose
    scale is the smallest power of two that keeps the block inside e4m3's range."""
    G, N, K = w.shape
    blocks = w.float().view(G, N // 128, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(2, 4)).clamp(min=1e-4)
    ex = torch.ceil(torch.log2(amax / 448.0))
    q = (blocks * torch.exp2(-ex)[:, :, None, :, None]).to(torch.float8_e4m3fn).view(G, N, K)
    return q.contiguous(), (ex.to(torch.int32) + 127).to(torch.uint8).contiguous()


def grouped_gemm_mxfp8(a: torch.Tensor, scale_a: torch.Tensor, w: torch.Tensor, scale_w: torch.Tensor, row_start: torch.Tensor,
                       row_count: torch.Tensor, out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None, grid: int = 0) -> torch.Tensor:
    """Grouped GEMM with power-of-two block scales applied inside the tensor core (block-scaled MMA),
    256 x 256 tiles on CTA pairs: no per-step promotion, so it runs well above ``grouped_gemm_fp8``.

    ``scale_a``: biased exponents, uint8 ``[rows, K/128]`` or the int32 ``[rows, K/512]`` packing that
    ``Buffer.dispatch(..., use_ue8m0=True)`` delivers; ``scale_w``: uint8 ``[G, N/128, K/128]``
    (``quantize_weights_ue8m0``).  ``K % 512 == 0`` and ``N % 256 == 0``."""
    rows, K = a.shape
    G, N, K2 = w.shape
    if K != K2 or K % 512 or N % 256:
        raise ValueError("K must be a multiple of 512, N of 256, and a and w must agree on K")
    if a.dtype != torch.float8_e4m3fn or w.dtype != torch.float8_e4m3fn:
        raise TypeError("a and w must be float8_e4m3fn")
    if scale_a.dtype == torch.int32:
        scale_a = scale_a.contiguous().view(torch.uint8)
    if scale_a.dtype != torch.uint8 or scale_w.dtype != torch.uint8:
        raise TypeError("scales must be UE8M0 exponent bytes")
    if scale_a.numel() != rows * (K // 128) or tuple(scale_w.shape) != (G, N // 128, K // 128):
        raise ValueError("scale shapes do not match")
    if row_start.numel() == G + 1:
        row_start = row_start[:G]
    for t in (a, scale_a, w, scale_w, row_start, row_count):
        if not t.is_contiguous():
            raise ValueError("inputs must be contiguous")
    dev = a.device
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)
        if status is None:
            status = torch.zeros(1, dtype=torch.int32, device=dev)
    p = _Params()
    p.a, p.scale_a, p.w, p.scale_w, p.d = a.data_ptr(), scale_a.data_ptr(), w.data_ptr(), scale_w.data_ptr(), out.data_ptr()
    p.row_start, p.row_count = row_start.data_ptr(), row_count.data_ptr()
    p.groups, p.N, p.K, p.a_rows, p.grid = G, N, K, rows, grid
    p.tile_mode = 3
    p.status = status.data_ptr()
    fn = _lib.lib().nixl_grouped_gemm_fp8_launch
    fn.argtypes = [ctypes.POINTER(_Params), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    with torch.cuda.device(dev):
        _lib.check(fn(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)), "nixl_grouped_gemm_fp8_launch (block-scaled)")
    out._nixl_status = status
    return out


def grouped_gemm_fp8(
    a: torch.Tensor,
    scale_a: torch.Tensor,
    w: torch.Tensor,
    scale_w: torch.Tensor,
    row_start: torch.Tensor,
    row_count: torch.Tensor,
    out: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
    fused_with=None,
    grid: int = 0,
    overlapped: bool = False,
    rows_per_expert: int = 0,
    tile_mode: int = 0,
) -> torch.Tensor:
    """``out[rows of g] = dequant(a[rows]) @ dequant(w[g]).T`` in bf16.

    ``a``: e4m3 ``[rows, K]``; ``scale_a``: fp32 ``[rows, K/128]``; ``w``: e4m3 ``[G, N, K]``;
    ``scale_w``: fp32 ``[G, N/128, K/128]``; ``row_start`` / ``row_count``: int32 ``[G]`` on the device.
    ``fused_with``: ``(buffer, handle)`` of the EP dispatch that is filling ``a`` (optional).
    ``overlapped``: that dispatch was launched on another stream and may still be running; the
    kernel then waits for the count exchange itself (``rows_per_expert`` names the layout) and
    ``grid`` should leave the dispatch's CTAs free (see ``Buffer.dispatch_gemm``).
    ``tile_mode``: 0 lets the library choose, 1 forces 128 x 128 tiles on single CTAs, 2 forces
    256 x 256 tiles on CTA pairs (``N % 256 == 0``)."""
    rows, K = a.shape
    G, N, K2 = w.shape
    if K != K2 or K % 128 or N % 128:
        raise ValueError("K and N must be multiples of 128 and agree between a and w")
    if a.dtype != torch.float8_e4m3fn or w.dtype != torch.float8_e4m3fn:
        raise TypeError("a and w must be float8_e4m3fn")
    if scale_a.shape != (rows, K // 128) or scale_w.shape != (G, N // 128, K // 128):
        raise ValueError("scale shapes do not match")
    if row_start.numel() == G + 1:
        row_start = row_start[:G]
    for t in (a, scale_a, w, scale_w, row_start, row_count):
        if not t.is_contiguous():
            raise ValueError("inputs must be contiguous")
    if row_start.dtype != torch.int32 or row_count.dtype != torch.int32:
        raise TypeError("row_start / row_count must be int32")
    dev = a.device
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)
        if status is None:
            status = torch.zeros(1, dtype=torch.int32, device=dev)
    p = _Params()
    p.a, p.scale_a, p.w, p.scale_w, p.d = a.data_ptr(), scale_a.data_ptr(), w.data_ptr(), scale_w.data_ptr(), out.data_ptr()
    p.row_start, p.row_count = row_start.data_ptr(), row_count.data_ptr()
    p.groups, p.N, p.K, p.a_rows, p.grid = G, N, K, rows, grid
    p.tile_mode = tile_mode
    p.status = status.data_ptr()
    if fused_with is not None:
        buf, handle = fused_with
        lay = buf._layout(handle.parity)
        base = buf.buffer.data_ptr()
        p.disp_flag = base + lay.off_disp_flag
        p.counts = base + lay.off_counts
        p.ranks, p.experts_total, p.expert_base = buf.num_ranks, buf.num_experts, buf.rank * buf.local_experts
        p.epoch, p.timeout_ns = handle.epoch, buf.timeout_ns
        if overlapped:
            # The dispatch runs on another stream right now: the kernel derives the row ranges itself.
            p.counts_flag = base + lay.off_counts_flag
            p.rows_per_expert = rows_per_expert
    fn = _lib.lib().nixl_grouped_gemm_fp8_launch
    fn.argtypes = [ctypes.POINTER(_Params), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    with torch.cuda.device(dev):
        _lib.check(fn(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)), "nixl_grouped_gemm_fp8_launch")
    out._nixl_status = status  # keeps the status word alive with the result
    return out


def reference_grouped_gemm(a, scale_a, w, scale_w, row_start, row_count):
    """fp32 PyTorch statement of the same product (test oracle)."""
    rows, K = a.shape
    G, N, _ = w.shape
    af = (a.float().view(rows, K // 128, 128) * scale_a.unsqueeze(2)).view(rows, K)
    wf = (w.float().view(G, N // 128, 128, K // 128, 128) * scale_w[:, :, None, :, None]).view(G, N, K)
    out = torch.zeros(rows, N, dtype=torch.float32, device=a.device)
    starts, counts = row_start.tolist(), row_count.tolist()
    for g in range(G):
        s, c = starts[g], counts[g]
        if c:
            out[s : s + c] = af[s : s + c] @ wf[g].t()
    return out

"""Fused paged-KV-cache transfer (prefill GPU -> decode GPU) on top of the agent.

``KVTransfer`` wires the kernel of ``csrc/src/kernels/kv_xfer.cu`` to registered memory: the
sender's cache tensors and the receiver's cache tensors become device-side memory views
(``nixl_agent.prep_mem_view``), and one launch gathers blocks by the sender's block table,
regroups KV heads for the receiver's tensor-parallel degree, optionally casts bf16 to fp8 e4m3
and scatters by the receiver's block table, signalling completion in the receiver's memory.

The reference moves KV caches as descriptor lists (its kvbench tool); the descriptor path
remains available through ``nixl_agent.initialize_xfer`` and is the baseline in
``benchmarks/kvbench/kv_transfer.py``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib


class _Params(ctypes.Structure):
    _fields_ = [
        ("src_view", ctypes.c_void_p),
        ("dst_view", ctypes.c_void_p),
        ("src_blocks", ctypes.c_void_p),
        ("dst_blocks", ctypes.c_void_p),
        ("n_pairs", ctypes.c_int32),
        ("n_tensors", ctypes.c_int32),
        ("tokens", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("head_bytes", ctypes.c_int32),
        ("cast_fp8", ctypes.c_int32),
        ("src_block_stride", ctypes.c_int64),
        ("src_token_stride", ctypes.c_int64),
        ("src_head_stride", ctypes.c_int64),
        ("dst_block_stride", ctypes.c_int64),
        ("dst_token_stride", ctypes.c_int64),
        ("dst_head_stride", ctypes.c_int64),
        ("dst_head_offset", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("done_signal", ctypes.c_void_p),
        ("done_value", ctypes.c_uint64),
        ("host_flag", ctypes.c_void_p),
        ("host_seq", ctypes.c_uint64),
        ("done_counter", ctypes.c_void_p),
        ("grid", ctypes.c_int32),
        ("status", ctypes.c_void_p),
    ]


@dataclass(frozen=True)
class KVLayout:
    """Shape of one cache tensor: ``[blocks, tokens, heads, head_dim]`` ("NHD") or
    ``[blocks, heads, tokens, head_dim]`` ("HND"); ``elem_bytes`` 2 for bf16, 1 for fp8."""

    tokens: int
    heads: int
    head_dim: int
    order: str = "NHD"
    elem_bytes: int = 2

    def strides(self) -> tuple[int, int, int]:
        row = self.head_dim * self.elem_bytes
        if self.order == "NHD":
            return (self.tokens * self.heads * row, self.heads * row, row)
        if self.order == "HND":
            return (self.tokens * self.heads * row, row, self.tokens * row)
        raise ValueError("order must be 'NHD' or 'HND'")

    @property
    def block_bytes(self) -> int:
        return self.tokens * self.heads * self.head_dim * self.elem_bytes


class KVTransfer:
    """A prepared sender->receiver KV path.

    Args:
        agent: the sender's ``nixl_agent`` (its backend must be the NVLink one).
        src_tensors: the sender's cache tensors, one per (layer, K/V), already registered.
        src_layout: layout of each sender tensor (bf16).
        remote_agent: receiver's agent name (metadata already loaded).
        remote_tensors: ``(addr, nbytes, device)`` of the receiver's cache tensors, same order.
        dst_layout: receiver layout; ``heads`` is the receiver's per-rank KV head count.
        dst_head_offset: head slot at the receiver where the sender's first head lands.
        cast_fp8: write fp8 e4m3 (receiver layout must have ``elem_bytes == 1``).
        scale: multiplier applied before the cast.
    """

    def __init__(
        self,
        agent,
        src_tensors: Sequence[torch.Tensor],
        src_layout: KVLayout,
        remote_agent: str,
        remote_tensors: Sequence[tuple[int, int, int]],
        dst_layout: KVLayout,
        dst_head_offset: int = 0,
        cast_fp8: bool = False,
        scale: float = 1.0,
    ):
        if len(src_tensors) != len(remote_tensors):
            raise ValueError("sender and receiver must expose the same number of cache tensors")
        if src_layout.tokens != dst_layout.tokens or src_layout.head_dim != dst_layout.head_dim:
            raise ValueError("block size and head_dim must agree on both sides")
        if dst_head_offset + src_layout.heads > dst_layout.heads:
            raise ValueError("sender heads do not fit at that head offset of the receiver")
        if src_layout.elem_bytes != 2:
            raise ValueError("the sender cache must be bf16")
        if cast_fp8 != (dst_layout.elem_bytes == 1):
            raise ValueError("cast_fp8 requires a 1-byte receiver layout (and only then)")
        self.agent = agent
        self.device = src_tensors[0].device
        self.src_layout, self.dst_layout = src_layout, dst_layout
        self.n_tensors = len(src_tensors)
        with torch.cuda.device(self.device):
            self.src_view = agent.prep_mem_view([(t.data_ptr(), t.numel() * t.element_size(), t.get_device()) for t in src_tensors], "VRAM")
            self.dst_view = agent.prep_mem_view(
                agent.get_remote_descs([(a, n, d, remote_agent) for a, n, d in remote_tensors], "VRAM")
            )
        # Scratch: the "last CTA" counter (zero between launches) and a pinned completion word.
        self._counter = torch.zeros(64, dtype=torch.int32, device=self.device)
        self._flag = torch.zeros(2, dtype=torch.int64).pin_memory()  # completion word, then the out-of-range word
        self._seq = 0
        self._p = _Params()
        sb, st, sh = src_layout.strides()
        db, dt, dh = dst_layout.strides()
        p = self._p
        p.src_view, p.dst_view = self.src_view, self.dst_view
        p.n_tensors = self.n_tensors
        p.tokens, p.heads, p.head_bytes = src_layout.tokens, src_layout.heads, src_layout.head_dim * 2
        p.cast_fp8 = 1 if cast_fp8 else 0
        p.src_block_stride, p.src_token_stride, p.src_head_stride = sb, st, sh
        p.dst_block_stride, p.dst_token_stride, p.dst_head_stride = db, dt, dh
        p.dst_head_offset = dst_head_offset
        p.scale = scale
        p.done_counter = self._counter.data_ptr()
        p.host_flag = self._flag.data_ptr()
        p.status = self._flag.data_ptr() + 8
        p.grid = 0
        self._launch = _lib.lib().nixl_kv_xfer_launch
        self._launch.argtypes = [ctypes.POINTER(_Params), ctypes.c_void_p]
        self._launch.restype = ctypes.c_int

    def post(
        self,
        src_blocks: torch.Tensor,
        dst_blocks: torch.Tensor,
        stream: Optional[torch.cuda.Stream] = None,
        done_signal_ptr: int = 0,
        done_value: int = 1,
    ) -> int:
        """Launch the transfer of ``len(src_blocks)`` block pairs; returns a ticket for ``done``.

        ``src_blocks`` / ``dst_blocks`` are int32 device tensors (block ids).  ``done_signal_ptr``
        optionally names a 64-bit counter in the receiver's registered memory (a peer pointer
        obtained from a memory view) that is incremented by ``done_value`` when all data landed.
        """
        if src_blocks.dtype != torch.int32 or dst_blocks.dtype != torch.int32:
            raise TypeError("block tables must be int32")
        if src_blocks.device != self.device or dst_blocks.device != self.device:
            raise ValueError("block tables must live on the sender's GPU")
        if src_blocks.numel() != dst_blocks.numel() or src_blocks.numel() == 0:
            raise ValueError("block tables must be non-empty and of equal length")
        self._seq += 1
        p = self._p
        p.src_blocks, p.dst_blocks = src_blocks.data_ptr(), dst_blocks.data_ptr()
        p.n_pairs = src_blocks.numel()
        p.done_signal, p.done_value = done_signal_ptr, done_value
        p.host_seq = self._seq
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            _lib.check(self._launch(ctypes.byref(p), ctypes.c_void_p(s.cuda_stream)), "nixl_kv_xfer_launch")
        return self._seq

    def done(self, ticket: int) -> bool:
        """True once the launch with that ticket has delivered all its data."""
        return _lib.read_u64(self._flag.data_ptr()) >= ticket

    def wait(self, ticket: int, spins: int = 200_000_000) -> None:
        """Blocks until the launch with that ticket has delivered.  Raises ``IndexError`` when a block id of a
        completed launch pointed outside its cache tensor (the kernel checks every id against the registered
        range, skips such a block and reports it; nothing outside the caches is touched)."""
        for _ in range(spins):
            if self.done(ticket):
                if _lib.read_u64(self._flag.data_ptr() + 8):
                    self._flag[1] = 0
                    raise IndexError("a block id pointed outside its cache tensor; that block was not transferred")
                return
        raise TimeoutError("KV transfer did not complete")

    def bytes_moved(self, n_pairs: int) -> int:
        return n_pairs * self.n_tensors * self.src_layout.block_bytes

    def close(self) -> None:
        if self.src_view:
            self.agent.release_mem_view(self.src_view)
            self.agent.release_mem_view(self.dst_view)
            self.src_view = self.dst_view = 0


def reference_kv_transfer(src, dst, src_blocks, dst_blocks, dst_head_offset, cast_fp8=False, scale=1.0):
    """Plain PyTorch statement of the same operation on one tensor pair (test oracle).

    ``src``: ``[blocks, tokens, heads_s, dim]`` bf16; ``dst``: ``[blocks, tokens, heads_d, dim]``
    bf16 or float8_e4m3fn; returns the updated ``dst`` (in place)."""
    h = src.shape[2]
    picked = src[src_blocks.long()]
    if cast_fp8:
        picked = (picked.float() * scale).to(torch.float8_e4m3fn)
        dst.view(torch.uint8)[dst_blocks.long(), :, dst_head_offset : dst_head_offset + h, :] = picked.view(torch.uint8)
    else:
        dst[dst_blocks.long(), :, dst_head_offset : dst_head_offset + h, :] = picked
    return dst

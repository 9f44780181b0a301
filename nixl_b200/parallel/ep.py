"""MoE expert-parallel dispatch / combine over one NVLink domain.

``Buffer`` follows the Python contract of the reference's ``nixl_ep.Buffer``
(``examples/device/ep/nixl_ep/buffer.py``: ``low_latency_dispatch`` :329,
``low_latency_combine`` :443, ``connect_ranks`` :842, ``barrier`` :878, the mask API :716-737)
and is built the same way - on the agent: every rank registers one symmetric buffer, peers
are reached through a remote memory view, and the kernels (``csrc/src/kernels/ep_kernels.cu``)
store straight into peers' HBM.

Differences that matter to a user:

* one algorithm serves both modes.  ``low_latency_dispatch`` returns the reference's
  ``[local_experts, ranks * max_tokens, hidden]`` layout; ``dispatch`` (throughput mode) returns a
  compact ``[rows, hidden]`` tensor with per-expert offsets, sized for 4096 tokens per GPU.
  The reference's high-throughput kernels need more than 8 ranks (two "RDMA ranks"); this mode
  is the single-box answer.
* rows of one expert arrive already packed and ordered by source rank; there is no second pass
  on the receiver, and ``recv_count`` is exact as soon as the counts are exchanged.
* fp8 scales are returned as ``[..., rows, hidden // 128]`` row-major (one contiguous write per
  token), not column-major.
* no wait ever traps: a peer that stays silent for ``timeout_ms`` is masked and reported by
  ``query_mask_buffer`` / ``status``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch

from ..ops import _lib

_ALIGN = 256


def _up(x: int, a: int = _ALIGN) -> int:
    return (x + a - 1) // a * a


class _Layout(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in (
        "off_counts", "off_counts_flag", "off_disp_flag", "off_recv_x", "off_recv_scales", "off_recv_info", "off_comb_x", "off_comb_flag", "off_comb_in",
        "off_grp", "off_grp_tokens")]


class _Scratch(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("cnt", "fill", "sent", "barrier", "status", "mask")]


class _DispatchParams(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p), ("topk_idx", ctypes.c_void_p),
        ("T", ctypes.c_int32), ("K", ctypes.c_int32), ("H", ctypes.c_int32), ("E", ctypes.c_int32), ("R", ctypes.c_int32), ("rank", ctypes.c_int32),
        ("use_fp8", ctypes.c_int32), ("round_scale", ctypes.c_int32), ("rows_per_expert", ctypes.c_int32), ("cap", ctypes.c_int32),
        ("phases", ctypes.c_int32), ("grid", ctypes.c_int32),
        ("peers", ctypes.c_void_p), ("lay", _Layout), ("epoch", ctypes.c_uint64), ("timeout_ns", ctypes.c_uint64),
        ("recv_count", ctypes.c_void_p), ("layout_range", ctypes.c_void_p), ("expert_offsets", ctypes.c_void_p), ("scr", _Scratch),
        ("send_row", ctypes.c_void_p), ("use_ue8m0", ctypes.c_int32),
        ("topk_weights", ctypes.c_void_p), ("max_tokens", ctypes.c_int32),
    ]


class _CombineParams(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p), ("recv_info", ctypes.c_void_p), ("recv_count", ctypes.c_void_p), ("expert_offsets", ctypes.c_void_p),
        ("topk_idx", ctypes.c_void_p), ("topk_weights", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("T", ctypes.c_int32), ("K", ctypes.c_int32), ("H", ctypes.c_int32), ("E", ctypes.c_int32), ("R", ctypes.c_int32), ("rank", ctypes.c_int32),
        ("phases", ctypes.c_int32), ("grid", ctypes.c_int32),
        ("peers", ctypes.c_void_p), ("lay", _Layout), ("epoch", ctypes.c_uint64), ("timeout_ns", ctypes.c_uint64), ("scr", _Scratch),
        ("pull", ctypes.c_int32), ("send_row", ctypes.c_void_p), ("use_logfmt", ctypes.c_int32), ("max_tokens", ctypes.c_int32),
    ]


@dataclass
class EPHandle:
    """What combine needs from the dispatch it answers."""

    parity: int
    epoch: int
    recv_count: torch.Tensor       # int32 [local_experts]
    expert_offsets: torch.Tensor   # int32 [local_experts + 1]
    layout_range: torch.Tensor     # int64 [local_experts, ranks]: (first row in expert << 32) | rows
    src_info: torch.Tensor         # int32 [rows, 2]: source rank, token * topk + k
    num_max_tokens: int
    hidden: int
    topk: int
    send_row: Optional[torch.Tensor] = None  # int32 [tokens, topk]: row each copy landed on at its receiver
    rows_per_expert: int = 0
    has_group_records: bool = False  # the dispatch was given the weights: combine may reduce per rank before returning rows


class EventOverlap:
    """A CUDA event the caller may wait on (``current_stream_wait``), as in the reference's utils."""

    def __init__(self, event: Optional[torch.cuda.Event] = None):
        self.event = event

    def current_stream_wait(self) -> None:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)


class Buffer:
    """Expert-parallel communication buffer of one rank.

    Args:
        rank, num_ranks: this rank and the EP world size (one NVLink box: up to 8; the kernels accept 64).
        num_experts: global number of routed experts (divisible by ``num_ranks``).
        hidden: model width (multiple of 256 for fp8 dispatch).
        num_max_dispatch_tokens_per_rank: upper bound of tokens a rank dispatches per call.
        num_topk: experts per token.
        device: CUDA device of this rank (default: current).
        agent: an existing ``nixl_agent`` to build on; otherwise one named ``ep<rank>`` is created.
        group: optional ``torch.distributed`` group used by ``connect_ranks`` to exchange metadata.
        timeout_ms: bound of every in-kernel wait on a peer.
        compact_rows: capacity of the throughput-mode layout; default worst case
            ``num_ranks * tokens * min(topk, local_experts)``.
        low_latency_mode: also size the buffer for the low-latency layout
            (``local_experts * num_ranks * tokens`` rows); pass False for a throughput-only buffer.
        combine_pull: combine by letting each token's home rank load its expert outputs straight
            from the expert ranks (every row crosses NVLink once) instead of having the expert
            ranks store them into a landing zone first.  ``None`` picks pull when the combine input
            was written into ``get_next_combine_buffer()`` and push otherwise.  All ranks must make
            the same choice in a given call.
    """

    def __init__(
        self,
        rank: int,
        num_ranks: int,
        num_experts: int,
        hidden: int,
        num_max_dispatch_tokens_per_rank: int,
        num_topk: int,
        device: Optional[torch.device] = None,
        agent=None,
        group=None,
        timeout_ms: int = 30000,
        compact_rows: Optional[int] = None,
        low_latency_mode: bool = True,
        explicitly_destroy: bool = False,
        combine_pull: Optional[bool] = None,
    ):
        from .. import nixl_agent, nixl_agent_config

        if num_experts % num_ranks:
            raise ValueError("num_experts must be divisible by num_ranks")
        self._init_args = dict(hidden=hidden, num_max_dispatch_tokens_per_rank=num_max_dispatch_tokens_per_rank, num_topk=num_topk,
                               timeout_ms=timeout_ms, compact_rows=compact_rows, low_latency_mode=low_latency_mode,
                               explicitly_destroy=explicitly_destroy, combine_pull=combine_pull)
        self._num_sms = getattr(self, "_num_sms", 0)
        self._store = getattr(self, "_store", None)
        self.rank, self.num_ranks, self.num_experts = rank, num_ranks, num_experts
        self.local_experts = num_experts // num_ranks
        self.hidden, self.max_tokens, self.topk = hidden, num_max_dispatch_tokens_per_rank, num_topk
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.group = group
        self.timeout_ns = int(timeout_ms) * 1_000_000
        self.explicitly_destroy = explicitly_destroy
        self.agent = agent or nixl_agent(f"ep{rank}", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
        self._own_agent = agent is None

        R, E, El, H, M, K = num_ranks, num_experts, self.local_experts, hidden, self.max_tokens, num_topk
        self.ll_rows = El * R * M
        self.compact_rows = compact_rows if compact_rows is not None else R * M * min(K, El)
        self.low_latency_mode = low_latency_mode
        self.combine_pull = combine_pull
        cap = max(self.ll_rows, self.compact_rows) if low_latency_mode else self.compact_rows
        self.cap = cap
        # one parity half
        off, lay = 0, {}
        for name, size in (
            ("off_counts", R * E * 4),
            ("off_counts_flag", R * 8),
            ("off_disp_flag", El * R * 8),
            ("off_comb_flag", R * 8),
            ("off_recv_info", cap * 8),
            ("off_recv_scales", cap * (H // 128) * 4),
            ("off_recv_x", cap * H * 2),
            ("off_comb_x", M * max(K, R) * H * 2),  # [M][K] rows (push) or [R][M] rows (rank-reduced combine)
            ("off_comb_in", cap * H * 2),
            ("off_grp", R * M * 80),
            ("off_grp_tokens", R * 4),
        ):
            lay[name] = off
            off = _up(off + size)
        self._half = off
        self._lay = lay
        self._barrier_off = 2 * self._half
        total = 2 * self._half + _up(R * 8)
        with torch.cuda.device(self.device):
            self.buffer = torch.zeros(total, dtype=torch.uint8, device=self.device)
            self._cnt = torch.zeros(3 * E, dtype=torch.int32, device=self.device)
            self._bar = torch.zeros(4, dtype=torch.int32, device=self.device)
            self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.mask = torch.zeros(R, dtype=torch.int32, device=self.device)
        self._reg = self.agent.register_memory(self.buffer)
        self._peers_view = 0
        self._epoch = 0
        self._barrier_epoch = 0
        self._connected: dict[int, str] = {}
        self._disp_cache: dict = {}
        self._side = None
        self._sms = 0
        with torch.cuda.device(self.device):
            self._gemm_status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._comb_params = _CombineParams()
        lib = _lib.lib()
        self._dispatch_fn = lib.nixl_ep_dispatch_launch
        self._dispatch_fn.argtypes = [ctypes.POINTER(_DispatchParams), ctypes.c_void_p]
        self._dispatch_fn.restype = ctypes.c_int
        self._combine_fn = lib.nixl_ep_combine_launch
        self._combine_fn.argtypes = [ctypes.POINTER(_CombineParams), ctypes.c_void_p]
        self._combine_fn.restype = ctypes.c_int
        self._barrier_fn = lib.nixl_ep_barrier_launch
        self._barrier_fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64, ctypes.c_uint64,
                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        self._barrier_fn.restype = ctypes.c_int

    # ------------------------------------------------------------------ sizing helpers

    @staticmethod
    def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int, num_topk: int = 8) -> int:
        """Bytes of symmetric buffer a rank allocates for these shapes (both parity halves)."""
        El = num_experts // num_ranks
        rows = El * num_ranks * num_max_dispatch_tokens_per_rank
        half = rows * (hidden * 4 + (hidden // 128) * 4 + 8) + num_max_dispatch_tokens_per_rank * num_topk * hidden * 2
        return 2 * half + (1 << 20)

    get_low_latency_buffer_size_hint = get_low_latency_rdma_size_hint
    get_rdma_size_hint = get_low_latency_rdma_size_hint

    # ------------------------------------------------------------------ reference-named utilities

    @staticmethod
    def is_sm90_compiled() -> bool:
        """The reference's flag for "the kernels were built with the features of sm_90 and later" (its callers use
        it to decide whether the fp8 and bulk-copy paths exist).  This library is built for sm_100a only and has them."""
        return True

    def set_tcp_store_group(self, store) -> None:
        """Use a ``torch.distributed`` store (e.g. ``TCPStore``) for the metadata exchange of ``connect_ranks``
        instead of a collective: ranks may then join at different times (elastic set-ups)."""
        self._store = store

    def set_num_sms(self, num_sms: int) -> None:
        """CTAs the dispatch and combine kernels use (0: one per SM), leaving the rest to concurrent compute."""
        self._num_sms = max(0, int(num_sms))

    @property
    def num_sms(self) -> int:
        return self._num_sms

    def get_dispatch_config(self, num_ranks: Optional[int] = None) -> dict:
        """Launch configuration in use (the reference returns tuned per-rank-count tables; here the kernels size
        their per-token thread groups themselves and the only knob is the CTA count)."""
        return {"num_sms": self._num_sms or torch.cuda.get_device_properties(self.device).multi_processor_count}

    get_combine_config = get_dispatch_config

    def get_comm_stream(self) -> torch.cuda.Stream:
        """The stream the communication kernels run on: the caller's current stream (no hidden stream)."""
        return torch.cuda.current_stream(self.device)

    def capture(self) -> "EventOverlap":
        """An event at the current point of the current stream."""
        return EventOverlap(self._record())

    def get_local_buffer_tensor(self, dtype: torch.dtype = torch.uint8, offset: int = 0, size: Optional[int] = None) -> torch.Tensor:
        """A typed view of this rank's symmetric buffer (debugging, custom kernels over the same memory)."""
        raw = self.buffer[offset : (offset + size) if size is not None else None]
        return raw.view(dtype)

    def update_memory_buffers(self, num_ranks: int, num_experts_per_rank: int, num_rdma_bytes: int = 0) -> None:
        """Re-size for another world size (ranks joined or left for good): every rank calls this with the new
        shape, then ``connect_ranks`` again.  Outstanding handles become invalid."""
        if num_ranks == self.num_ranks and num_experts_per_rank == self.local_experts:
            return
        agent, rank, device, group, store, sms = self.agent, self.rank, self.device, self.group, self._store, self._num_sms
        own = self._own_agent
        self.destroy()
        self.__init__(rank, num_ranks, num_ranks * num_experts_per_rank, device=device, agent=agent, group=group, **self._init_args)
        self._own_agent, self._store, self._num_sms = own, store, sms

    # ------------------------------------------------------------------ connection management

    def local_metadata(self) -> dict:
        """What a peer needs to reach this rank: agent metadata and the buffer's descriptor."""
        return {
            "rank": self.rank,
            "agent": self.agent.name,
            "md": self.agent.get_agent_metadata(),
            "buffer": (self.buffer.data_ptr(), self.buffer.numel(), self.buffer.get_device()),
            "epoch": self._epoch,
            "barrier_epoch": self._barrier_epoch,
        }

    @property
    def epoch(self) -> int:
        """Number of dispatches issued so far; ranks that talk to each other must agree on it."""
        return self._epoch

    def set_epoch(self, epoch: int, barrier_epoch: Optional[int] = None) -> None:
        """Adopt the step counters of a running group (a rank that joins late or comes back after
        having been disconnected).  ``connect_ranks`` does this itself from the peers' metadata."""
        self._epoch = int(epoch)
        if barrier_epoch is not None:
            self._barrier_epoch = int(barrier_epoch)

    def connect_ranks(self, remote_ranks: Optional[Sequence[int]] = None, metadata: Optional[Sequence[dict]] = None) -> None:
        """Make the listed ranks reachable (all ranks by default).

        ``metadata`` is the list of every rank's ``local_metadata()``; when omitted it is gathered
        over the ``torch.distributed`` group given at construction."""
        if metadata is None and self.num_ranks == 1:
            metadata = [self.local_metadata()]
        if metadata is None and self._store is not None:
            import pickle

            self._store.set(f"nixl_ep/md/{self.rank}", pickle.dumps(self.local_metadata()))
            want = list(remote_ranks) if remote_ranks is not None else list(range(self.num_ranks))
            metadata = [pickle.loads(self._store.get(f"nixl_ep/md/{r}")) for r in sorted(set(want) | {self.rank})]
        if metadata is None:
            import torch.distributed as dist

            if self.group is None and not dist.is_initialized():
                raise ValueError("connect_ranks needs `metadata` or a torch.distributed group")
            metadata = [None] * self.num_ranks
            dist.all_gather_object(metadata, self.local_metadata(), group=self.group)
        by_rank = {m["rank"]: m for m in metadata if m is not None}
        wanted = list(remote_ranks) if remote_ranks is not None else list(range(self.num_ranks))
        for r in wanted:
            if r == self.rank or r in self._connected:
                continue
            m = by_rank[r]
            if m["agent"] != self.agent.name:
                self.agent.add_remote_agent(m["md"])
            self._connected[r] = m["agent"]
        self._peer_desc = {**getattr(self, "_peer_desc", {}), **{r: by_rank[r]["buffer"] for r in by_rank}}
        # Flags carry the step number: a rank that missed steps (it joins late, or was away) catches up
        # with the ranks it connects to.  Callers connect between steps, when the live ranks agree.
        self._epoch = max([self._epoch] + [int(by_rank[r].get("epoch", 0)) for r in wanted if r in by_rank])
        self._barrier_epoch = max([self._barrier_epoch] + [int(by_rank[r].get("barrier_epoch", 0)) for r in wanted if r in by_rank])
        self._rebuild_view()
        with torch.cuda.device(self.device):
            for r in wanted:
                self.mask[r] = 0

    def disconnect_ranks(self, remote_ranks: Sequence[int]) -> None:
        """Stop talking to the listed ranks: they become holes in the peer table and are masked."""
        for r in remote_ranks:
            if r == self.rank:
                continue
            name = self._connected.pop(r, None)
            if name and name != self.agent.name:
                try:
                    self.agent.remove_remote_agent(name)
                except Exception:
                    pass
            self.mask[r] = 1
        self._rebuild_view()

    def _rebuild_view(self) -> None:
        from .. import _bindings as nb

        if self._peers_view:
            self.agent.release_mem_view(self._peers_view)
            self._peers_view = 0
        rows = []
        for r in range(self.num_ranks):
            if r == self.rank:
                rows.append((self.buffer.data_ptr(), self.buffer.numel(), self.buffer.get_device(), self.agent.name))
            elif r in self._connected:
                a, n, d = self._peer_desc[r]
                rows.append((a, n, d, self._connected[r]))
            else:
                rows.append((0, 0, 0, nb.NIXL_NULL_AGENT))
        with torch.cuda.device(self.device):
            self._peers_view = self.agent.prep_mem_view(self.agent.get_remote_descs(rows, "VRAM"))

    # ------------------------------------------------------------------ mask / status

    def query_mask_buffer(self) -> torch.Tensor:
        return self.mask.clone()

    def update_mask_buffer(self, rank: int, masked: bool) -> None:
        self.mask[rank] = 1 if masked else 0

    def clean_mask_buffer(self) -> None:
        self.mask.zero_()
        self._status.zero_()

    @property
    def status(self) -> int:
        """Bit 0: a peer timed out; bit 1: a grid barrier timed out; bit 2: capacity exceeded."""
        return int(self._status.item())

    # ------------------------------------------------------------------ internals

    def _layout(self, parity: int) -> _Layout:
        lay = _Layout()
        for name, off in self._lay.items():
            setattr(lay, name, off + parity * self._half)
        return lay

    def _scratch(self) -> _Scratch:
        E = self.num_experts
        s = _Scratch()
        base = self._cnt.data_ptr()
        s.cnt, s.fill, s.sent = base, base + 4 * E, base + 8 * E
        s.barrier, s.status, s.mask = self._bar.data_ptr(), self._status.data_ptr(), self.mask.data_ptr()
        return s

    def _region(self, parity: int, name: str, nbytes: int) -> torch.Tensor:
        start = self._lay[name] + parity * self._half
        return self.buffer[start : start + nbytes]

    def dispatch_gemm(self, x: torch.Tensor, topk_idx: torch.Tensor, w: torch.Tensor, scale_w: torch.Tensor,
                      low_latency: bool = True, out: Optional[torch.Tensor] = None, dispatch_ctas: int = 32):
        """Dispatch fused with the grouped expert GEMM (fp8, ``w [local_experts, N, hidden]``).

        The dispatch kernel is launched on a side stream with ``dispatch_ctas`` CTAs; the GEMM
        follows immediately on the current stream with the remaining SMs and consumes rows as
        their (expert, source) arrival flags come in, so token movement and expert math overlap
        instead of running back to back.  Returns ``(d [rows, N] bf16, handle, recv_x, scales)``;
        ``handle.recv_count`` / ``expert_offsets`` are valid once the current stream has caught up."""
        from ..ops.grouped_gemm import grouped_gemm_fp8

        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
            self._sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        cur = torch.cuda.current_stream(self.device)
        self._side.wait_stream(cur)
        rpe = self.num_ranks * self.max_tokens if low_latency else 0
        with torch.cuda.stream(self._side):
            recv_x, scales, handle, _, keep = self._dispatch(x, topk_idx, True, False, rpe, 5, False, grid=dispatch_ctas)
        self._keep = keep
        rows = self.ll_rows if low_latency else self.compact_rows
        if out is None:
            out = torch.empty(rows, w.shape[1], dtype=torch.bfloat16, device=self.device)
        d = grouped_gemm_fp8(recv_x[:rows], scales[:rows], w, scale_w, handle.expert_offsets, handle.recv_count, out=out,
                             status=self._gemm_status, fused_with=(self, handle), grid=max(1, self._sms - dispatch_ctas),
                             overlapped=True, rows_per_expert=rpe)
        cur.wait_stream(self._side)
        return d, handle, recv_x, scales

    def _dispatch(self, x, topk_idx, use_fp8, round_scale, rows_per_expert, phases_now, hook_later, grid=0, use_ue8m0=False, topk_weights=None):
        if not self._peers_view:
            if self.num_ranks == 1:
                self.connect_ranks(metadata=[self.local_metadata()])
            else:
                raise RuntimeError("connect_ranks() must run before dispatch")
        T, H = x.shape
        K = topk_idx.shape[1]
        if rows_per_expert and not self.low_latency_mode:
            raise ValueError("buffer was created with low_latency_mode=False")
        if H != self.hidden or K != self.topk or T > self.max_tokens:
            raise ValueError("dispatch shapes exceed what the buffer was sized for")
        if x.dtype != torch.bfloat16 or topk_idx.dtype != torch.int64 or not x.is_contiguous() or not topk_idx.is_contiguous():
            raise TypeError("x must be contiguous bf16 and topk_idx contiguous int64")
        self._epoch += 1
        epoch, parity = self._epoch, self._epoch & 1
        El, R = self.local_experts, self.num_ranks
        # Per-parity outputs, views and parameter block are built once and reused: the Python
        # cost of a call is a handful of attribute stores plus one foreign call.
        key = (parity, bool(use_fp8), rows_per_expert, bool(use_ue8m0))
        slot = self._disp_cache.get(key)
        if slot is None:
            with torch.cuda.device(self.device):
                recv_count = torch.empty(El, dtype=torch.int32, device=self.device)
                layout_range = torch.empty(El, R, dtype=torch.int64, device=self.device)
                expert_offsets = torch.empty(El + 1, dtype=torch.int32, device=self.device)
                send_row = torch.empty(self.max_tokens, K, dtype=torch.int32, device=self.device)
            p = _DispatchParams()
            p.K, p.H, p.E, p.R, p.rank = K, H, self.num_experts, R, self.rank
            p.use_fp8 = int(use_fp8)
            p.use_ue8m0 = int(bool(use_ue8m0 and use_fp8))
            p.rows_per_expert = rows_per_expert
            p.cap = self.ll_rows if rows_per_expert else self.compact_rows
            p.grid = 0
            p.lay = self._layout(parity)
            p.timeout_ns = self.timeout_ns
            p.recv_count, p.layout_range, p.expert_offsets = recv_count.data_ptr(), layout_range.data_ptr(), expert_offsets.data_ptr()
            p.scr = self._scratch()
            p.send_row = send_row.data_ptr()
            rows = p.cap
            row_bytes = H if use_fp8 else 2 * H
            raw = self._region(parity, "off_recv_x", rows * row_bytes)
            recv_x = raw.view(torch.float8_e4m3fn if use_fp8 else torch.bfloat16).view(rows, H)
            scales = None
            if use_fp8 and use_ue8m0:
                # biased exponent bytes, four per 32-bit word (row pitch H/128 bytes)
                scales = self._region(parity, "off_recv_scales", rows * (H // 128)).view(torch.int32).view(rows, H // 512)
            elif use_fp8:
                scales = self._region(parity, "off_recv_scales", rows * (H // 128) * 4).view(torch.float32).view(rows, H // 128)
            src_info = self._region(parity, "off_recv_info", rows * 8).view(torch.int32).view(rows, 2)
            slot = (p, recv_count, layout_range, expert_offsets, recv_x, scales, src_info, send_row)
            self._disp_cache[key] = slot
        p, recv_count, layout_range, expert_offsets, recv_x, scales, src_info, send_row = slot

        p.x, p.topk_idx, p.T = x.data_ptr(), topk_idx.data_ptr(), T
        p.topk_weights = topk_weights.data_ptr() if topk_weights is not None else None
        p.max_tokens = self.max_tokens
        p.round_scale = int(round_scale)
        p.peers = self._peers_view
        p.epoch = epoch
        p.grid = grid or self._num_sms
        stream_ptr = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        fn, ref = self._dispatch_fn, ctypes.byref(p)

        def launch(phases: int) -> None:
            p.phases = phases
            with torch.cuda.device(self.device):
                _lib.check(fn(ref, stream_ptr), "nixl_ep_dispatch_launch")

        launch(phases_now)
        hook = (lambda: launch(2)) if hook_later else None
        handle = EPHandle(parity, epoch, recv_count, expert_offsets, layout_range, src_info, self.max_tokens, H, K, send_row[:T], rows_per_expert,
                          has_group_records=topk_weights is not None)
        keep = (x, topk_idx, topk_weights, p)  # the hook may launch later: keep inputs alive
        return recv_x, scales, handle, hook, keep

    # ------------------------------------------------------------------ routing statistics, reference-named entry points

    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: Optional[int] = None):
        """Routing statistics of ``topk_idx [tokens, topk]``, as the reference's
        ``Buffer.get_dispatch_layout`` returns them: ``(num_tokens_per_rank [ranks] int32,
        num_tokens_per_rdma_rank (None: one NVLink domain), num_tokens_per_expert [experts] int32,
        is_token_in_rank [tokens, ranks] bool, event)``.  Dispatch does not need them (it counts by
        itself); they are for capacity planning and load statistics."""
        E = num_experts or self.num_experts
        T, K = topk_idx.shape
        with torch.cuda.device(self.device):
            per_rank = torch.empty(self.num_ranks, dtype=torch.int32, device=self.device)
            per_expert = torch.empty(E, dtype=torch.int32, device=self.device)
            in_rank = torch.empty(T, self.num_ranks, dtype=torch.bool, device=self.device)
            fn = _lib.lib().nixl_ep_layout_launch
            fn.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p,
                           ctypes.c_void_p, ctypes.c_void_p]
            fn.restype = ctypes.c_int
            _lib.check(fn(topk_idx.data_ptr(), T, K, E, self.num_ranks, per_rank.data_ptr(), per_expert.data_ptr(), in_rank.data_ptr(),
                          ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)), "nixl_ep_layout_launch")
        return per_rank, None, per_expert, in_rank, EventOverlap(None)

    def ht_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: Optional[torch.Tensor] = None, use_fp8: bool = True, **_ignored):
        """The reference's high-throughput dispatch name.  Its multi-node forwarding design needs more
        than one NVLink domain; on one NVSwitch box this is the throughput-mode ``dispatch`` (rows
        arrive packed per local expert, not per token).  Returns ``(recv_x | (recv_x, scales),
        num_recv_tokens_per_expert int32 [local_experts], handle, event)``."""
        recv_x, scales, handle = self.dispatch(x, topk_idx, use_fp8=use_fp8, topk_weights=topk_weights)
        return ((recv_x, scales) if use_fp8 else recv_x), handle.recv_count, handle, EventOverlap(None)

    def ht_combine(self, x: torch.Tensor, handle: EPHandle, topk_idx: torch.Tensor, topk_weights: torch.Tensor, **_ignored):
        """Counterpart of ``ht_dispatch``: ``(combined_x, event)``."""
        return self.combine(x, topk_idx, topk_weights, handle), EventOverlap(None)

    # ------------------------------------------------------------------ low-latency mode

    def low_latency_dispatch(
        self,
        x: torch.Tensor,
        topk_idx: torch.Tensor,
        num_max_dispatch_tokens_per_rank: Optional[int] = None,
        num_experts: Optional[int] = None,
        use_fp8: bool = True,
        round_scale: bool = False,
        use_ue8m0: bool = False,
        async_finish: bool = False,
        return_recv_hook: bool = False,
    ):
        """Dispatch tokens to their experts.

        Returns ``(recv, recv_count, handle, event, hook)`` where ``recv`` is
        ``(packed_recv_x, packed_recv_x_scales)`` for fp8 or ``packed_recv_x`` for bf16, shaped
        ``[local_experts, ranks * max_tokens, hidden]``; only the first ``recv_count[e]`` rows of
        expert ``e`` are valid.  With ``use_ue8m0`` the scales are powers of two and arrive as biased
        exponent bytes packed four to an int32 (``[local_experts, ranks * max_tokens, hidden // 512]``),
        the form Blackwell's block-scaled MMAs take; ``dequant_ue8m0`` turns them back into floats.  The tensors alias the communication buffer: at most two
        dispatches' results are alive at a time."""
        if use_ue8m0 and (not use_fp8 or self.hidden % 512):
            raise ValueError("UE8M0 scales need fp8 dispatch and hidden % 512 == 0")
        if num_max_dispatch_tokens_per_rank not in (None, self.max_tokens) or num_experts not in (None, self.num_experts):
            raise ValueError("buffer was sized for other shapes")
        rpe = self.num_ranks * self.max_tokens
        recv_x, scales, handle, hook, keep = self._dispatch(x, topk_idx, use_fp8, round_scale, rpe, 1 if return_recv_hook else 3, return_recv_hook,
                                                            use_ue8m0=use_ue8m0)
        El = self.local_experts
        packed = recv_x[: El * rpe].view(El, rpe, self.hidden)
        event = EventOverlap(self._record() if async_finish else None)
        self._keep = keep
        if use_fp8:
            return (packed, scales[: El * rpe].view(El, rpe, -1)), handle.recv_count, handle, event, hook
        return packed, handle.recv_count, handle, event, hook

    def low_latency_combine(
        self,
        x: torch.Tensor,
        topk_idx: torch.Tensor,
        topk_weights: torch.Tensor,
        handle: EPHandle,
        use_logfmt: bool = False,
        zero_copy: bool = False,
        async_finish: bool = False,
        return_recv_hook: bool = False,
        out: Optional[torch.Tensor] = None,
    ):
        """Send expert outputs ``x [local_experts, ranks * max_tokens, hidden]`` (bf16) back and
        reduce ``sum_k w[t,k] * y[t,k]``.  Returns ``(combined_x [tokens, hidden], event, hook)``.

        ``zero_copy=True`` (on every rank) says ``x`` was written into ``get_next_combine_buffer(handle)``:
        the home ranks then load the rows directly from there.

        ``use_logfmt=True`` sends the rows in a logarithmic 10-bit format (0.66 of the bf16 bytes on
        the wire, decoded inside the reduction; role of the reference's LogFMT-10,
        examples/device/ep/csrc/kernels/nixl_ep_ll.cu:459-616).  It implies the push path, since the
        encoding happens on the way out, and needs ``hidden % 512 == 0``."""
        if use_logfmt and zero_copy:
            raise ValueError("use_logfmt encodes rows as they are sent; it cannot be combined with zero_copy")
        flat = x.reshape(-1, self.hidden)
        out, hook = self._combine(flat, topk_idx, topk_weights, handle, 1 if return_recv_hook else 3, return_recv_hook, out,
                                  pull=False if use_logfmt else (True if zero_copy else None), use_logfmt=use_logfmt)
        return out, EventOverlap(self._record() if async_finish else None), hook

    # ------------------------------------------------------------------ throughput mode

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, use_fp8: bool = True, round_scale: bool = False, use_ue8m0: bool = False,
                 topk_weights: Optional[torch.Tensor] = None):
        """Throughput-mode dispatch: compact layout.

        With ``topk_weights`` (float32 ``[tokens, topk]``, ``topk <= 8``) the expert ranks are also told which of
        their rows belong to one token and with which weights; ``combine`` then adds those rows up on the
        expert rank and returns one row per (token, rank) instead of one per (token, expert): with top-8
        routing over 8 ranks about a third fewer bytes come back over NVLink.

        Returns ``(recv_x [rows, hidden], scales [rows, hidden//128] | None, handle)``; rows of
        local expert ``e`` are ``handle.expert_offsets[e] : handle.expert_offsets[e] + handle.recv_count[e]``.
        With ``use_ue8m0`` the scales are exponent bytes packed as int32 ``[rows, hidden//512]``, the
        form ``grouped_gemm_mxfp8`` consumes."""
        if use_ue8m0 and (not use_fp8 or self.hidden % 512):
            raise ValueError("UE8M0 scales need fp8 dispatch and hidden % 512 == 0")
        if topk_weights is not None:
            if topk_weights.dtype != torch.float32 or not topk_weights.is_contiguous() or topk_weights.shape != topk_idx.shape:
                raise TypeError("topk_weights must be contiguous float32 of topk_idx's shape")
            if topk_idx.shape[1] > 8 or self.num_ranks > 32:
                topk_weights = None  # a group record holds eight copies: fall back to the per-copy combine
        recv_x, scales, handle, _, keep = self._dispatch(x, topk_idx, use_fp8, round_scale, 0, 3, False, use_ue8m0=use_ue8m0,
                                                         topk_weights=topk_weights)
        self._keep = keep
        return recv_x, scales, handle

    def combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle: EPHandle, out: Optional[torch.Tensor] = None,
                use_logfmt: bool = False):
        """Throughput-mode combine of ``x [rows, hidden]`` bf16 (same row order as ``dispatch`` delivered).
        ``use_logfmt`` as in :meth:`low_latency_combine`."""
        out, _ = self._combine(x, topk_idx, topk_weights, handle, 3, False, out, pull=False if use_logfmt else None, use_logfmt=use_logfmt)
        return out

    def _combine(self, x, topk_idx, topk_weights, handle, phases_now, hook_later, out, pull=None, use_logfmt=False):
        if use_logfmt and self.hidden % 512:
            raise ValueError("use_logfmt needs hidden % 512 == 0")
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise TypeError("combine input must be contiguous bf16")
        if topk_weights.dtype != torch.float32 or not topk_weights.is_contiguous():
            raise TypeError("topk_weights must be contiguous float32")
        T, K = topk_idx.shape
        with torch.cuda.device(self.device):
            if out is None:
                out = torch.empty(T, self.hidden, dtype=torch.bfloat16, device=self.device)
        rows = self.ll_rows if handle.rows_per_expert else self.compact_rows
        staged = self._region(handle.parity, "off_comb_in", rows * self.hidden * 2).view(torch.bfloat16).view(rows, self.hidden)
        if pull is None and handle.has_group_records and not use_logfmt and self.combine_pull is None:
            pull = 2  # the expert ranks know which rows belong to one token: one row per (token, rank) comes back
        if pull is None:
            # Unless told otherwise: pull when the caller wrote its outputs into the exposed buffer
            # (nothing to copy), push when they live elsewhere (staging them first costs more than it saves).
            pull = self.combine_pull if self.combine_pull is not None else x.data_ptr() == staged.data_ptr()
        if pull == 2 and not handle.has_group_records:
            raise ValueError("rank-reduced combine needs a dispatch that was given topk_weights")
        if pull == 1 or pull is True:
            if x.shape[0] > rows:
                raise ValueError("combine input has more rows than the buffer holds")
            if x.data_ptr() != staged.data_ptr():
                staged[: x.shape[0]].copy_(x)  # callers that write into get_next_combine_buffer() skip this copy
        p = self._comb_params
        p.pull = int(pull)
        p.max_tokens = self.max_tokens
        p.use_logfmt = int(use_logfmt)
        p.send_row = handle.send_row.data_ptr() if pull else None
        p.x = x.data_ptr()
        p.recv_info = handle.src_info.data_ptr()
        p.recv_count, p.expert_offsets = handle.recv_count.data_ptr(), handle.expert_offsets.data_ptr()
        p.topk_idx, p.topk_weights, p.out = topk_idx.data_ptr(), topk_weights.data_ptr(), out.data_ptr()
        p.T, p.K, p.H, p.E, p.R, p.rank = T, K, self.hidden, self.num_experts, self.num_ranks, self.rank
        p.grid = self._num_sms
        p.peers = self._peers_view
        p.lay = self._layout(handle.parity)
        p.epoch, p.timeout_ns = handle.epoch, self.timeout_ns
        p.scr = self._scratch()
        stream_ptr = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        fn, ref = self._combine_fn, ctypes.byref(p)

        def launch(phases: int) -> None:
            p.phases = phases
            with torch.cuda.device(self.device):
                _lib.check(fn(ref, stream_ptr), "nixl_ep_combine_launch")

        launch(phases_now)
        self._keep_c = (x, topk_idx, topk_weights, out, p)
        return out, ((lambda: launch(2)) if hook_later else None)

    def get_next_combine_buffer(self, handle: EPHandle) -> torch.Tensor:
        """The symmetric region pull-mode combine reads from, shaped like the dispatch result
        (``[local_experts, ranks * max_tokens, hidden]`` for the low-latency layout, ``[rows, hidden]``
        for the compact one).  An expert GEMM that writes its output here makes combine copy-free."""
        rows = self.ll_rows if handle.rows_per_expert else self.compact_rows
        flat = self._region(handle.parity, "off_comb_in", rows * self.hidden * 2).view(torch.bfloat16).view(rows, self.hidden)
        if handle.rows_per_expert:
            return flat.view(self.local_experts, handle.rows_per_expert, self.hidden)
        return flat

    # ------------------------------------------------------------------ misc

    def _record(self) -> torch.cuda.Event:
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        return ev

    def barrier(self) -> None:
        """Barrier across connected ranks through the symmetric buffers (bounded wait)."""
        if not self._peers_view:
            return
        self._barrier_epoch += 1
        stream = torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            _lib.check(
                self._barrier_fn(self._peers_view, self._barrier_off, self.num_ranks, self.rank, self._barrier_epoch, self.timeout_ns,
                                 self._status.data_ptr(), self.mask.data_ptr(), ctypes.c_void_p(stream.cuda_stream)),
                "nixl_ep_barrier_launch",
            )

    def destroy(self) -> None:
        if self._peers_view:
            self.agent.release_mem_view(self._peers_view)
            self._peers_view = 0
        if self._reg is not None:
            torch.cuda.synchronize(self.device)
            self.agent.deregister_memory(self._reg)
            self._reg = None

    def __del__(self):
        if not getattr(self, "explicitly_destroy", True):
            try:
                self.destroy()
            except Exception:
                pass


# ---------------------------------------------------------------------- PyTorch oracles (tests, baselines)

def per_token_cast_to_fp8(x: torch.Tensor, round_scale: bool = False):
    """1x128 block quantisation used by dispatch, in plain PyTorch: returns (e4m3, fp32 scales)."""
    T, H = x.shape
    g = x.float().view(T, H // 128, 128)
    amax = g.abs().amax(dim=2).clamp(min=1e-4)
    if round_scale:
        ex = torch.ceil(torch.log2(amax / 448.0))
        scale = torch.exp2(ex)
        inv = torch.exp2(-ex)
    else:
        scale = amax / 448.0
        inv = 448.0 / amax
    q = (g * inv.unsqueeze(2)).to(torch.float8_e4m3fn).view(T, H)
    return q, scale


def dequant_ue8m0(packed: torch.Tensor) -> torch.Tensor:
    """int32 ``[..., G/4]`` of biased exponent bytes -> float32 ``[..., G]`` scales (2 ** (byte - 127))."""
    b = packed.contiguous().view(torch.uint8).to(torch.int32)
    return torch.ldexp(torch.ones_like(b, dtype=torch.float32), b - 127)


def dequant_fp8(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    rows, H = q.shape
    return (q.float().view(rows, H // 128, 128) * scale.unsqueeze(2)).view(rows, H)

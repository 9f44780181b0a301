"""Paged KV blocks between two agents by prepared descriptor lists: the path that reaches any peer, over any backend.

``KVTransfer`` (kv_transfer.py) is one kernel launch between GPUs of an NVLink box.  A decode worker on another host is
out of a kernel's reach; what crosses hosts is the agent's own transfer over the TCP backend.  ``KVBlockTransfer`` keeps
that path cheap per request: every block of every cache tensor is prepared once on both sides (``prep_xfer_dlist``), and
a request names block numbers only (``make_prepped_xfer``), which is how serving engines drive the reference
(its kvbench does the same with descriptor lists).  It works on CPU and CUDA tensors alike; which backend carries a
request is the agent's choice (NVLINK inside a box, TCP across boxes).

The receiving side calls :func:`describe_blocks` and hands the bytes to the sender by any channel (a notification will
do); the sender builds a ``KVBlockTransfer`` from them.
"""
from __future__ import annotations

from typing import Sequence, Union

import torch


def _block_rows(caches: Sequence[torch.Tensor]):
    """(address, length, device) of every block of every tensor, tensor-major; all tensors share the block count."""
    if not caches:
        raise ValueError("no cache tensors")
    blocks = caches[0].shape[0]
    rows = []
    for t in caches:
        if t.shape[0] != blocks:
            raise ValueError("cache tensors differ in their number of blocks")
        if not t.is_contiguous():
            raise ValueError("cache tensors must be contiguous (a block is one run of bytes)")
        nbytes = t[0].numel() * t.element_size()
        dev = t.get_device() if t.is_cuda else 0
        base = t.data_ptr()
        rows.extend((base + b * nbytes, nbytes, dev) for b in range(blocks))
    return rows, blocks


def describe_blocks(agent, caches: Sequence[torch.Tensor]) -> bytes:
    """What a peer needs to address the blocks of ``caches`` (which must be registered with ``agent``): the serialized
    descriptor list, tensor-major, ``len(caches) * blocks`` entries."""
    rows, _ = _block_rows(caches)
    mem = "VRAM" if caches[0].is_cuda else "DRAM"
    return agent.get_serialized_descs(agent.get_xfer_descs(rows, mem))


class KVBlockTransfer:
    """Moves numbered blocks between this agent's cache tensors and a peer's.

    Args:
        agent: the local ``nixl_agent``; ``caches`` must be registered with it.
        caches: local cache tensors, each ``[blocks, ...]`` and contiguous.
        remote_agent: the peer's name; its metadata must be loaded.
        remote_blocks: the peer's :func:`describe_blocks` bytes.  The peer must have as many tensors; its block count
            and block size may differ in number but not in size.
    """

    def __init__(self, agent, caches: Sequence[torch.Tensor], remote_agent: str, remote_blocks: bytes):
        self.agent = agent
        self.remote_agent = remote_agent
        rows, self.blocks = _block_rows(caches)
        self.tensors = len(caches)
        mem = "VRAM" if caches[0].is_cuda else "DRAM"
        theirs = agent.deserialize_descs(remote_blocks)
        if theirs.descCount() % self.tensors:
            raise ValueError(f"the peer describes {theirs.descCount()} blocks, not a multiple of {self.tensors} tensors")
        self.remote_blocks = theirs.descCount() // self.tensors
        for t in range(self.tensors):
            if theirs[t * self.remote_blocks][1] != rows[t * self.blocks][1]:
                raise ValueError(f"tensor {t}: a block is {rows[t * self.blocks][1]} bytes here and {theirs[t * self.remote_blocks][1]} bytes at the peer")
        self._local = agent.prep_xfer_dlist("NIXL_INIT_AGENT", agent.get_xfer_descs(rows, mem))
        self._remote = agent.prep_xfer_dlist(remote_agent, theirs)
        self.block_bytes = sum(rows[t * self.blocks][1] for t in range(self.tensors))

    def _indices(self, blocks: Sequence[int], per_tensor: int):
        for b in blocks:
            if not 0 <= b < per_tensor:
                raise IndexError(f"block {b} outside 0..{per_tensor - 1}")
        return [t * per_tensor + int(b) for t in range(self.tensors) for b in blocks]

    def post(self, local_blocks: Sequence[int], remote_blocks: Sequence[int], op: str = "WRITE", notif: Union[bytes, str] = b""):
        """Starts moving ``local_blocks[i]`` <-> ``remote_blocks[i]`` of every tensor (WRITE: to the peer, READ: from it);
        ``notif`` reaches the peer after the data.  Returns the request handle for :meth:`done` / :meth:`wait`."""
        if len(local_blocks) != len(remote_blocks):
            raise ValueError("as many local as remote blocks")
        handle = self.agent.make_prepped_xfer(op, self._local, self._indices(local_blocks, self.blocks), self._remote,
                                              self._indices(remote_blocks, self.remote_blocks), notif)
        if self.agent.transfer(handle) == "ERR":
            self.agent.release_xfer_handle(handle)
            raise RuntimeError("the transfer could not be posted")
        return handle

    def done(self, handle) -> bool:
        state = self.agent.check_xfer_state(handle)
        if state == "ERR":
            raise RuntimeError("the transfer failed")
        return state == "DONE"

    def wait(self, handle, seconds: float = 120.0) -> None:
        import time

        deadline = time.time() + seconds
        while not self.done(handle):
            if time.time() > deadline:
                raise TimeoutError("KV block transfer")
        self.agent.release_xfer_handle(handle)

    def bytes_moved(self, n_blocks: int) -> int:
        return n_blocks * self.block_bytes

    def close(self) -> None:
        for h in (self._local, self._remote):
            if h is not None:
                self.agent.release_dlist_handle(h)
        self._local = self._remote = None

"""Storage side of KV-cache benchmarking: per-rank file regions read into and written from a buffer.

Role of the reference's benchmark/kvbench/test/storage_backend.py (``StorageBackend`` /
``FilesystemBackend``) and of the ``StorageOp`` entries of its traffic patterns
(test/traffic_pattern.py): a rank prepares a file with a region to read and a region to write, gets
transfer handles between those regions and a buffer, and runs them through the agent.  Host
buffers go through the POSIX backend, CUDA buffers through the GDS backend; ``ObjectBackend`` does the
same against an object store (OBJ: S3 or a directory; AZURE_BLOB).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch


@dataclass
class StorageOp:
    """What one rank does to its file in one traffic pattern."""

    file_path: str
    file_size: int
    read_offset: int = 0
    read_size: int = 0
    write_offset: int = 0
    write_size: int = 0

    def __post_init__(self):
        if self.read_offset + self.read_size > self.file_size or self.write_offset + self.write_size > self.file_size:
            raise ValueError("read / write region exceeds file_size")


@dataclass
class StorageHandle:
    tp_idx: int
    rank: int
    read_size: int
    write_size: int
    op: StorageOp
    fd: int


class FilesystemBackend:
    """Files under ``base_path`` (or at the paths the ops name), moved by the agent's file backends."""

    def __init__(self, agent, base_path: str = ".", chunk_bytes: int = 0):
        self.agent = agent
        self.base_path = base_path
        self.chunk_bytes = int(chunk_bytes)  # 0: one descriptor per region
        self._handles: List[StorageHandle] = []
        self._regs = []
        self._backends_made = set()
        os.makedirs(base_path, exist_ok=True)

    def _backend_for(self, buffer: torch.Tensor) -> str:
        name = "GDS" if buffer.is_cuda else "POSIX"
        if name not in self._backends_made:
            if name not in self.agent.backends:
                self.agent.create_backend(name, {})
            self._backends_made.add(name)
        return name

    def default_op(self, tp_idx: int, rank: int, read_size: int, write_size: int) -> StorageOp:
        path = os.path.join(self.base_path, f"kvbench_tp{tp_idx}_rank{rank}.bin")
        return StorageOp(path, read_size + write_size, 0, read_size, read_size, write_size)

    def prepare(self, tp_idx: int, rank: int, read_size: int = 0, write_size: int = 0, op: Optional[StorageOp] = None) -> StorageHandle:
        """Creates (or extends) the file, fills the read region with a rank-dependent pattern and
        registers the file with the agent."""
        op = op or self.default_op(tp_idx, rank, read_size, write_size)
        fd = os.open(op.file_path, os.O_RDWR | os.O_CREAT, 0o644)
        if os.fstat(fd).st_size < op.file_size:
            os.ftruncate(fd, op.file_size)
        if op.read_size:
            pattern = bytes((rank * 31 + i) & 0xFF for i in range(256))
            left, off = op.read_size, op.read_offset
            block = pattern * 4096
            while left > 0:
                n = os.pwrite(fd, block[: min(left, len(block))], off)
                left -= n
                off += n
        reg = self.agent.register_memory([(0, op.file_size, fd, "")], "FILE")
        self._regs.append(reg)
        h = StorageHandle(tp_idx, rank, op.read_size, op.write_size, op, fd)
        self._handles.append(h)
        return h

    def _descs(self, fd: int, file_offset: int, size: int, buffer: torch.Tensor):
        base = buffer.data_ptr()
        dev = buffer.device.index or 0 if buffer.is_cuda else 0
        chunk = self.chunk_bytes or size
        local, remote = [], []
        for off in range(0, size, chunk):
            n = min(chunk, size - off)
            local.append((base + off, n, dev))
            remote.append((file_offset + off, n, fd))
        mem = "VRAM" if buffer.is_cuda else "DRAM"
        return self.agent.get_xfer_descs(local, mem), self.agent.get_xfer_descs(remote, "FILE")

    def _handle(self, op_name: str, h: StorageHandle, file_offset: int, size: int, buffer: torch.Tensor):
        if buffer.numel() * buffer.element_size() < size:
            raise ValueError("buffer is smaller than the storage region")
        backend = self._backend_for(buffer)
        local, remote = self._descs(h.fd, file_offset, size, buffer)
        return self.agent.initialize_xfer(op_name, local, remote, self.agent.name, backends=[backend])

    def get_read_handle(self, h: StorageHandle, buffer: torch.Tensor):
        """Transfer handle that fills ``buffer`` from the file's read region."""
        return self._handle("READ", h, h.op.read_offset, h.read_size, buffer)

    def get_write_handle(self, h: StorageHandle, buffer: torch.Tensor):
        """Transfer handle that stores ``buffer`` into the file's write region."""
        return self._handle("WRITE", h, h.op.write_offset, h.write_size, buffer)

    def close(self, remove_files: bool = False) -> None:
        for reg in self._regs:
            try:
                self.agent.deregister_memory(reg)
            except Exception:
                pass
        for h in self._handles:
            os.close(h.fd)
            if remove_files:
                try:
                    os.unlink(h.op.file_path)
                except OSError:
                    pass
        self._regs, self._handles = [], []


class ObjectBackend:
    """The same interface over an object store (the OBJ backend: an S3 service when ``params`` name an endpoint, a
    directory otherwise; or AZURE_BLOB).  Objects are written whole, so a rank's read region and write region are objects
    of their own (``<prefix>_tp<i>_rank<r>.read`` / ``.write``), cut into ``chunk_bytes`` objects when that is set."""

    def __init__(self, agent, params: Optional[Dict[str, str]] = None, chunk_bytes: int = 0, backend: str = "OBJ", prefix: str = "kvbench"):
        self.agent = agent
        self.backend = backend
        self.chunk_bytes = int(chunk_bytes)
        self.prefix = prefix
        self._regs = []
        self._next_id = 1
        if backend not in agent.backends:
            agent.create_backend(backend, dict(params or {}))

    def _objects(self, name: str, size: int):
        """[(device id, key, length)] of the objects that make up one region; registers them."""
        chunk = self.chunk_bytes or size
        rows = []
        for k, off in enumerate(range(0, size, chunk)):
            rows.append((self._next_id, f"{name}.{k}" if self.chunk_bytes else name, min(chunk, size - off)))
            self._next_id += 1
        self._regs.append(self.agent.register_memory([(0, n, dev, key) for dev, key, n in rows], "OBJ"))
        return rows

    def prepare(self, tp_idx: int, rank: int, read_size: int = 0, write_size: int = 0, op: Optional[StorageOp] = None) -> StorageHandle:
        """Registers the objects and puts the rank's pattern into the ones that will be read."""
        base = f"{self.prefix}_tp{tp_idx}_rank{rank}"
        h = StorageHandle(tp_idx, rank, read_size, write_size, op or StorageOp(base, read_size + write_size, 0, read_size, read_size, write_size), -1)
        h.read_objects = self._objects(base + ".read", read_size) if read_size else []
        h.write_objects = self._objects(base + ".write", write_size) if write_size else []
        if read_size:
            pattern = torch.tensor([(rank * 31 + i) & 0xFF for i in range(256)], dtype=torch.uint8).repeat((read_size + 255) // 256)[:read_size].contiguous()
            reg = self.agent.register_memory(pattern)
            _run(self.agent, self._handle("WRITE", h.read_objects, pattern))
            self.agent.deregister_memory(reg)
        return h

    def _handle(self, op_name: str, objects, buffer: torch.Tensor):
        if buffer.is_cuda:
            raise ValueError("object stores take host buffers")
        total = sum(n for _, _, n in objects)
        if buffer.numel() * buffer.element_size() < total:
            raise ValueError("buffer is smaller than the storage region")
        base, local, remote, off = buffer.data_ptr(), [], [], 0
        for dev, _, n in objects:
            local.append((base + off, n, 0))
            remote.append((0, n, dev))
            off += n
        return self.agent.initialize_xfer(op_name, self.agent.get_xfer_descs(local, "DRAM"), self.agent.get_xfer_descs(remote, "OBJ"), self.agent.name,
                                          backends=[self.backend])

    def get_read_handle(self, h: StorageHandle, buffer: torch.Tensor):
        return self._handle("READ", h.read_objects, buffer)

    def get_write_handle(self, h: StorageHandle, buffer: torch.Tensor):
        return self._handle("WRITE", h.write_objects, buffer)

    def read_back(self, h: StorageHandle, n: int) -> bytes:
        """The first ``n`` bytes of the write region, fetched from the store."""
        first = [h.write_objects[0]]
        n = min(n, first[0][2])
        buf = torch.zeros(first[0][2], dtype=torch.uint8)
        reg = self.agent.register_memory(buf)
        _run(self.agent, self._handle("READ", first, buf))
        self.agent.deregister_memory(reg)
        return bytes(buf[:n].tolist())

    def close(self, remove_files: bool = False) -> None:
        for reg in self._regs:
            try:
                self.agent.deregister_memory(reg)
            except Exception:
                pass
        self._regs = []


def _run(agent, handle) -> float:
    t0 = time.perf_counter()
    state = agent.transfer(handle)
    while state == "PROC":
        state = agent.check_xfer_state(handle)
    if state != "DONE":
        raise RuntimeError(f"storage transfer ended in state {state}")
    return time.perf_counter() - t0


def storage_perftest(base_path: str, size: int, iters: int = 10, mem: str = "cpu", chunk_bytes: int = 0, rank: int = 0,
                     keep_files: bool = False, store: str = "file", store_params: Optional[Dict[str, str]] = None) -> Dict[str, float]:
    """Times reading ``size`` bytes from storage into a buffer and writing them back, ``iters`` times.  ``store`` is
    "file" (a file under ``base_path``), "obj" or "azure_blob" (objects; ``store_params`` go to the backend, and a
    directory store uses ``base_path`` as its bucket when none is named)."""
    from nixl_b200 import nixl_agent, nixl_agent_config

    on_gpu = mem.lower() in ("cuda", "vram")
    agent = nixl_agent(f"kvbench_storage_{rank}_{os.getpid()}", nixl_agent_config(backends=[]))
    buf = torch.zeros(size, dtype=torch.uint8, device="cuda" if on_gpu else "cpu")
    if store != "file":
        backend = {"obj": "OBJ", "azure_blob": "AZURE_BLOB"}[store]
        params = dict(store_params or {})
        if "endpoint_override" not in params and "connection_string" not in params:
            params.setdefault("bucket" if backend == "OBJ" else "container_name", base_path)
        fs = ObjectBackend(agent, params, chunk_bytes, backend)
        reg = agent.register_memory(buf)
        h = fs.prepare(0, rank, read_size=size, write_size=size)
        rh, wh = fs.get_read_handle(h, buf), fs.get_write_handle(h, buf)
        reads, writes = [], []
        for _ in range(iters):
            reads.append(_run(agent, rh))
            writes.append(_run(agent, wh))
        back = fs.read_back(h, 1 << 16)
        ok = back == bytes((rank * 31 + i) & 0xFF for i in range(len(back)))
        agent.release_xfer_handle(rh)
        agent.release_xfer_handle(wh)
        fs.close()
        agent.deregister_memory(reg)
        med = lambda v: sorted(v)[len(v) // 2]  # noqa: E731
        return {"bench": "kvbench-storage", "store": store, "mem": mem, "bytes": size, "iters": iters, "chunk_bytes": chunk_bytes or size,
                "read_ms_p50": round(med(reads) * 1e3, 3), "write_ms_p50": round(med(writes) * 1e3, 3),
                "read_GBps": round(size / med(reads) / 1e9, 3), "write_GBps": round(size / med(writes) / 1e9, 3), "verified": bool(ok)}
    fs = FilesystemBackend(agent, base_path, chunk_bytes)
    fs._backend_for(buf)
    reg = agent.register_memory(buf)
    h = fs.prepare(0, rank, read_size=size, write_size=size)
    rh, wh = fs.get_read_handle(h, buf), fs.get_write_handle(h, buf)
    reads, writes = [], []
    for _ in range(iters):
        reads.append(_run(agent, rh))
        if on_gpu:
            torch.cuda.synchronize()
        writes.append(_run(agent, wh))
    # The write region now holds what was read: the rank's pattern.
    with open(h.op.file_path, "rb") as f:
        f.seek(h.op.write_offset)
        back = f.read(min(size, 1 << 16))
    ok = back == bytes((rank * 31 + i) & 0xFF for i in range(len(back)))
    agent.release_xfer_handle(rh)
    agent.release_xfer_handle(wh)
    fs.close(remove_files=not keep_files)
    agent.deregister_memory(reg)
    med = lambda v: sorted(v)[len(v) // 2]  # noqa: E731
    return {"bench": "kvbench-storage", "mem": mem, "bytes": size, "iters": iters, "chunk_bytes": chunk_bytes or size,
            "read_ms_p50": round(med(reads) * 1e3, 3), "write_ms_p50": round(med(writes) * 1e3, 3),
            "read_GBps": round(size / med(reads) / 1e9, 3), "write_GBps": round(size / med(writes) / 1e9, 3), "verified": bool(ok)}

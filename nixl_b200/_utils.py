"""Raw host buffers for tests and examples (the reference's ``nixl._utils`` module,
src/bindings/python/nixl_utils.cpp): page-aligned allocations addressed by integer, which is what
descriptor tuples ``(addr, len, dev_id)`` want and what O_DIRECT file I/O needs."""
from __future__ import annotations

import ctypes

_libc = ctypes.CDLL(None, use_errno=True)
_libc.aligned_alloc.restype = ctypes.c_void_p
_libc.aligned_alloc.argtypes = [ctypes.c_size_t, ctypes.c_size_t]
_libc.free.argtypes = [ctypes.c_void_p]
_libc.memcmp.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]

IO_SIZE = 4096


def malloc_passthru(size: int) -> int:
    """A 4096-byte aligned host buffer of at least ``size`` bytes; returns its address."""
    rounded = (int(size) + IO_SIZE - 1) // IO_SIZE * IO_SIZE
    addr = _libc.aligned_alloc(IO_SIZE, max(rounded, IO_SIZE))
    if not addr:
        raise MemoryError(f"aligned_alloc({size}) failed")
    return int(addr)


def free_passthru(addr: int) -> None:
    _libc.free(ctypes.c_void_p(addr))


def ba_buf(addr: int, size: int) -> None:
    """Fills the buffer with 0xba."""
    ctypes.memset(ctypes.c_void_p(addr), 0xBA, int(size))


def verify_transfer(addr1: int, addr2: int, size: int) -> None:
    """Raises AssertionError unless the two buffers hold the same bytes."""
    if _libc.memcmp(ctypes.c_void_p(addr1), ctypes.c_void_p(addr2), int(size)) != 0:
        raise AssertionError("buffers differ")

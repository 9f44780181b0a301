"""ctypes access to ``libnixl_kernels.so`` (the fused sm_100a kernels with a C ABI).

The library is built in-tree by ``make -C csrc``.  Importing this module on a machine with a
GPU but without the library is an error: the ops never fall back to eager PyTorch.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libnixl_kernels.so")

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing; build it with `make -C csrc -j8`")
        _lib = ctypes.CDLL(LIB_PATH)
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with CUDA error {rc}")


def read_u64(address: int) -> int:
    """Volatile read of a host word (a pinned flag written by a kernel)."""
    return ctypes.c_uint64.from_address(address).value

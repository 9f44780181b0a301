"""Host-side helpers for the GPU device API exercisers (``csrc/src/kernels/device_api_kernels.cu``).

User kernels include ``csrc/include/device/nixl_device.cuh`` directly; the functions here launch
the library's own test and benchmark kernels that call that API."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

LEVELS = {"THREAD": 0, "WARP": 1, "BLOCK": 2}


class DevPutParams(ctypes.Structure):
    _fields_ = [
        ("local_tiles", ctypes.c_void_p), ("remote_tiles", ctypes.c_void_p), ("local_signals", ctypes.c_void_p), ("remote_signals", ctypes.c_void_p),
        ("peer_ids", ctypes.c_void_p),
        ("peers", ctypes.c_int32), ("rank", ctypes.c_int32), ("iters", ctypes.c_int32), ("window", ctypes.c_int32), ("compute_passes", ctypes.c_int32),
        ("ctas_per_peer", ctypes.c_int32),
        ("tile_bytes", ctypes.c_uint64), ("ack_offset", ctypes.c_uint64), ("timeout_ns", ctypes.c_uint64), ("status", ctypes.c_void_p),
    ]


def put_test(level: str, src_view: int, dst_view: int, sig_view: int, size: int, iters: int, use_get: bool = False, device=None):
    """Runs the correctness kernel; returns ``[status, refused_status, ptr_ok, bad_ptr_is_null]``."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    fn = _lib.lib().nixl_devapi_put_test
    fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p]
    fn.restype = ctypes.c_int
    with torch.cuda.device(dev):
        out = torch.full((4,), -99, dtype=torch.int32, device=dev)
        _lib.check(fn(LEVELS[level], src_view, dst_view, sig_view, size, iters, int(use_get), out.data_ptr(),
                      ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)), "nixl_devapi_put_test")
        torch.cuda.synchronize(dev)
    return out.tolist()


def put_signal_launch(params: DevPutParams, device) -> None:
    fn = _lib.lib().nixl_devapi_put_signal_launch
    fn.argtypes = [ctypes.POINTER(DevPutParams), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    dev = torch.device(device)
    with torch.cuda.device(dev):
        _lib.check(fn(ctypes.byref(params), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)), "nixl_devapi_put_signal_launch")

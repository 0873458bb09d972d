"""ctypes binding of libdeform_sdpa.so (the C ABI declared in include/dsdpa.h).

The library is the product: if it is missing, loading fails loudly.  There is no CPU
or PyTorch fallback anywhere in this package.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import os

_HERE = Path(__file__).resolve().parent
# DSDPA_LIBRARY selects another build of the same library (the checked debug build,
# libdeform_sdpa_checked.so) for a whole process.
LIB_PATH = Path(os.environ["DSDPA_LIBRARY"]) if os.environ.get("DSDPA_LIBRARY") else _HERE / "libdeform_sdpa.so"

# dsdpa_status
OK = 0
ERR_NULL_POINTER = 1
ERR_BAD_DTYPE = 2
ERR_BAD_HEAD_DIM = 3
ERR_BAD_SHAPE = 4
ERR_MISALIGNED = 5
ERR_WORKSPACE = 6
ERR_BAD_FLAGS = 7
ERR_CUDA = 8
ERR_DEVICE_TIMEOUT = 9
ERR_TOO_LARGE = 10
ERR_PEER_ACCESS = 11
ERR_DEVICE_BOUNDS = 12

# dsdpa_dtype
F32, BF16, F16 = 0, 1, 2

# flags
FLAG_MAPS_FROM_L2 = 0x1
FLAG_DETERMINISTIC = 0x2
FLAG_SCATTER_GLOBAL = 0x4
FLAG_SCATTER = 0x8
FLAG_ROUNDED_WEIGHTS = 0x10

# limit of dsdpa_backward_static_scratch (DSDPA_STATIC_SCRATCH_BYTES)
STATIC_SCRATCH_BYTES = 64 << 20

# size of the handle of dsdpa_peer_export / dsdpa_peer_import (DSDPA_PEER_HANDLE_BYTES)
PEER_HANDLE_BYTES = 64

# Every symbol include/dsdpa.h declares (checked by the CPU test-suite).
EXPORTS = (
    "dsdpa_forward",
    "dsdpa_backward_workspace_bytes",
    "dsdpa_backward_supports_dcoords",
    "dsdpa_backward",
    "dsdpa_forward_mirrored",
    "dsdpa_backward_mirrored",
    "dsdpa_peer_export",
    "dsdpa_peer_import",
    "dsdpa_peer_release",
    "dsdpa_backward_static_scratch",
    "dsdpa_status_string",
    "dsdpa_version",
    "dsdpa_last_cuda_error",
    "dsdpa_kernel_launches",
    "dsdpa_device_error",
    "dsdpa_selftest_bounded_wait",
    "dsdpa_build_is_checked",
    "dsdpa_describe_plan",
)


class Problem(ctypes.Structure):
    """Mirror of ``struct dsdpa_problem``."""
    _fields_ = [
        ("B", ctypes.c_int), ("V", ctypes.c_int), ("Hh", ctypes.c_int),
        ("W", ctypes.c_int), ("H", ctypes.c_int), ("D", ctypes.c_int), ("S", ctypes.c_int),
        ("sm_scale", ctypes.c_float), ("dtype", ctypes.c_int), ("flags", ctypes.c_uint),
    ]


class Mirrors(ctypes.Structure):
    """Mirror of ``struct dsdpa_mirrors``: second destinations of out, dq, dk, dv (0 = none)."""
    _fields_ = [("out", ctypes.c_void_p), ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p)]


class DsdpaError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"libdeform_sdpa: {message} (status {status})")
        self.status = status


_lib = None


def lib() -> ctypes.CDLL:
    """Load the library once.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python {(_HERE / 'build.py')}` "
            "(there is no fallback path)")
    L = ctypes.CDLL(str(LIB_PATH))
    vp, ci = ctypes.c_void_p, ctypes.c_int
    pp = ctypes.POINTER(Problem)
    L.dsdpa_forward.argtypes = [pp, vp, vp, vp, vp, vp, vp, ci, vp]
    L.dsdpa_forward.restype = ci
    L.dsdpa_backward_workspace_bytes.argtypes = [pp]
    L.dsdpa_backward_workspace_bytes.restype = ctypes.c_size_t
    L.dsdpa_backward_supports_dcoords.argtypes = [pp]
    L.dsdpa_backward_supports_dcoords.restype = ci
    L.dsdpa_backward.argtypes = [pp] + [vp] * 11 + [vp, ctypes.c_size_t, ci, vp]
    L.dsdpa_backward.restype = ci
    L.dsdpa_forward_mirrored.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, ci, vp]
    L.dsdpa_forward_mirrored.restype = ci
    L.dsdpa_backward_mirrored.argtypes = [pp] + [vp] * 11 + [vp, ctypes.c_size_t, ctypes.POINTER(Mirrors), ci, vp]
    L.dsdpa_backward_mirrored.restype = ci
    L.dsdpa_peer_export.argtypes = [vp, ci, ctypes.c_char_p, ctypes.POINTER(ctypes.c_size_t)]
    L.dsdpa_peer_export.restype = ci
    L.dsdpa_peer_import.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ci, ctypes.POINTER(vp)]
    L.dsdpa_peer_import.restype = ci
    L.dsdpa_peer_release.argtypes = [vp, ctypes.c_size_t, ci]
    L.dsdpa_peer_release.restype = ci
    L.dsdpa_backward_static_scratch.argtypes = [pp] + [vp] * 10 + [ci, vp]
    L.dsdpa_backward_static_scratch.restype = ci
    L.dsdpa_status_string.argtypes = [ci]
    L.dsdpa_status_string.restype = ctypes.c_char_p
    L.dsdpa_version.argtypes = []
    L.dsdpa_version.restype = ci
    L.dsdpa_last_cuda_error.argtypes = []
    L.dsdpa_last_cuda_error.restype = ci
    L.dsdpa_kernel_launches.argtypes = []
    L.dsdpa_kernel_launches.restype = ctypes.c_ulonglong
    L.dsdpa_device_error.argtypes = [ci]
    L.dsdpa_device_error.restype = ci
    L.dsdpa_selftest_bounded_wait.argtypes = [ctypes.c_uint, ci, vp]
    L.dsdpa_selftest_bounded_wait.restype = ci
    L.dsdpa_build_is_checked.argtypes = []
    L.dsdpa_build_is_checked.restype = ci
    L.dsdpa_describe_plan.argtypes = [pp, ctypes.c_char_p, ctypes.c_size_t]
    L.dsdpa_describe_plan.restype = ci
    _lib = L
    return L


def status_string(status: int) -> str:
    return lib().dsdpa_status_string(int(status)).decode()


def check(status: int) -> None:
    """Turn a non-zero dsdpa_status into an exception (ValueError for argument errors,
    DsdpaError for runtime failures), the way the reference's asserts surface."""
    if status == OK:
        return
    msg = status_string(status)
    if status == ERR_CUDA:
        msg += f" (cudaError {lib().dsdpa_last_cuda_error()})"
        raise DsdpaError(status, msg)
    if status in (ERR_DEVICE_TIMEOUT, ERR_PEER_ACCESS, ERR_DEVICE_BOUNDS):
        raise DsdpaError(status, msg)
    if status == ERR_BAD_DTYPE:
        raise NotImplementedError(f"libdeform_sdpa: {msg}")
    raise ValueError(f"libdeform_sdpa: {msg} (status {status})")


def describe_plan(problem: Problem) -> str:
    buf = ctypes.create_string_buffer(512)
    check(lib().dsdpa_describe_plan(ctypes.byref(problem), buf, len(buf)))
    return buf.value.decode()

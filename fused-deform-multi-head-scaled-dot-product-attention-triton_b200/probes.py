"""ctypes binding of libdsdpa_probes.so: the bandwidth probes behind the benchmark's roofline
denominators (csrc/probes/dsdpa_probes.cu).  Measurement tooling; the operator never loads it."""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libdsdpa_probes.so"

# access patterns of shared_pattern()
SHARED_PATTERNS = {
    0: "one contiguous 512-byte line per warp",
    1: "four unrelated 128-byte rows per warp (8 lanes each)",
    2: "two unrelated 256-byte-aligned spans per warp (16 lanes each)",
    3: "two unrelated 256-byte spans across a 256-byte boundary (16 lanes each)",
    4: "one 512-byte span at 128-byte alignment per warp",
    5: "rows r, r+1, r+W, r+W+1 (the four corners of one bilinear sample, W=28)",
}

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with build.py")
        L = ctypes.CDLL(str(LIB_PATH))
        vp, ci, pd, pi = ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int)
        L.dsdpa_probe_l2_read_bandwidth.argtypes = [vp, ctypes.c_size_t, ci, ci, vp, pd, pi]
        L.dsdpa_probe_shared_pattern.argtypes = [ci, ci, ci, vp, pd, pi]
        L.dsdpa_probe_l1_row_gather_bandwidth.argtypes = [vp, ci, ci, vp, pd, pi]
        for f in (L.dsdpa_probe_l2_read_bandwidth, L.dsdpa_probe_shared_pattern, L.dsdpa_probe_l1_row_gather_bandwidth):
            f.restype = ci
        _lib = L
    return _lib


def _finish(status: int, g: ctypes.c_double, err: ctypes.c_int) -> float:
    if status != 0:
        raise RuntimeError(f"bandwidth probe failed (status {status}, cudaError {err.value})")
    return g.value


def l2_read(buffer_ptr: int, nbytes: int, device: int, iters: int = 5) -> float:
    """GB/s of 128-bit reads of an L2-resident buffer by every SM."""
    g, err = ctypes.c_double(), ctypes.c_int()
    return _finish(lib().dsdpa_probe_l2_read_bandwidth(buffer_ptr, nbytes, iters, device, None, ctypes.byref(g),
                                                        ctypes.byref(err)), g, err)


def shared_pattern(pattern: int, device: int, iters: int = 5) -> float:
    """GB/s of 128-bit shared-memory loads in one of SHARED_PATTERNS."""
    g, err = ctypes.c_double(), ctypes.c_int()
    return _finish(lib().dsdpa_probe_shared_pattern(pattern, iters, device, None, ctypes.byref(g), ctypes.byref(err)),
                   g, err)


def l1_row_gather(buffer_ptr: int, device: int, iters: int = 5) -> float:
    """GB/s of a gather of 128-byte rows (8 lanes each) from a 64 KB global buffer that stays in L1."""
    g, err = ctypes.c_double(), ctypes.c_int()
    return _finish(lib().dsdpa_probe_l1_row_gather_bandwidth(buffer_ptr, iters, device, None, ctypes.byref(g),
                                                              ctypes.byref(err)), g, err)

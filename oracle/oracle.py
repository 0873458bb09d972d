"""ctypes front end of the CPU oracle (``deform_sdpa_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, by the smoke run and by the
CPU-baseline leg of the benchmark; the product path never imports it.

The C file restates the reference's pure-PyTorch path (reference file
``ops/torch.py``, lines 5-28) and the gradients autograd derives from it.  All
functions take and return contiguous fp32 CPU tensors in the reference's layouts:
``q, k, v, out [B, V, Hh, L, D]`` and ``coords [B, V, L, V, S, 2]``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_BUILD = _HERE / "_build"
_LIB = None


def build(force: bool = False) -> None:
    """Compile the two builds of the oracle with the Makefile beside this file."""
    src = _HERE / "deform_sdpa_oracle.c"
    outs = [_BUILD / "liboracle_avx2.so", _BUILD / "liboracle_generic.so"]
    fresh = all(o.exists() and o.stat().st_mtime >= src.stat().st_mtime for o in outs)
    if fresh and not force:
        return
    subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True)


def _cpu_has_avx2_fma() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = set(line.split(":", 1)[1].split())
                    return "avx2" in flags and "fma" in flags
    except OSError:
        pass
    return False


def _lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    name = "liboracle_avx2.so" if _cpu_has_avx2_fma() else "liboracle_generic.so"
    path = _BUILD / name
    if not path.exists():
        build()
    lib = ctypes.CDLL(str(path))
    fp = ctypes.c_void_p
    ci = ctypes.c_int
    dims = [ci] * 7 + [ctypes.c_float]
    lib.dsdpa_oracle_forward_range.argtypes = [fp] * 6 + dims + [ctypes.c_longlong, ctypes.c_longlong, ci]
    lib.dsdpa_oracle_forward_range.restype = ci
    lib.dsdpa_oracle_backward_range.argtypes = [fp] * 9 + dims + [ci, ci, ci]
    lib.dsdpa_oracle_backward_range.restype = ci
    lib.dsdpa_oracle_max_threads.argtypes = []
    lib.dsdpa_oracle_max_threads.restype = ci
    _LIB = lib
    return lib


def max_threads() -> int:
    """Threads the oracle uses when ``nthreads`` is 0 (OpenMP's default team)."""
    return int(_lib().dsdpa_oracle_max_threads())


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(device="cpu", dtype=torch.float32).contiguous()


def _dims(q, coords, W, H):
    B, V, Hh, L, D = q.shape
    S = coords.shape[-2]
    if L != W * H:
        raise ValueError(f"L={L} is not W*H={W * H}")
    if tuple(coords.shape) != (B, V, L, V, S, 2):
        raise ValueError(f"coords shape {tuple(coords.shape)} does not match q shape {tuple(q.shape)}")
    return B, V, Hh, L, D, S


def forward(q, k, v, coords, W, H, sm_scale, *, qh_range=None, nthreads=0):
    """Oracle forward.  Returns ``(out, lse)`` as fp32 CPU tensors.

    ``qh_range=(begin, end)`` restricts the work to a range of the flattened
    ``[B, V, Hh, L]`` query-head index; rows outside the range stay zero.
    """
    q, k, v, coords = _f32(q), _f32(k), _f32(v), _f32(coords)
    B, V, Hh, L, D, S = _dims(q, coords, W, H)
    out = torch.zeros_like(q)
    lse = torch.zeros(B, V, Hh, L, dtype=torch.float32)
    lo, hi = (0, B * V * Hh * L) if qh_range is None else qh_range
    rc = _lib().dsdpa_oracle_forward_range(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), coords.data_ptr(), out.data_ptr(), lse.data_ptr(),
        B, V, Hh, W, H, D, S, float(sm_scale), lo, hi, nthreads)
    if rc != 0:
        raise RuntimeError(f"oracle forward failed with status {rc}")
    return out, lse


def backward(q, k, v, coords, dout, W, H, sm_scale, *, bh_range=None, with_dcoords=False, nthreads=0):
    """Oracle backward.  Returns ``(dq, dk, dv, dcoords_or_None)`` as fp32 CPU tensors.

    ``bh_range=(begin, end)`` restricts the work to a range of the flattened
    ``[B, Hh]`` (batch, head) index; rows of other slices stay zero.
    """
    q, k, v, coords, dout = _f32(q), _f32(k), _f32(v), _f32(coords), _f32(dout)
    B, V, Hh, L, D, S = _dims(q, coords, W, H)
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    dc = torch.zeros_like(coords) if with_dcoords else None
    lo, hi = (0, B * Hh) if bh_range is None else bh_range
    rc = _lib().dsdpa_oracle_backward_range(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), coords.data_ptr(), dout.data_ptr(),
        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dc.data_ptr() if dc is not None else None,
        B, V, Hh, W, H, D, S, float(sm_scale), lo, hi, nthreads)
    if rc != 0:
        raise RuntimeError(f"oracle backward failed with status {rc}")
    return dq, dk, dv, dc

"""The operator: ``deform_sdpa_triton(q, k, v, coords, W_IMG, H_IMG, sm_scale)``.

Host-side mirror of the reference's ``_fused_deform_sdpa`` autograd function
(reference ops/triton.py:377-466): same positional signature, same tensor layouts,
same saved-tensor and gradient contract (grads for q, k, v; ``None`` for the rest),
with the device work done by libdeform_sdpa.so through its C ABI.  The name keeps the
reference's ``_triton`` suffix so that call sites do not change; nothing here uses
Triton.
"""
from __future__ import annotations

import ctypes
import os
import warnings

import torch

from . import cabi

_DTYPES = {torch.float32: cabi.F32, torch.bfloat16: cabi.BF16, torch.float16: cabi.F16}

# Process-wide default flags (DSDPA_FLAG_*), e.g. to force a path in tests.
default_flags = 0

# Debug aid, off by default: when set (or with DSDPA_CHECK_DEVICE_ERRORS=1 in the environment),
# the autograd function synchronises the device after every backward and raises if a kernel
# recorded that one of its bounded waits ran out (such a kernel returns without writing its
# results).  Without it nobody looks at that record unless the caller polls
# ``cabi.lib().dsdpa_device_error(device)`` itself.
check_device_errors = os.environ.get("DSDPA_CHECK_DEVICE_ERRORS", "0") not in ("", "0")


def _problem(q, coords, W, H, sm_scale, flags) -> cabi.Problem:
    if q.dtype not in _DTYPES:
        # the reference raises NotImplementedError for other dtypes (ops/triton.py:375)
        raise NotImplementedError(f"deform_sdpa: unsupported dtype {q.dtype}")
    B, V, Hh, L, D = q.shape
    S = coords.shape[-2]
    return cabi.Problem(B, V, Hh, int(W), int(H), D, S, float(sm_scale), _DTYPES[q.dtype], int(flags))


def _check_inputs(q, k, v, coords, W, H):
    if not (q.is_cuda and k.is_cuda and v.is_cuda and coords.is_cuda):
        raise RuntimeError("deform_sdpa: tensors must live on a CUDA device (there is no CPU path)")
    if q.dim() != 5 or coords.dim() != 6:
        raise ValueError("deform_sdpa: q/k/v must be [B, V, heads, L, D] and coords [B, V, L, V, S, 2]")
    if not (q.shape == k.shape == v.shape):
        # ops/triton.py:384-385
        raise ValueError(f"deform_sdpa: q, k, v shapes differ: {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if not (q.dtype == k.dtype == v.dtype):
        raise ValueError("deform_sdpa: q, k, v dtypes differ")
    B, V, Hh, L, D = q.shape
    if D not in (16, 32, 64, 128, 256):
        # ops/triton.py:386
        raise ValueError(f"deform_sdpa: head dim {D} not in {{16, 32, 64, 128, 256}}")
    if L != int(W) * int(H):
        # ops/triton.py:387
        raise ValueError(f"deform_sdpa: L={L} is not W_IMG*H_IMG={int(W) * int(H)}")
    S = coords.shape[-2]
    if tuple(coords.shape) != (B, V, L, V, S, 2):
        raise ValueError(f"deform_sdpa: coords shape {tuple(coords.shape)} does not match [B, V, L, V, S, 2]")
    if not (q.device == k.device == v.device == coords.device):
        raise ValueError("deform_sdpa: tensors are on different devices")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _check_mirror(name, m, like):
    if m is None:
        return
    if m.shape != like.shape or m.dtype != like.dtype or not m.is_contiguous() or not (m.is_cuda or m.is_pinned()):
        raise ValueError(f"mirror {name!r} must be a contiguous CUDA (or pinned host) tensor of shape "
                         f"{tuple(like.shape)} and dtype {like.dtype}")


def forward_raw(q, k, v, coords, W, H, sm_scale, flags=None, out_mirror=None):
    """Forward through the C ABI.  Returns ``(out, lse)``; no autograd.

    ``out_mirror``: a second tensor (same shape and dtype as ``out``; it may live on another GPU
    whose memory this process has mapped, or in pinned host memory) that the kernel stores every
    row of ``out`` to as well."""
    flags = default_flags if flags is None else flags
    _check_inputs(q, k, v, coords, W, H)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    coords = coords.contiguous().to(torch.float32)
    prob = _problem(q, coords, W, H, sm_scale, flags)
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:4], device=q.device, dtype=torch.float32)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    _check_mirror("out", out_mirror, out)
    st = cabi.lib().dsdpa_forward_mirrored(ctypes.byref(prob), _ptr(q), _ptr(k), _ptr(v), _ptr(coords), _ptr(out),
                                           _ptr(lse), _ptr(out_mirror), q.device.index, ctypes.c_void_p(stream))
    cabi.check(st)
    return out, lse


def backward_raw(q, k, v, coords, out, lse, dout, W, H, sm_scale, flags=None, want_dcoords=False, mirrors=None):
    """Backward through the C ABI.  Returns ``(dq, dk, dv, dcoords_or_None)``.

    ``mirrors``: optional dict with any of the keys ``out``, ``dq``, ``dk``, ``dv``: tensors (possibly
    in another GPU's memory mapped into this process) that receive a second copy of that result
    (of the ``out`` input, for ``out``), stored by the kernels that produce it."""
    flags = default_flags if flags is None else flags
    q, k, v, out = q.contiguous(), k.contiguous(), v.contiguous(), out.contiguous()
    coords = coords.contiguous().to(torch.float32)
    dout = dout.contiguous()  # the reference asserts this (ops/triton.py:425); here it is made so
    if dout.dtype != q.dtype:
        dout = dout.to(q.dtype)
    prob = _problem(q, coords, W, H, sm_scale, flags)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dcoords = torch.empty_like(coords) if want_dcoords else None
    L = cabi.lib()
    ws_bytes = int(L.dsdpa_backward_workspace_bytes(ctypes.byref(prob)))
    ws = torch.empty(max(ws_bytes, 16), device=q.device, dtype=torch.uint8) if ws_bytes else None
    stream = torch.cuda.current_stream(q.device).cuda_stream
    mir = None
    if mirrors:
        unknown = set(mirrors) - {"out", "dq", "dk", "dv"}
        if unknown:
            raise ValueError(f"unknown mirrors {sorted(unknown)}")
        for name, t in mirrors.items():
            _check_mirror(name, t, q)
        mir = cabi.Mirrors(*(mirrors[n].data_ptr() if mirrors.get(n) is not None else None
                             for n in ("out", "dq", "dk", "dv")))
    st = L.dsdpa_backward_mirrored(ctypes.byref(prob), _ptr(q), _ptr(k), _ptr(v), _ptr(coords), _ptr(out), _ptr(lse),
                                   _ptr(dout), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dcoords), _ptr(ws), ws_bytes,
                                   ctypes.byref(mir) if mir is not None else None,
                                   q.device.index, ctypes.c_void_p(stream))
    cabi.check(st)
    if ws is not None:
        ws.record_stream(torch.cuda.current_stream(q.device))
    return dq, dk, dv, dcoords


class _FusedDeformSDPA(torch.autograd.Function):
    """Counterpart of the reference's ``_fused_deform_sdpa`` (ops/triton.py:377-464)."""

    @staticmethod
    def forward(ctx, q, k, v, coords, WIDTH, HEIGHT, sm_scale):
        out, lse = forward_raw(q, k, v, coords, WIDTH, HEIGHT, sm_scale)
        # the reference saves q, k, v, coords, o, M (ops/triton.py:413); coords stay normalised here
        ctx.save_for_backward(q, k, v, coords, out, lse)
        ctx.sm_scale = float(sm_scale)
        ctx.WIDTH, ctx.HEIGHT = int(WIDTH), int(HEIGHT)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, coords, out, lse = ctx.saved_tensors
        want_dc = ctx.needs_input_grad[3]
        if want_dc:
            # the coordinate gradient rides on the two-pass form; where that form cannot run (a map
            # too large for its index builder, scatter flags) coords get None, as in the reference
            prob = _problem(q, coords, ctx.WIDTH, ctx.HEIGHT, ctx.sm_scale, default_flags)
            if not cabi.lib().dsdpa_backward_supports_dcoords(ctypes.byref(prob)):
                warnings.warn("deform_sdpa: the coordinate gradient is not available for this problem "
                              "(scatter form of the backward); coords receive no gradient", UserWarning, stacklevel=2)
                want_dc = False
        dq, dk, dv, dc = backward_raw(q, k, v, coords, out, lse, do, ctx.WIDTH, ctx.HEIGHT, ctx.sm_scale,
                                      want_dcoords=want_dc)
        if check_device_errors:
            cabi.check(cabi.lib().dsdpa_device_error(q.device.index))
        if dc is not None and dc.dtype != coords.dtype:
            dc = dc.to(coords.dtype)
        # ops/triton.py:464 returns (dq, dk, dv, None, None, None, None)
        return dq, dk, dv, dc, None, None, None


deform_sdpa_triton = _FusedDeformSDPA.apply
deform_sdpa = deform_sdpa_triton

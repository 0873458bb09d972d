"""Size-independent properties of the operator, written against plain callables so that the same
checks run on the CPU oracle at a small size (which validates the checks themselves) and on the
CUDA path at the benchmark's full sizes (where the oracle would take minutes).

``fwd(q, k, v, coords) -> out`` and ``bwd(q, k, v, coords, dout) -> (dq, dk, dv)``; tensors of the
reference's layouts, ``q, k, v, dout, out [B, V, Hh, L, D]``, ``coords [B, V, L, V, S, 2]``.
"""
from __future__ import annotations

import torch


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return (a - b).abs().max().item() / max(b.abs().max().item(), 1e-30)


def check_constant_values_come_back(fwd, q, k, coords, tol):
    """Attention weights sum to one and, for coordinates inside the map, so do the four bilinear
    weights: a value map that is 1 everywhere gives out == 1."""
    ones = torch.ones_like(k)
    out = fwd(q, k, ones, coords)
    assert torch.isfinite(out).all()
    assert (out.double() - 1.0).abs().max().item() <= tol


def check_forward_is_linear_in_v(fwd, q, k, v, coords):
    """out(2v) == 2 out(v), bit for bit: doubling is exact in every storage type and commutes
    with every rounding on the way."""
    a = fwd(q, k, v, coords)
    b = fwd(q, k, v * 2, coords)
    assert torch.equal(b, a * 2)


def check_value_gradient_is_the_adjoint(fwd, bwd, q, k, v, coords, dout, v_probe, tol):
    """out is linear in v, so <dv, v'> == <dout, out(v')> for any v'."""
    _, _, dv = bwd(q, k, v, coords, dout)
    lhs = (dv.double() * v_probe.double()).sum().item()
    rhs = (dout.double() * fwd(q, k, v_probe, coords).double()).sum().item()
    scale = (dout.double().abs() * fwd(q, k, v_probe.abs(), coords).double().abs()).sum().item()
    assert abs(lhs - rhs) <= tol * scale, (lhs, rhs, scale)


def check_query_gradient_vanishes_for_constant_keys(bwd, q, v, coords, dout, tol):
    """Keys that are the same row everywhere make every logit of a query equal (coordinates
    inside the map), whatever q is: the softmax does not depend on q, so dq == 0 up to the
    rounding of the stored out that delta is formed from."""
    B, V, Hh, L, D = q.shape
    row = torch.linspace(-1.0, 1.0, D, device=q.device).to(q.dtype)
    k_const = row.expand(B, V, Hh, L, D).contiguous()
    dq, dk, _ = bwd(q, k_const, v, coords, dout)
    scale = max(dout.double().abs().max().item() * v.double().abs().max().item(), 1e-30)
    assert dq.double().abs().max().item() <= tol * scale


def check_batch_elements_are_independent(fwd, bwd, q, k, v, coords, dout, b, tol):
    """Batch element ``b`` of a full run equals the run of that element alone (the property the
    partitioner rests on)."""
    sl = slice(b, b + 1)
    out_full = fwd(q, k, v, coords)
    grads_full = bwd(q, k, v, coords, dout)
    out_one = fwd(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), coords[sl].contiguous())
    grads_one = bwd(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), coords[sl].contiguous(),
                    dout[sl].contiguous())
    # (an implementation may tile a one-element batch differently, so rounding may differ)
    for name, f, o in zip(("out", "dq", "dk", "dv"), (out_full,) + tuple(grads_full), (out_one,) + tuple(grads_one)):
        assert _rel(f[sl], o) <= tol, name


def check_slice_against(reference_fwd, reference_bwd, fwd_out, grads, q, k, v, coords, dout, b, h, tol):
    """One (batch, head) slice of results computed at full size against a trusted implementation
    run on that slice alone (fp32 CPU tensors in and out)."""
    sl = (slice(b, b + 1), slice(None), slice(h, h + 1))
    qs, ks, vs, ds = (t[sl].float().cpu().contiguous() for t in (q, k, v, dout))
    cs = coords[b:b + 1].float().cpu().contiguous()
    ref_out = reference_fwd(qs, ks, vs, cs)
    ref_grads = reference_bwd(qs, ks, vs, cs, ds)
    assert _rel(fwd_out[sl].float().cpu(), ref_out) <= tol, "out"
    for name, g, r in zip(("dq", "dk", "dv"), grads, ref_grads):
        assert _rel(g[sl].float().cpu(), r) <= tol, name

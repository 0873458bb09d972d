"""The size-independent properties (tests/properties.py) hold for the CPU oracle on a small case.
This pins the checks themselves; tests/test_gpu_properties.py applies them to the CUDA path at
the benchmark's full sizes."""
import torch

import properties as prop


def _case(coords_kind="uniform", B=2, V=2, Hh=2, W=5, H=4, D=16, S=3, seed=3):
    g = torch.Generator().manual_seed(seed)
    L = W * H
    q, k, v, dout, probe = (torch.randn(B, V, Hh, L, D, generator=g) for _ in range(5))
    coords = torch.rand(B, V, L, V, S, 2, generator=g)
    if coords_kind == "oob":
        coords = coords * 1.6 - 0.3
    return q, k, v, dout, probe, coords, W, H, 0.37


def _callables(oracle, W, H, scale):
    fwd = lambda q, k, v, c: oracle.forward(q, k, v, c, W, H, scale)[0]          # noqa: E731
    bwd = lambda q, k, v, c, do: oracle.backward(q, k, v, c, do, W, H, scale)[:3]  # noqa: E731
    return fwd, bwd


def test_properties_hold_for_the_oracle(oracle):
    q, k, v, dout, probe, coords, W, H, scale = _case()
    fwd, bwd = _callables(oracle, W, H, scale)
    prop.check_constant_values_come_back(fwd, q, k, coords, tol=1e-5)
    prop.check_forward_is_linear_in_v(fwd, q, k, v, coords)
    prop.check_value_gradient_is_the_adjoint(fwd, bwd, q, k, v, coords, dout, probe, tol=1e-5)
    prop.check_query_gradient_vanishes_for_constant_keys(bwd, q, v, coords, dout, tol=1e-5)
    prop.check_batch_elements_are_independent(fwd, bwd, q, k, v, coords, dout, b=1, tol=1e-6)
    out, grads = fwd(q, k, v, coords), bwd(q, k, v, coords, dout)
    prop.check_slice_against(fwd, bwd, out, grads, q, k, v, coords, dout, b=1, h=0, tol=1e-6)


def test_properties_that_survive_out_of_range_coordinates(oracle):
    q, k, v, dout, probe, coords, W, H, scale = _case("oob")
    fwd, bwd = _callables(oracle, W, H, scale)
    prop.check_forward_is_linear_in_v(fwd, q, k, v, coords)
    prop.check_value_gradient_is_the_adjoint(fwd, bwd, q, k, v, coords, dout, probe, tol=1e-5)
    prop.check_batch_elements_are_independent(fwd, bwd, q, k, v, coords, dout, b=0, tol=1e-6)


def test_the_checks_notice_a_wrong_implementation(oracle):
    """A forward whose weights do not sum to one, and a backward with a scaled dv, fail."""
    import pytest
    q, k, v, dout, probe, coords, W, H, scale = _case()
    fwd, bwd = _callables(oracle, W, H, scale)
    with pytest.raises(AssertionError):
        prop.check_constant_values_come_back(lambda *a: fwd(*a) * 1.01, q, k, coords, tol=1e-5)
    with pytest.raises(AssertionError):
        bad = lambda *a: tuple(g * s for g, s in zip(bwd(*a), (1.0, 1.0, 1.02)))   # noqa: E731
        prop.check_value_gradient_is_the_adjoint(fwd, bad, q, k, v, coords, dout, probe, tol=1e-5)
    with pytest.raises(AssertionError):
        prop.check_forward_is_linear_in_v(lambda q_, k_, v_, c_: fwd(q_, k_, v_, c_) + 1.0, q, k, v, coords)


def test_tolerances_of_the_full_size_checks_fit_16_bit_storage(oracle):
    """The tolerances tests/test_gpu_properties.py uses for 16-bit storage, tried on an emulation of
    such a path: inputs rounded to bf16, exact arithmetic (the oracle), results rounded to bf16 -- at
    the benchmark's C5 geometry with fewer batch elements and heads."""
    W = H = 28
    B, V, Hh, D, S, scale = 2, 8, 2, 64, 32, 0.125
    L = W * H
    g = torch.Generator().manual_seed(5)
    bf = lambda t: t.to(torch.bfloat16)     # noqa: E731
    q, k, v, dout, probe = (bf(torch.randn(B, V, Hh, L, D, generator=g)) for _ in range(5))
    coords = torch.rand(B, V, L, V, S, 2, generator=g)

    def fwd(q_, k_, v_, c_):
        return bf(oracle.forward(q_.float(), k_.float(), v_.float(), c_, W, H, scale)[0])

    def bwd(q_, k_, v_, c_, do_):
        # (delta is formed from the stored, rounded out on the CUDA path; the oracle recomputes it
        # exactly, which only makes this emulation the stricter of the two for the dq check)
        return tuple(bf(t) for t in oracle.backward(q_.float(), k_.float(), v_.float(), c_, do_.float(), W, H, scale)[:3])

    prop.check_constant_values_come_back(fwd, q, k, coords, tol=4e-3)
    prop.check_forward_is_linear_in_v(fwd, q, k, v, coords)
    prop.check_value_gradient_is_the_adjoint(fwd, bwd, q, k, v, coords, dout, probe, tol=2e-3)
    prop.check_query_gradient_vanishes_for_constant_keys(bwd, q, v, coords, dout, tol=2e-2)
    prop.check_batch_elements_are_independent(fwd, bwd, q, k, v, coords, dout, b=1, tol=1e-2)

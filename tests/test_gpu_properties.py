"""The CUDA path at the benchmark's FULL sizes (C1-C5 as the benchmark runs them), checked through
properties that need no full-size reference (tests/properties.py, pinned on the CPU oracle by
tests/test_properties_oracle.py), plus two (batch, head) slices of every result against the oracle."""
import pytest
import torch

import properties as prop
from conftest import TOL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    import ops
    return ops.backend


def _device_inputs(backend, cfg, dev):
    """The configuration's seeded inputs, generated one batch element at a time."""
    parts = []
    for b in range(cfg.B):
        q, k, v, coords, dout = backend.inputs.make_inputs(cfg, batch_range=(b, b + 1))
        parts.append(tuple(t.to(dev, cfg.dtype) for t in (q, k, v, dout)) + (coords.to(dev),))
    q, k, v, dout, coords = (torch.cat([p[i] for p in parts]).contiguous() for i in range(5))
    return q, k, v, dout, coords


@pytest.mark.parametrize("cfgname", ["C1", "C2", "C3", "C4", "C5"])
def test_full_size_properties(backend, oracle, cfgname):
    cfg = backend.inputs.CONFIGS[cfgname]
    dev = torch.device("cuda", 0)
    q, k, v, dout, coords = _device_inputs(backend, cfg, dev)
    args = (cfg.W, cfg.H, cfg.sm_scale)
    narrow = cfg.dtype != torch.float32
    inside = cfg.coords != "oob"          # every coordinate inside the map

    def fwd(q_, k_, v_, c_):
        return backend.forward_raw(q_, k_, v_, c_, *args)[0]

    def bwd(q_, k_, v_, c_, do_):
        out_, lse_ = backend.forward_raw(q_, k_, v_, c_, *args)
        return backend.backward_raw(q_, k_, v_, c_, out_, lse_, do_, *args)[:3]

    if inside:
        # (one storage-type ulp below 1 is the coarsest step there)
        prop.check_constant_values_come_back(fwd, q, k, coords, tol=4e-3 if narrow else 1e-5)
        prop.check_query_gradient_vanishes_for_constant_keys(bwd, q, v, coords, dout, tol=2e-2 if narrow else 1e-4)
    prop.check_forward_is_linear_in_v(fwd, q, k, v, coords)
    probe = torch.randn(q.shape, device=dev, generator=torch.Generator(device=dev).manual_seed(77)).to(cfg.dtype)
    prop.check_value_gradient_is_the_adjoint(fwd, bwd, q, k, v, coords, dout, probe, tol=2e-3 if narrow else 1e-5)
    prop.check_batch_elements_are_independent(fwd, bwd, q, k, v, coords, dout, b=cfg.B - 1,
                                              tol=1e-2 if narrow else 1e-5)

    out = fwd(q, k, v, coords)
    grads = bwd(q, k, v, coords, dout)
    torch.cuda.synchronize()
    backend.cabi.check(backend.cabi.lib().dsdpa_device_error(0))
    ref_fwd = lambda q_, k_, v_, c_: oracle.forward(q_, k_, v_, c_, *args)[0]             # noqa: E731
    ref_bwd = lambda q_, k_, v_, c_, do_: oracle.backward(q_, k_, v_, c_, do_, *args)[:3]  # noqa: E731
    for b, h in ((0, 0), (cfg.B - 1, cfg.Hh - 1)):
        prop.check_slice_against(ref_fwd, ref_bwd, out, grads, q, k, v, coords, dout, b, h, tol=TOL[cfg.dtype])

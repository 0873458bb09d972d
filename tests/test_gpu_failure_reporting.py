"""How a kernel's failure reaches the host, tested without faulting or hanging a GPU.

Every wait inside the kernels is bounded: when it runs out, the kernel records the fact in the
library's error word and returns, and dsdpa_device_error() reports it.  The self-test entry makes
exactly that happen -- one warp waits on a barrier nobody completes, with a limit of a few hundred
polls -- so the whole chain (give up, record, return, report once, clear) runs for real.
"""
import ctypes

import pytest
import torch

from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_once_and_the_context_stays_usable():
    import ops
    be = ops.backend
    cabi, lib = be.cabi, be.cabi.lib()
    dev = torch.device("cuda", 0)
    assert lib.dsdpa_device_error(0) == cabi.OK
    stream = torch.cuda.current_stream(dev).cuda_stream
    cabi.check(lib.dsdpa_selftest_bounded_wait(300, 0, ctypes.c_void_p(stream)))
    assert lib.dsdpa_device_error(0) == cabi.ERR_DEVICE_TIMEOUT      # reported ...
    assert lib.dsdpa_device_error(0) == cabi.OK                      # ... once
    with pytest.raises(cabi.DsdpaError):
        cabi.check(cabi.ERR_DEVICE_TIMEOUT)
    # the device still computes, and correctly
    c = load_golden("tiny_f32_uniform")
    out, _ = be.forward_raw(*(c[n].to(dev) for n in ("q", "k", "v", "coords")), c["W"], c["H"], c["sm_scale"])
    assert rel_err(out, c["out"]) < 1e-4
    assert lib.dsdpa_selftest_bounded_wait(0, 0, None) == cabi.ERR_BAD_SHAPE


def test_the_operator_can_be_told_to_look_at_the_record(monkeypatch):
    """By default nobody polls the error word.  With ``check_device_errors`` set, the autograd
    function synchronises after every backward and raises if a kernel gave up; here a pending
    record (left by the self-test) is what it finds."""
    import ops
    from ops.triton import deform_sdpa_triton
    be = ops.backend
    cabi, lib = be.cabi, be.cabi.lib()
    op = be.op
    dev = torch.device("cuda", 0)
    c = load_golden("tiny_f32_uniform")

    def step():
        q, k, v = (c[n].to(dev).requires_grad_(True) for n in ("q", "k", "v"))
        deform_sdpa_triton(q, k, v, c["coords"].to(dev), c["W"], c["H"], c["sm_scale"]).backward(c["dout"].to(dev))
        return q.grad

    monkeypatch.setattr(op, "check_device_errors", True)
    assert rel_err(step(), c["dq"]) < 1e-4                     # nothing pending: no exception
    cabi.check(lib.dsdpa_selftest_bounded_wait(200, 0, None))
    with pytest.raises(cabi.DsdpaError, match="bounded wait"):
        step()
    monkeypatch.setattr(op, "check_device_errors", False)
    cabi.check(lib.dsdpa_selftest_bounded_wait(200, 0, None))
    step()                                                      # default: the record is not looked at
    assert lib.dsdpa_device_error(0) == cabi.ERR_DEVICE_TIMEOUT

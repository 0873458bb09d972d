"""dsdpa_backward_static_scratch: the backward for callers that are not allowed to allocate.

A serving loop with a frozen memory budget, or a plugin whose host owns the device heap, cannot
hand dsdpa_backward the scratch buffer it asks for.  For them the library carries a fixed
64 MiB scratch array in its own image and this entry point uses it; the price is a size
limit and that calls must not overlap on the GPU.  The test calls it through the C ABI twice
in a row, with different inputs, and compares each result with what the ordinary entry
point (scratch allocated by the caller) gives for the same inputs: the second call must not
see anything of the first one in the shared array.  Both entry points run the same kernels in
the same fixed summation order, so the comparison is exact (bit for bit), which a leak of even
one stale scratch word would break; the CPU oracle is compared within the path's tolerance on
top.  The second call is also watched for allocations: neither the driver's free-memory figure
nor torch's allocator may move across it.

The file name sorts last on purpose, so that a run stopping at the first failure has
already been through every other test.
"""
import ctypes

import pytest
import torch

from conftest import TOL, rel_err


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _inputs(seed, dtype, dev, B=1, V=3, Hh=2, W=14, H=14, D=32, S=8):
    g = torch.Generator().manual_seed(seed)
    L = W * H
    q, k, v, dout = (torch.randn(B, V, Hh, L, D, generator=g).to(dtype).to(dev) for _ in range(4))
    coords = (torch.rand(B, V, L, V, S, 2, generator=g) * 1.2 - 0.1).to(dev)
    return q, k, v, dout, coords, (B, V, Hh, W, H, D, S)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_backward_matches_ordinary_backward_twice(dtype, oracle):
    import ops
    be = ops.backend
    cabi = be.cabi
    lib = cabi.lib()
    dev = torch.device("cuda", 0)
    sm_scale = 0.25
    for call, seed in enumerate((101, 202)):      # two calls in a row, different data
        q, k, v, dout, coords, (B, V, Hh, W, H, D, S) = _inputs(seed, dtype, dev)
        out, lse = be.forward_raw(q, k, v, coords, W, H, sm_scale)
        ref_dq, ref_dk, ref_dv, _ = be.backward_raw(q, k, v, coords, out, lse, dout, W, H, sm_scale)
        dt = {torch.float32: cabi.F32, torch.bfloat16: cabi.BF16}[dtype]
        prob = cabi.Problem(B, V, Hh, W, H, D, S, sm_scale, dt, 0)
        need = lib.dsdpa_backward_workspace_bytes(ctypes.byref(prob))
        assert 0 < need <= cabi.STATIC_SCRATCH_BYTES
        # poisoned outputs: every element has to be written by the call
        dq, dk, dv = (torch.full_like(q, float("nan")) for _ in range(3))
        stream = torch.cuda.current_stream(dev).cuda_stream
        torch.cuda.synchronize()
        free_before, allocated_before = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev)
        st = lib.dsdpa_backward_static_scratch(ctypes.byref(prob), _ptr(q), _ptr(k), _ptr(v), _ptr(coords),
                                               _ptr(out), _ptr(lse), _ptr(dout), _ptr(dq), _ptr(dk), _ptr(dv),
                                               0, ctypes.c_void_p(stream))
        cabi.check(st)
        torch.cuda.synchronize()
        if call > 0:
            # (the first call on a device may make the driver place the library's image)
            assert torch.cuda.mem_get_info(dev)[0] == free_before
            assert torch.cuda.memory_allocated(dev) == allocated_before
        cabi.check(lib.dsdpa_device_error(0))
        o_dq, o_dk, o_dv, _ = oracle.backward(q.float().cpu(), k.float().cpu(), v.float().cpu(), coords.cpu(),
                                              dout.float().cpu(), W, H, sm_scale)
        tol = TOL[dtype]
        for name, got, ref, orc in (("dq", dq, ref_dq, o_dq), ("dk", dk, ref_dk, o_dk), ("dv", dv, ref_dv, o_dv)):
            assert torch.isfinite(got.float()).all(), (call, name)
            assert torch.equal(got, ref), (call, name, rel_err(got, ref))
            assert rel_err(got, orc) < tol, (call, name, rel_err(got, orc))


def test_static_scratch_backward_refuses_what_does_not_fit():
    """Needs no GPU: the size check answers before any CUDA call."""
    import ops
    cabi = ops.backend.cabi
    lib = cabi.lib()
    big = cabi.Problem(32, 8, 16, 28, 28, 64, 32, 0.125, cabi.BF16, 0)   # several GB of scratch
    assert lib.dsdpa_backward_workspace_bytes(ctypes.byref(big)) > cabi.STATIC_SCRATCH_BYTES
    ok = ctypes.c_void_p(4096)
    st = lib.dsdpa_backward_static_scratch(ctypes.byref(big), *([ok] * 10), 0, None)
    assert st == cabi.ERR_TOO_LARGE
    assert "maximum" in cabi.status_string(st)
    assert lib.dsdpa_backward_static_scratch(None, *([ok] * 10), 0, None) == cabi.ERR_NULL_POINTER

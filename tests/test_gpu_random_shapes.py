"""Seeded random small problems against the CPU oracle: every storage type and head dimension,
odd map shapes (single rows and columns included), one to several views, heads and samples,
coordinates that reach outside the map, every backward form, and the coordinate gradient where the
form has one.  The reference has no tests of its own for this path; these cover the shapes its
asserts admit (ops/triton.py:385-388) beyond the named configurations."""
import random

import pytest
import torch

from conftest import TOL, rel_err

pytestmark = pytest.mark.gpu

FLAGS = {"two_pass": 0x0, "maps_from_l2": 0x1, "scatter": 0x8, "scatter_global": 0x4}


def _cases(n=36, seed=2024):
    rng = random.Random(seed)
    out = []
    for i in range(n):
        dtype = rng.choice([torch.float32, torch.float32, torch.bfloat16, torch.float16])
        D = rng.choice([32, 64] if dtype == torch.float32 else [16, 32, 64, 128])
        case = dict(B=rng.randint(1, 3), V=rng.randint(1, 4), Hh=rng.randint(1, 3), W=rng.randint(1, 12),
                    H=rng.randint(1, 12), D=D, S=rng.randint(1, 9), dtype=dtype,
                    lo=rng.choice([0.0, -0.3, -1.5]), hi=rng.choice([1.0, 1.3, 2.5]),
                    flags=rng.choice(list(FLAGS)), seed=1000 + i)
        out.append(case)
    return out


def _id(c):
    return (f"{c['flags']}-{str(c['dtype']).split('.')[-1]}-B{c['B']}V{c['V']}h{c['Hh']}-{c['W']}x{c['H']}"
            f"-D{c['D']}S{c['S']}")


@pytest.mark.parametrize("case", _cases(), ids=_id)
def test_random_problem_matches_the_oracle(case, oracle):
    import ops
    be = ops.backend
    g = torch.Generator().manual_seed(case["seed"])
    B, V, Hh, W, H, D, S = (case[k] for k in ("B", "V", "Hh", "W", "H", "D", "S"))
    L = W * H
    dt = case["dtype"]
    q, k, v, dout = (torch.randn(B, V, Hh, L, D, generator=g).to(dt) for _ in range(4))
    coords = torch.rand(B, V, L, V, S, 2, generator=g) * (case["hi"] - case["lo"]) + case["lo"]
    sm_scale = D ** -0.5
    flags = FLAGS[case["flags"]]
    dev = torch.device("cuda", 0)
    qd, kd, vd, dd, cd = (t.to(dev) for t in (q, k, v, dout, coords))
    out, lse = be.forward_raw(qd, kd, vd, cd, W, H, sm_scale, flags=flags)
    want_dc = case["flags"] in ("two_pass", "maps_from_l2")
    dq, dk, dv, dc = be.backward_raw(qd, kd, vd, cd, out, lse, dd, W, H, sm_scale, flags=flags, want_dcoords=want_dc)
    torch.cuda.synchronize()
    o_ref, lse_ref = oracle.forward(q, k, v, coords, W, H, sm_scale)
    dq_ref, dk_ref, dv_ref, dc_ref = oracle.backward(q, k, v, coords, dout, W, H, sm_scale, with_dcoords=True)
    tol = TOL[dt]
    errs = dict(out=rel_err(out, o_ref), lse=rel_err(lse, lse_ref), dq=rel_err(dq, dq_ref), dk=rel_err(dk, dk_ref),
                dv=rel_err(dv, dv_ref))
    if want_dc:
        errs["dcoords"] = rel_err(dc, dc_ref)
    for name, e in errs.items():
        assert e < tol, (name, e, case)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_every_sample_at_the_same_place(dtype, oracle):
    """All coordinates equal: one anchor per map row collects every sample of a tile, so its list
    is longer than the work list's length buckets distinguish (576 entries) and all but two groups
    of lanes of the gather pass have nothing to do.  Also the other extreme in the same map:
    coordinates exactly on a pixel, where three of the four corner weights are zero."""
    import ops
    be = ops.backend
    B, V, Hh, W, H, D, S = 1, 2, 2, 6, 6, 32, 16
    L = W * H
    g = torch.Generator().manual_seed(77)
    q, k, v, dout = (torch.randn(B, V, Hh, L, D, generator=g).to(dtype) for _ in range(4))
    dev = torch.device("cuda", 0)
    for point in ((0.37, 0.61), (0.4, 0.8)):          # between pixels; exactly pixel (2, 4) of a 6x6 map
        coords = torch.tensor(point).expand(B, V, L, V, S, 2).contiguous()
        qd, kd, vd, dd, cd = (t.to(dev) for t in (q, k, v, dout, coords))
        out, lse = be.forward_raw(qd, kd, vd, cd, W, H, 0.3)
        dq, dk, dv, dc = be.backward_raw(qd, kd, vd, cd, out, lse, dd, W, H, 0.3, want_dcoords=True)
        torch.cuda.synchronize()
        o_ref, _ = oracle.forward(q, k, v, coords, W, H, 0.3)
        dq_ref, dk_ref, dv_ref, dc_ref = oracle.backward(q, k, v, coords, dout, W, H, 0.3, with_dcoords=True)
        tol = TOL[dtype]
        for name, got, ref in (("out", out, o_ref), ("dq", dq, dq_ref), ("dk", dk, dk_ref), ("dv", dv, dv_ref),
                               ("dcoords", dc, dc_ref)):
            assert rel_err(got, ref) < tol, (name, point, rel_err(got, ref))

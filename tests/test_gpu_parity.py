"""Parity of the CUDA path (through the C ABI) with the reference.

Golden cases compare against outputs of the reference's own ops/torch.py committed
under tests/golden; the configuration cases compare against the CPU oracle on the same
seeded inputs.  Tolerances are the ones stated for the path: 1e-4 (max-norm relative)
for fp32 storage, 2e-2 for 16-bit storage with fp32 accumulation.
"""
import ctypes

import pytest
import torch

from conftest import TOL, golden_names, load_golden, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    import ops
    return ops.backend


def _run(backend, case_or_tensors, flags, dtype, W, H, sm_scale):
    q, k, v, coords, dout = case_or_tensors
    dev = torch.device("cuda", 0)
    qd, kd, vd = (t.to(dev, dtype) for t in (q, k, v))
    cd, dd = coords.to(dev), dout.to(dev, dtype)
    out, lse = backend.forward_raw(qd, kd, vd, cd, W, H, sm_scale, flags=flags)
    dq, dk, dv, _ = backend.backward_raw(qd, kd, vd, cd, out, lse, dd, W, H, sm_scale, flags=flags)
    torch.cuda.synchronize()
    backend.cabi.check(backend.cabi.lib().dsdpa_device_error(0))
    return out, lse, dq, dk, dv


FLAG_SETS = {
    "default": 0,                 # two-pass backward where the shape allows it
    "maps_from_l2": 0x1,
    "deterministic": 0x2,
    "scatter": 0x8,               # one-kernel scatter, shared-memory privatised where it fits
    "scatter_global": 0x4,        # one-kernel scatter, reductions straight to global memory
    "scatter_maps_from_l2": 0x9,
}


@pytest.mark.parametrize("flagname", list(FLAG_SETS))
@pytest.mark.parametrize("name", golden_names())
def test_golden_vectors(backend, name, flagname):
    c = load_golden(name)
    dt = c["dtype"]
    out, lse, dq, dk, dv = _run(backend, (c["q"], c["k"], c["v"], c["coords"], c["dout"]), FLAG_SETS[flagname],
                                dt, c["W"], c["H"], c["sm_scale"])
    tol = TOL[dt]
    assert out.dtype == dt and dq.dtype == dt and dk.dtype == dt and dv.dtype == dt
    assert rel_err(out, c["out"]) < tol
    assert rel_err(dq, c["dq"]) < tol
    assert rel_err(dk, c["dk"]) < tol
    assert rel_err(dv, c["dv"]) < tol
    assert torch.isfinite(lse).all()


def test_autograd_function_matches_golden(backend):
    from ops.triton import deform_sdpa_triton
    c = load_golden("oob_f32")
    dev = torch.device("cuda", 0)
    q, k, v = (c[n].to(dev).requires_grad_(True) for n in ("q", "k", "v"))
    out = deform_sdpa_triton(q, k, v, c["coords"].to(dev), c["W"], c["H"], c["sm_scale"])
    out.backward(c["dout"].to(dev))
    assert rel_err(out, c["out"]) < 1e-4
    assert rel_err(q.grad, c["dq"]) < 1e-4
    assert rel_err(k.grad, c["dk"]) < 1e-4
    assert rel_err(v.grad, c["dv"]) < 1e-4


# name -> overrides that shrink the configuration to what the oracle finishes in seconds
CONFIG_CASES = {
    "C1": {},
    "C2": {},
    "C3": dict(B=1, Hh=2),
    "C4": dict(B=1, Hh=2),
    "C5": dict(B=1, Hh=2),
}


@pytest.mark.parametrize("cfgname", list(CONFIG_CASES))
def test_configs_against_oracle(backend, oracle, cfgname):
    from dataclasses import replace
    cfg = replace(backend.inputs.CONFIGS[cfgname], **CONFIG_CASES[cfgname])
    q, k, v, coords, dout = backend.inputs.make_inputs(cfg)
    out, lse, dq, dk, dv = _run(backend, (q, k, v, coords, dout), 0, cfg.dtype, cfg.W, cfg.H, cfg.sm_scale)
    o_ref, lse_ref = oracle.forward(q, k, v, coords, cfg.W, cfg.H, cfg.sm_scale)
    dq_ref, dk_ref, dv_ref, _ = oracle.backward(q, k, v, coords, dout, cfg.W, cfg.H, cfg.sm_scale)
    tol = TOL[cfg.dtype]
    errs = dict(out=rel_err(out, o_ref), dq=rel_err(dq, dq_ref), dk=rel_err(dk, dk_ref), dv=rel_err(dv, dv_ref),
                lse=rel_err(lse, lse_ref))
    print(cfgname, {n: f"{e:.2e}" for n, e in errs.items()})
    for n, e in errs.items():
        assert e < tol, (n, e)


def test_two_pass_backward_is_bit_reproducible(backend):
    """The two-pass dK/dV sums every pixel's contributions in a fixed order: two runs on the
    same inputs agree bit for bit (the scatter forms, built on floating-point atomics, do not
    promise that)."""
    cfg = backend.inputs.CONFIGS["C2"]
    q, k, v, coords, dout = backend.inputs.make_inputs(cfg)
    a = _run(backend, (q, k, v, coords, dout), 0x2, cfg.dtype, cfg.W, cfg.H, cfg.sm_scale)
    b = _run(backend, (q, k, v, coords, dout), 0x2, cfg.dtype, cfg.W, cfg.H, cfg.sm_scale)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("flagname", ["default", "maps_from_l2"])
@pytest.mark.parametrize("name", golden_names())
def test_coordinate_gradient_matches_reference(backend, name, flagname):
    """The reference's Triton operator returns no gradient for coords (ops/triton.py:464); its
    PyTorch path does, through grid_sample.  The golden vectors hold that gradient."""
    c = load_golden(name)
    dt = c["dtype"]
    dev = torch.device("cuda", 0)
    q, k, v, dout = (c[n].to(dev, dt) for n in ("q", "k", "v", "dout"))
    coords = c["coords"].to(dev)
    flags = FLAG_SETS[flagname]
    out, lse = backend.forward_raw(q, k, v, coords, c["W"], c["H"], c["sm_scale"], flags=flags)
    dq, dk, dv, dc = backend.backward_raw(q, k, v, coords, out, lse, dout, c["W"], c["H"], c["sm_scale"],
                                          flags=flags, want_dcoords=True)
    torch.cuda.synchronize()
    tol = TOL[dt]
    assert dc.dtype == torch.float32 and dc.shape == coords.shape
    assert rel_err(dc, c["dcoords"]) < tol
    # asking for the coordinate gradient does not change the others
    assert rel_err(dq, c["dq"]) < tol and rel_err(dk, c["dk"]) < tol and rel_err(dv, c["dv"]) < tol


def test_autograd_returns_coordinate_gradient(backend):
    from ops.triton import deform_sdpa_triton
    c = load_golden("clustered_f32")
    dev = torch.device("cuda", 0)
    q, k, v = (c[n].to(dev).requires_grad_(True) for n in ("q", "k", "v"))
    coords = c["coords"].to(dev).requires_grad_(True)
    out = deform_sdpa_triton(q, k, v, coords, c["W"], c["H"], c["sm_scale"])
    out.backward(c["dout"].to(dev))
    assert coords.grad is not None
    assert rel_err(coords.grad, c["dcoords"]) < 1e-4
    assert rel_err(q.grad, c["dq"]) < 1e-4


def test_coordinate_gradient_needs_the_two_pass_form(backend):
    c = load_golden("tiny_f32_uniform")
    dev = torch.device("cuda", 0)
    q, k, v, dout = (c[n].to(dev) for n in ("q", "k", "v", "dout"))
    coords = c["coords"].to(dev)
    out, lse = backend.forward_raw(q, k, v, coords, c["W"], c["H"], c["sm_scale"])
    with pytest.raises(ValueError):
        backend.backward_raw(q, k, v, coords, out, lse, dout, c["W"], c["H"], c["sm_scale"], flags=0x8,
                             want_dcoords=True)


@pytest.mark.parametrize("cfgname", ["C2", "C3", "C4", "C5"])
def test_coordinate_gradient_on_configs_against_oracle(backend, oracle, cfgname):
    from dataclasses import replace
    cfg = replace(backend.inputs.CONFIGS[cfgname], B=1, Hh=2)
    q, k, v, coords, dout = backend.inputs.make_inputs(cfg)
    dev = torch.device("cuda", 0)
    qd, kd, vd, dd = (t.to(dev) for t in (q, k, v, dout))
    cd = coords.to(dev)
    out, lse = backend.forward_raw(qd, kd, vd, cd, cfg.W, cfg.H, cfg.sm_scale)
    _, _, _, dc = backend.backward_raw(qd, kd, vd, cd, out, lse, dd, cfg.W, cfg.H, cfg.sm_scale, want_dcoords=True)
    _, _, _, dc_ref = oracle.backward(q, k, v, coords, dout, cfg.W, cfg.H, cfg.sm_scale, with_dcoords=True)
    # for 16-bit storage delta = out.dout uses the rounded out, as in the reference
    assert rel_err(dc, dc_ref) < TOL[cfg.dtype]


@pytest.mark.parametrize("flagname", ["scatter", "scatter_global"])
def test_scatter_forms_agree_run_to_run_up_to_rounding(backend, flagname):
    """The scatter forms add with floating-point atomics, in whatever order the hardware
    serves them: two runs may differ, but only by the rounding of fp32 sums of a few hundred
    O(1) terms; dq, which no atomic touches, is identical."""
    cfg = backend.inputs.CONFIGS["C2"]
    data = backend.inputs.make_inputs(cfg)
    a = _run(backend, data, FLAG_SETS[flagname], cfg.dtype, cfg.W, cfg.H, cfg.sm_scale)
    b = _run(backend, data, FLAG_SETS[flagname], cfg.dtype, cfg.W, cfg.H, cfg.sm_scale)
    assert torch.equal(a[0], b[0]) and torch.equal(a[2], b[2])       # out, dq
    for x, y in zip(a[3:], b[3:]):                                    # dk, dv
        assert rel_err(x, y) < 2e-6


@pytest.mark.parametrize("results", ["pinned", "pinned_direct", "pageable"])
def test_host_pipeline_equals_one_shot_call(backend, results):
    """The chunked host-buffer front end gives exactly what the device call gives, whether the
    kernels store the results into pinned host memory themselves or they are copied out."""
    from dataclasses import replace
    cfg = replace(backend.inputs.CONFIGS["C2"], B=5)
    q, k, v, coords, dout = backend.inputs.make_inputs(cfg, pin=True)
    dev = torch.device("cuda", 0)
    ref = _run(backend, (q, k, v, coords, dout), 0, cfg.dtype, cfg.W, cfg.H, cfg.sm_scale)
    out, dq, dk, dv = (torch.zeros_like(q) for _ in range(4))
    if results != "pageable":
        out, dq, dk, dv = (t.pin_memory() for t in (out, dq, dk, dv))
    pipe = backend.HostPipeline(dev, cfg.W, cfg.H, cfg.sm_scale, chunk=2, direct_results=results == "pinned_direct")
    pipe.run(q, k, v, coords, dout, out=out, dq=dq, dk=dk, dv=dv)
    torch.cuda.synchronize()
    assert torch.equal(out, ref[0].cpu())
    assert torch.equal(dq, ref[2].cpu()) and torch.equal(dk, ref[3].cpu()) and torch.equal(dv, ref[4].cpu())


def test_host_pipeline_with_given_chunk_sizes(backend):
    """Explicit chunk sizes give the same bits; sizes that do not cover the batch are refused; the
    transfer rates of a timed run are reported."""
    from dataclasses import replace
    cfg = replace(backend.inputs.CONFIGS["C2"], B=5)
    q, k, v, coords, dout = backend.inputs.make_inputs(cfg, pin=True)
    dev = torch.device("cuda", 0)
    ref = _run(backend, (q, k, v, coords, dout), 0, cfg.dtype, cfg.W, cfg.H, cfg.sm_scale)
    out, dq, dk, dv = (torch.zeros_like(q).pin_memory() for _ in range(4))
    pipe = backend.HostPipeline(dev, cfg.W, cfg.H, cfg.sm_scale, sizes=[2, 3])
    pipe.time_transfers = True
    pipe.run(q, k, v, coords, dout, out=out, dq=dq, dk=dk, dv=dv)
    torch.cuda.synchronize()
    assert torch.equal(out, ref[0].cpu()) and torch.equal(dk, ref[3].cpu()) and torch.equal(dv, ref[4].cpu())
    rates = pipe.transfer_rates()
    assert rates["h2d_GBps"] > 0 and rates["d2h_GBps"] > 0
    with pytest.raises(ValueError):
        backend.HostPipeline(dev, cfg.W, cfg.H, cfg.sm_scale, sizes=[2, 2]).run(q, k, v, coords, dout, out=out, dq=dq,
                                                                               dk=dk, dv=dv)


@pytest.mark.parametrize("B,parts,results", [(5, 2, "pinned"), (1, 3, "pinned"), (2, 4, "pageable"), (3, 2, "pinned_direct")])
def test_host_pipeline_with_head_groups_at_both_ends(backend, B, parts, results):
    """The first and the last batch element cut into groups of heads (uneven ones too, a batch of
    one where both ends are the same element): the same bits as the one-shot call.  With direct
    result stores the cut is not made."""
    from dataclasses import replace
    cfg = replace(backend.inputs.CONFIGS["C2"], B=B, Hh=5)
    q, k, v, coords, dout = backend.inputs.make_inputs(cfg, pin=True)
    dev = torch.device("cuda", 0)
    ref = _run(backend, (q, k, v, coords, dout), 0, cfg.dtype, cfg.W, cfg.H, cfg.sm_scale)
    out, dq, dk, dv = (torch.zeros_like(q) for _ in range(4))
    if results != "pageable":
        out, dq, dk, dv = (t.pin_memory() for t in (out, dq, dk, dv))
    pipe = backend.HostPipeline(dev, cfg.W, cfg.H, cfg.sm_scale, head_parts=parts,
                                direct_results=results == "pinned_direct")
    chunks = pipe.schedule(B, cfg.Hh)
    if results == "pinned_direct":
        assert all(h0 == 0 and h1 == cfg.Hh for _, _, h0, h1 in chunks)
    else:
        assert sum(1 for c in chunks if (c[2], c[3]) != (0, cfg.Hh)) == (parts if B == 1 else 2 * parts)
    pipe.run(q, k, v, coords, dout, out=out, dq=dq, dk=dk, dv=dv)
    torch.cuda.synchronize()
    assert torch.equal(out, ref[0].cpu())
    assert torch.equal(dq, ref[2].cpu()) and torch.equal(dk, ref[3].cpu()) and torch.equal(dv, ref[4].cpu())


def test_link_probe_feeds_a_weighted_plan(backend):
    """The host-link probe returns two positive rates, and a plan weighted by them covers the
    batch with contiguous shards (one GPU: one rank's figures stand in for several)."""
    h2d, d2h = backend.host.measure_link(torch.device("cuda", 0), nbytes=8 << 20, reps=2)
    assert h2d > 0.1 and d2h > 0.1
    weights = backend.host.balance_weights([(h2d, d2h), (h2d / 2, d2h / 2), (h2d, d2h)], 64.2e6, 51.4e6, 0.01)
    plan = backend.partition.shard_plan(12, 4, 3, weights=weights)
    sizes = [s.b1 - s.b0 for s in plan]
    assert sum(sizes) == 12 and sizes[1] < sizes[0] == sizes[2]
    assert [s.b0 for s in plan] == [0, sizes[0], sizes[0] + sizes[1]]


EDGE_CASES = [
    # B, V, Hh, W, H, D, S, dtype, coords range
    (1, 2, 1, 5, 3, 256, 3, torch.float32, (-0.2, 1.2)),     # widest head dim, fp32: 32 lanes x 2 vectors per row
    (1, 2, 2, 4, 4, 256, 5, torch.bfloat16, (0.0, 1.0)),
    (2, 1, 3, 1, 1, 32, 4, torch.float32, (-0.5, 1.5)),      # a single pixel, a single view
    (1, 3, 2, 1, 7, 16, 1, torch.float16, (0.0, 1.0)),       # one column, one sample per view, narrowest rows
    (1, 2, 1, 33, 31, 64, 9, torch.bfloat16, (0.0, 1.0)),    # odd everything, several gather tiles
    (3, 2, 5, 6, 6, 128, 2, torch.float16, (-0.1, 1.1)),
]


@pytest.mark.parametrize("flagname", ["default", "maps_from_l2", "scatter"])
@pytest.mark.parametrize("case", EDGE_CASES, ids=lambda c: f"B{c[0]}V{c[1]}h{c[2]}_{c[3]}x{c[4]}_D{c[5]}S{c[6]}_{str(c[7])[6:]}")
def test_edge_shapes_against_oracle(backend, oracle, case, flagname):
    B, V, Hh, W, H, D, S, dt, (lo, hi) = case
    g = torch.Generator().manual_seed(B * 1000 + D + S)
    L = W * H
    q, k, v, dout = (torch.randn(B, V, Hh, L, D, generator=g).to(dt) for _ in range(4))
    coords = torch.rand(B, V, L, V, S, 2, generator=g) * (hi - lo) + lo
    sm = D ** -0.5
    out, lse, dq, dk, dv = _run(backend, (q, k, v, coords, dout), FLAG_SETS[flagname], dt, W, H, sm)
    o_ref, _ = oracle.forward(q, k, v, coords, W, H, sm)
    dq_ref, dk_ref, dv_ref, _ = oracle.backward(q, k, v, coords, dout, W, H, sm)
    tol = TOL[dt]
    assert rel_err(out, o_ref) < tol
    assert rel_err(dq, dq_ref) < tol and rel_err(dk, dk_ref) < tol and rel_err(dv, dv_ref) < tol


def test_non_contiguous_inputs_are_accepted(backend):
    """The reference's forward takes arbitrary strides (ops/triton.py:400-403); here they are
    made contiguous on the way in."""
    from ops.triton import deform_sdpa_triton
    c = load_golden("oob_f32")
    dev = torch.device("cuda", 0)
    # build q with the head and view axes swapped in memory
    q = c["q"].to(dev).transpose(1, 2).contiguous().transpose(1, 2)
    assert not q.is_contiguous()
    coords64 = c["coords"].to(dev).double()          # any float dtype is accepted for coords
    out = deform_sdpa_triton(q, c["k"].to(dev), c["v"].to(dev), coords64, c["W"], c["H"], c["sm_scale"])
    assert rel_err(out, c["out"]) < 1e-4


def test_large_map_runs_the_two_pass_backward_with_fewer_histograms(backend, oracle):
    """A map of 8000 pixels does not leave the index builder room for eight histograms: it
    builds the same lists with fewer, and the two-pass form (coordinate gradient included) runs."""
    B, V, Hh, W, H, D, S = 1, 2, 1, 100, 80, 16, 2
    g = torch.Generator().manual_seed(5)
    L = W * H
    q, k, v, dout = (torch.randn(B, V, Hh, L, D, generator=g) for _ in range(4))
    coords = torch.rand(B, V, L, V, S, 2, generator=g) * 1.1 - 0.05
    text = backend.cabi.describe_plan(backend.cabi.Problem(B, V, Hh, W, H, D, S, 0.25, backend.cabi.F32, 0))
    assert "bwd_pass_a[" in text and "bwd_gather" in text
    out, lse, dq, dk, dv = _run(backend, (q, k, v, coords, dout), 0, torch.float32, W, H, 0.25)
    o_ref, _ = oracle.forward(q, k, v, coords, W, H, 0.25)
    dq_ref, dk_ref, dv_ref, dc_ref = oracle.backward(q, k, v, coords, dout, W, H, 0.25, with_dcoords=True)
    assert rel_err(out, o_ref) < 1e-4 and rel_err(dq, dq_ref) < 1e-4
    assert rel_err(dk, dk_ref) < 1e-4 and rel_err(dv, dv_ref) < 1e-4
    dev = torch.device("cuda", 0)
    *_, dc = backend.backward_raw(q.to(dev), k.to(dev), v.to(dev), coords.to(dev), out, lse, dout.to(dev), W, H, 0.25,
                                  want_dcoords=True)
    assert rel_err(dc, dc_ref) < 1e-4


def test_huge_map_falls_back_to_the_scatter_backward(backend, oracle):
    """A map whose anchors do not fit even one histogram in shared memory (here 250x240) runs
    the scatter form by itself.  That form has no coordinate gradient: the C ABI refuses one,
    and the autograd function returns None for coords, as the reference does
    (ops/triton.py:464), with a warning."""
    B, V, Hh, W, H, D, S = 1, 1, 1, 250, 240, 16, 2
    g = torch.Generator().manual_seed(6)
    L = W * H
    q, k, v, dout = (torch.randn(B, V, Hh, L, D, generator=g) for _ in range(4))
    coords = torch.rand(B, V, L, V, S, 2, generator=g) * 1.1 - 0.05
    prob = backend.cabi.Problem(B, V, Hh, W, H, D, S, 0.25, backend.cabi.F32, 0)
    text = backend.cabi.describe_plan(prob)
    assert "bwd_scatter[" in text and "bwd_gather" not in text
    assert backend.cabi.lib().dsdpa_backward_supports_dcoords(ctypes.byref(prob)) == 0
    out, lse, dq, dk, dv = _run(backend, (q, k, v, coords, dout), 0, torch.float32, W, H, 0.25)
    o_ref, _ = oracle.forward(q, k, v, coords, W, H, 0.25)
    dq_ref, dk_ref, dv_ref, _ = oracle.backward(q, k, v, coords, dout, W, H, 0.25)
    assert rel_err(out, o_ref) < 1e-4 and rel_err(dq, dq_ref) < 1e-4
    assert rel_err(dk, dk_ref) < 1e-4 and rel_err(dv, dv_ref) < 1e-4
    dev = torch.device("cuda", 0)
    with pytest.raises(ValueError):
        backend.backward_raw(q.to(dev), k.to(dev), v.to(dev), coords.to(dev), out, lse, dout.to(dev), W, H, 0.25,
                             want_dcoords=True)
    # through autograd a training step still runs: coords get no gradient
    from ops.triton import deform_sdpa_triton
    qd, kd, vd, cd = (t.to(dev).requires_grad_(True) for t in (q, k, v, coords))
    with pytest.warns(UserWarning, match="coordinate gradient"):
        deform_sdpa_triton(qd, kd, vd, cd, W, H, 0.25).backward(dout.to(dev))
    assert cd.grad is None and rel_err(qd.grad, dq_ref) < 1e-4 and rel_err(kd.grad, dk_ref) < 1e-4


@pytest.mark.parametrize("flagname", ["default", "scatter", "scatter_global"])
@pytest.mark.parametrize("name", ["oob_f32", "bf16_d64_clustered", "d16_f16", "d128_f32"])
def test_mirrors_receive_the_same_bits(backend, name, flagname):
    """The mirrored entry points store every result a second time (the destination a sharded
    job gathers into): the copies equal the results bit for bit, results are unchanged by the
    presence of mirrors, and a missing mirror is simply not written."""
    c = load_golden(name)
    dt, flags = c["dtype"], FLAG_SETS[flagname]
    dev = torch.device("cuda", 0)
    q, k, v, dout = (c[n].to(dev, dt) for n in ("q", "k", "v", "dout"))
    coords = c["coords"].to(dev)
    args = (c["W"], c["H"], c["sm_scale"])
    out0, lse0 = backend.forward_raw(q, k, v, coords, *args, flags=flags)
    m_out = torch.full_like(out0, 7.0)
    out1, lse1 = backend.forward_raw(q, k, v, coords, *args, flags=flags, out_mirror=m_out)
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1) and torch.equal(m_out, out0)

    mir = {n: torch.full_like(out0, 7.0) for n in ("out", "dq", "dk", "dv")}
    dq, dk, dv, _ = backend.backward_raw(q, k, v, coords, out0, lse0, dout, *args, flags=flags, mirrors=mir)
    torch.cuda.synchronize()
    backend.cabi.check(backend.cabi.lib().dsdpa_device_error(0))
    assert torch.equal(mir["out"], out0)
    assert torch.equal(mir["dq"], dq) and torch.equal(mir["dk"], dk) and torch.equal(mir["dv"], dv)
    tol = TOL[dt]
    assert rel_err(dq, c["dq"]) < tol and rel_err(dk, c["dk"]) < tol and rel_err(dv, c["dv"]) < tol

    # a subset of mirrors: the others stay untouched
    only = {"dk": torch.full_like(out0, 7.0)}
    _, dk2, _, _ = backend.backward_raw(q, k, v, coords, out0, lse0, dout, *args, flags=flags, mirrors=only)
    if flagname == "default":   # (the scatter forms sum with atomics: not bit-reproducible)
        assert torch.equal(only["dk"], dk) and torch.equal(dk2, dk)
    else:
        assert torch.equal(only["dk"], dk2)


def test_mirror_arguments_are_checked(backend):
    c = load_golden("tiny_f32_uniform")
    dev = torch.device("cuda", 0)
    q, k, v = (c[n].to(dev) for n in ("q", "k", "v"))
    coords = c["coords"].to(dev)
    with pytest.raises(ValueError):
        backend.forward_raw(q, k, v, coords, c["W"], c["H"], c["sm_scale"], out_mirror=torch.empty_like(q)[..., :8])
    out, lse = backend.forward_raw(q, k, v, coords, c["W"], c["H"], c["sm_scale"])
    with pytest.raises(ValueError):
        backend.backward_raw(q, k, v, coords, out, lse, c["dout"].to(dev), c["W"], c["H"], c["sm_scale"],
                             mirrors={"dz": torch.empty_like(q)})


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs with peer access")
def test_mirrors_in_another_gpus_memory(backend):
    """Mirrors that lie on a second GPU: the library switches peer access on before it launches,
    and the kernels' plain stores land there (the path a sharded job's gather takes)."""
    if not torch.cuda.can_device_access_peer(0, 1):
        pytest.skip("GPU 0 cannot reach GPU 1")
    c = load_golden("bf16_d64_clustered")
    dt = c["dtype"]
    d0, d1 = torch.device("cuda", 0), torch.device("cuda", 1)
    q, k, v, dout = (c[n].to(d0, dt) for n in ("q", "k", "v", "dout"))
    coords = c["coords"].to(d0)
    args = (c["W"], c["H"], c["sm_scale"])
    m_out = torch.zeros(q.shape, dtype=dt, device=d1)
    out, lse = backend.forward_raw(q, k, v, coords, *args, out_mirror=m_out)
    mir = {n: torch.zeros(q.shape, dtype=dt, device=d1) for n in ("out", "dq", "dk", "dv")}
    dq, dk, dv, _ = backend.backward_raw(q, k, v, coords, out, lse, dout, *args, mirrors=mir)
    torch.cuda.synchronize(d0)
    backend.cabi.check(backend.cabi.lib().dsdpa_device_error(0))
    assert torch.equal(m_out.to(d0), out) and torch.equal(mir["out"].to(d0), out)
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert torch.equal(mir[n].to(d0), t), n


def test_a_mirror_the_device_cannot_store_to_is_refused(backend):
    """A mirror in memory CUDA does not know (pageable host memory) is refused with a status
    before anything is launched; the results of the call are not produced."""
    import ctypes
    import numpy as np
    cabi = backend.cabi
    c = load_golden("tiny_f32_uniform")
    dev = torch.device("cuda", 0)
    q, k, v = (c[n].to(dev) for n in ("q", "k", "v"))
    coords = c["coords"].to(dev)
    B, V, Hh, L, D = q.shape
    prob = cabi.Problem(B, V, Hh, c["W"], c["H"], D, coords.shape[4], c["sm_scale"], cabi.F32, 0)
    out = torch.zeros_like(q)
    lse = torch.zeros(q.shape[:4], device=dev)
    host = np.zeros(q.numel() + 8, dtype=np.float32)
    addr = (host.ctypes.data + 15) & ~15
    before = cabi.lib().dsdpa_kernel_launches()
    vp = ctypes.c_void_p
    st = cabi.lib().dsdpa_forward_mirrored(ctypes.byref(prob), vp(q.data_ptr()), vp(k.data_ptr()), vp(v.data_ptr()),
                                           vp(coords.data_ptr()), vp(out.data_ptr()), vp(lse.data_ptr()), vp(addr),
                                           0, None)
    assert st == cabi.ERR_PEER_ACCESS
    assert cabi.lib().dsdpa_kernel_launches() == before
    with pytest.raises(cabi.DsdpaError):
        cabi.check(st)
    torch.cuda.synchronize()
    assert not out.any()


@pytest.mark.parametrize("cfgname", ["C2", "C3", "C5"])
def test_mirrors_at_benchmark_shapes(backend, cfgname):
    """Same as above at the benchmark shapes (one batch element): staged and L1/L2 paths, gather
    pass with and without split key pixels."""
    from dataclasses import replace
    cfg = replace(backend.inputs.CONFIGS[cfgname], B=1)
    q, k, v, coords, dout = backend.inputs.make_inputs(cfg)
    dev = torch.device("cuda", 0)
    q, k, v, dout = (t.to(dev, cfg.dtype) for t in (q, k, v, dout))
    coords = coords.to(dev)
    args = (cfg.W, cfg.H, cfg.sm_scale)
    out, lse = backend.forward_raw(q, k, v, coords, *args)
    dq, dk, dv, _ = backend.backward_raw(q, k, v, coords, out, lse, dout, *args)
    mir = {n: torch.zeros_like(q) for n in ("out", "dq", "dk", "dv")}
    m_fwd = torch.zeros_like(q)
    out2, lse2 = backend.forward_raw(q, k, v, coords, *args, out_mirror=m_fwd)
    dq2, dk2, dv2, _ = backend.backward_raw(q, k, v, coords, out2, lse2, dout, *args, mirrors=mir)
    torch.cuda.synchronize()
    backend.cabi.check(backend.cabi.lib().dsdpa_device_error(0))
    assert torch.equal(out, out2) and torch.equal(m_fwd, out) and torch.equal(mir["out"], out)
    for name, a, b in (("dq", dq, dq2), ("dk", dk, dk2), ("dv", dv, dv2)):
        assert torch.equal(a, b), name          # the two-pass backward is deterministic
        assert torch.equal(mir[name], a), name


@pytest.mark.parametrize("name", ["bf16_d64_uniform", "bf16_d64_clustered", "bf16_d32_oob", "d16_f16", "oob_f32"])
@pytest.mark.parametrize("maps", ["staged", "l2"])
def test_rounded_weights_option(backend, oracle, name, maps):
    """DSDPA_FLAG_ROUNDED_WEIGHTS (16-bit storage, forward): the weights that multiply V rows are
    rounded to the storage type.  Still within the storage type's tolerance of the reference and
    of exact arithmetic on the stored inputs; no effect at all on fp32 storage."""
    c = load_golden(name)
    dt = c["dtype"]
    dev = torch.device("cuda", 0)
    q, k, v = (c[n].to(dev, dt) for n in ("q", "k", "v"))
    coords = c["coords"].to(dev)
    args = (c["W"], c["H"], c["sm_scale"])
    base = 0x1 if maps == "l2" else 0
    out0, lse0 = backend.forward_raw(q, k, v, coords, *args, flags=base)
    out1, lse1 = backend.forward_raw(q, k, v, coords, *args, flags=base | backend.cabi.FLAG_ROUNDED_WEIGHTS)
    torch.cuda.synchronize()
    assert torch.equal(lse0, lse1)                      # the logits and the normaliser are untouched
    if dt == torch.float32:
        assert torch.equal(out0, out1)
        return
    exact, _ = oracle.forward(q.float().cpu(), k.float().cpu(), v.float().cpu(), c["coords"], *args)
    assert rel_err(out1, c["out"]) < TOL[dt]
    assert rel_err(out1, exact) < TOL[dt] / 2
    assert rel_err(out0, exact) <= rel_err(out1, exact) * 1.5 + 1e-6   # the default is the more exact one

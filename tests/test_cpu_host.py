"""Host-side checks that need no GPU: the C-ABI library loads and exports what
include/dsdpa.h declares, argument validation answers before any CUDA call, the
planner produces sane launches for the five configurations, and the seeded input
generator is reproducible shard by shard."""
import ctypes
import re
from dataclasses import replace
from pathlib import Path

import pytest
import torch

import ops

ROOT = Path(__file__).resolve().parent.parent
be = ops.backend
cabi = be.cabi


def test_header_symbols_are_exported():
    text = (ROOT / "include" / "dsdpa.h").read_text()
    declared = set(re.findall(r"\b(dsdpa_[a-z0-9_]+)\s*\(", text))
    assert declared, "no declarations found in include/dsdpa.h"
    assert declared == set(cabi.EXPORTS)
    lib = cabi.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert lib.dsdpa_version() == 100


def test_problem_struct_matches_header():
    # ten 4-byte fields, in the header's order
    assert ctypes.sizeof(cabi.Problem) == 40
    assert [f[0] for f in cabi.Problem._fields_] == ["B", "V", "Hh", "W", "H", "D", "S", "sm_scale", "dtype", "flags"]


def _prob(**kw):
    base = dict(B=2, V=3, Hh=2, W=6, H=5, D=32, S=4, sm_scale=0.5, dtype=cabi.F32, flags=0)
    base.update(kw)
    return cabi.Problem(*[base[f[0]] for f in cabi.Problem._fields_])


def _fwd_status(prob, ptrs=(None,) * 6):
    return cabi.lib().dsdpa_forward(ctypes.byref(prob), *ptrs, 0, None)


@pytest.mark.parametrize("kw,status", [
    (dict(dtype=7), cabi.ERR_BAD_DTYPE),
    (dict(D=48), cabi.ERR_BAD_HEAD_DIM),
    (dict(D=8), cabi.ERR_BAD_HEAD_DIM),
    (dict(B=0), cabi.ERR_BAD_SHAPE),
    (dict(S=-1), cabi.ERR_BAD_SHAPE),
    (dict(W=70000, H=70000), cabi.ERR_BAD_SHAPE),
    (dict(flags=0x100), cabi.ERR_BAD_FLAGS),
    (dict(flags=0x2 | 0x8), cabi.ERR_BAD_FLAGS),
    (dict(sm_scale=float("nan")), cabi.ERR_BAD_SHAPE),
])
def test_bad_problems_are_rejected_without_touching_cuda(kw, status):
    assert _fwd_status(_prob(**kw)) == status


def test_null_and_misaligned_pointers():
    p = _prob()
    assert _fwd_status(p) == cabi.ERR_NULL_POINTER
    ok = ctypes.c_void_p(4096)
    bad = ctypes.c_void_p(4096 + 4)
    assert _fwd_status(p, (ok, ok, bad, ok, ok, ok)) == cabi.ERR_MISALIGNED
    lib = cabi.lib()
    # backward: workspace too small for 16-bit storage
    p16 = _prob(dtype=cabi.BF16)
    need = lib.dsdpa_backward_workspace_bytes(ctypes.byref(p16))
    assert need > 0
    st = lib.dsdpa_backward(ctypes.byref(p16), *([ok] * 10), None, ok, need - 1, 0, None)
    assert st == cabi.ERR_WORKSPACE
    st = lib.dsdpa_backward(ctypes.byref(p16), *([ok] * 10), None, None, 0, 0, None)
    assert st == cabi.ERR_WORKSPACE
    assert lib.dsdpa_backward(ctypes.byref(p16), *([None] * 10), None, None, 0, 0, None) == cabi.ERR_NULL_POINTER


def test_status_strings_and_exceptions():
    for st in range(0, 12):
        assert cabi.status_string(st)
    assert cabi.status_string(12345) == "unknown status"
    with pytest.raises(NotImplementedError):
        cabi.check(cabi.ERR_BAD_DTYPE)
    with pytest.raises(ValueError):
        cabi.check(cabi.ERR_BAD_HEAD_DIM)
    with pytest.raises(cabi.DsdpaError):
        cabi.check(cabi.ERR_DEVICE_TIMEOUT)
    cabi.check(cabi.OK)


def test_workspace_is_zero_for_fp32_scatter_and_grows_with_two_pass():
    lib = cabi.lib()
    scatter = _prob(flags=cabi.FLAG_SCATTER)
    assert lib.dsdpa_backward_workspace_bytes(ctypes.byref(scatter)) == 0
    two = _prob(flags=cabi.FLAG_DETERMINISTIC)
    assert lib.dsdpa_backward_workspace_bytes(ctypes.byref(two)) > 0


def test_plans_of_the_five_configurations():
    for name, cfg in be.inputs.CONFIGS.items():
        dt = {torch.float32: cabi.F32, torch.bfloat16: cabi.BF16}[cfg.dtype]
        text = cabi.describe_plan(cabi.Problem(cfg.B, cfg.V, cfg.Hh, cfg.W, cfg.H, cfg.D, cfg.S, cfg.sm_scale, dt, 0))
        m = re.search(r"fwd\[(\w+) nstage=(\d+) nw=(\d+) nq=(\d+) tiles=(\d+) q_per_tile=(\d+) ctas=(\d+) smem=(\d+)\]", text)
        assert m, text
        kind, nstage, nw, nq, tiles, qpt, ctas, smem = m.group(1), *map(int, m.groups()[1:])
        assert smem <= 232448
        assert tiles * qpt >= cfg.V * cfg.L            # every query is covered
        assert ctas == cfg.B * cfg.Hh * tiles
        map_bytes = cfg.L * cfg.D * cfg.elem_size()
        fits = 2 * map_bytes + 4096 + 16 <= 232448
        assert (kind == "staged") == fits, (name, text)
        assert "bwd_gather[" in text
    # forcing the L2 path is honoured
    c1 = be.inputs.CONFIGS["C1"]
    text = cabi.describe_plan(cabi.Problem(c1.B, c1.V, c1.Hh, c1.W, c1.H, c1.D, c1.S, 0.5, cabi.F32, cabi.FLAG_MAPS_FROM_L2))
    assert text.startswith("fwd[l2")


def test_backward_form_by_map_size_and_flags():
    """The two-pass form (and with it the coordinate gradient) runs for maps up to the index
    builder's limit -- with fewer histograms for large ones -- and gives way to the scatter form
    beyond it or under the scatter flags; the gather pass's grid is units x slabs."""
    lib = cabi.lib()

    def plan(W, H, flags=0, dtype=cabi.F32, D=16):
        prob = cabi.Problem(1, 2, 1, W, H, D, 2, 0.25, dtype, flags)
        return cabi.describe_plan(prob), lib.dsdpa_backward_supports_dcoords(ctypes.byref(prob))

    for W, H in ((14, 14), (100, 80), (160, 160)):
        text, dc = plan(W, H)
        assert "bwd_pass_a[" in text and "bwd_gather[" in text and dc == 1, (W, H, text)
    text, dc = plan(250, 240)
    assert "bwd_scatter[" in text and "bwd_gather" not in text and dc == 0
    text, dc = plan(14, 14, cabi.FLAG_SCATTER)
    assert "bwd_scatter[" in text and dc == 0
    assert lib.dsdpa_backward_supports_dcoords(None) == 0
    m = re.search(r"bwd_gather\[tpv=(\d+) QB=(\d+) nslab=(\d+) ctas=(\d+) smem=(\d+) segments=(\d+)\]", plan(14, 14)[0])
    tpv, qb, nslab, ctas, smem, segments = map(int, m.groups())
    assert tpv * qb >= 14 * 14 and ctas == 1 * 1 * 2 * nslab and smem <= 232448 and segments == 1 * 2 * tpv * 2
    # 16-bit storage runs the gather pass with fewer threads than fp32 storage: its plan leaves room
    c5 = be.inputs.CONFIGS["C5"]
    t5 = cabi.describe_plan(cabi.Problem(c5.B, c5.V, c5.Hh, c5.W, c5.H, c5.D, c5.S, c5.sm_scale, cabi.BF16, 0))
    assert re.search(r"bwd_gather\[tpv=2 QB=392 ", t5), t5


def test_rounded_weights_flag_is_a_16_bit_forward_option():
    c5 = be.inputs.CONFIGS["C5"]
    args = (c5.B, c5.V, c5.Hh, c5.W, c5.H, c5.D, c5.S, c5.sm_scale)
    text = cabi.describe_plan(cabi.Problem(*args, cabi.BF16, cabi.FLAG_ROUNDED_WEIGHTS))
    assert text.startswith("fwd[staged+rw")
    text = cabi.describe_plan(cabi.Problem(*args, cabi.BF16, cabi.FLAG_ROUNDED_WEIGHTS | cabi.FLAG_MAPS_FROM_L2))
    assert text.startswith("fwd[l2+rw")
    c1 = be.inputs.CONFIGS["C1"]
    text = cabi.describe_plan(cabi.Problem(c1.B, c1.V, c1.Hh, c1.W, c1.H, c1.D, c1.S, 0.5, cabi.F32,
                                           cabi.FLAG_ROUNDED_WEIGHTS))
    assert text.startswith("fwd[staged ")      # accepted, without effect on fp32 storage


def test_operator_refuses_cpu_tensors():
    from ops.triton import deform_sdpa_triton
    q = torch.zeros(1, 1, 1, 4, 16)
    c = torch.zeros(1, 1, 4, 1, 2, 2)
    with pytest.raises(RuntimeError, match="no CPU path"):
        deform_sdpa_triton(q, q, q, c, 2, 2, 1.0)


def test_seeded_inputs_are_shard_invariant():
    cfg = replace(be.inputs.CONFIGS["C2"], B=3)
    full = be.inputs.make_inputs(cfg)
    part = be.inputs.make_inputs(cfg, batch_range=(1, 3))
    for a, b in zip(full, part):
        assert torch.equal(a[1:3], b)
    q, k, v, coords, dout = full
    assert q.shape == (3, cfg.V, cfg.Hh, cfg.L, cfg.D) and coords.shape == (3, cfg.V, cfg.L, cfg.V, cfg.S, 2)
    # C2 draws coordinates from U[-0.1, 1.1): some fall outside the map on purpose
    frac_out = ((coords < 0) | (coords > 1)).any(-1).float().mean().item()
    assert 0.2 < frac_out < 0.4
    c3 = replace(be.inputs.CONFIGS["C3"], B=1, Hh=1)
    coords3 = be.inputs.make_inputs(c3)[3]
    assert coords3.min() >= 0 and coords3.max() <= 1


def test_algorithmic_byte_counts():
    c = be.inputs.CONFIGS
    assert c["C1"].gather_bytes_per_qh() == 262144 and c["C2"].gather_bytes_per_qh() == 98304
    assert c["C3"].gather_bytes_per_qh() == 393216 and c["C4"].gather_bytes_per_qh() == 49152
    assert c["C5"].gather_bytes_per_qh() == 262144
    assert round(c["C1"].hbm_bytes_per_qh()) == 644 and round(c["C1"].hbm_bytes_per_qh(True)) == 1156
    assert round(c["C3"].hbm_bytes_per_qh()) == 900 and round(c["C4"].hbm_bytes_per_qh()) == 564
    assert c["C5"].query_heads == 3211264

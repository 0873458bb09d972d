"""Pins the CPU oracle to the reference: every golden vector under tests/golden was
produced by the reference's ops/torch.py (forward + autograd), and the oracle must
reproduce out, dq, dk, dv and the coordinate gradient on each of them."""
import pytest
import torch

from conftest import golden_names, load_golden, rel_err

# The oracle accumulates in double and takes fp32 inputs, so against the reference's
# fp32 arithmetic it agrees to rounding; 16-bit cases differ by the reference's final
# rounding of its outputs to the storage type.
PIN_TOL = {torch.float32: 5e-6, torch.bfloat16: 8e-3, torch.float16: 1e-3}


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_vectors(oracle, name):
    c = load_golden(name)
    out, lse = oracle.forward(c["q"], c["k"], c["v"], c["coords"], c["W"], c["H"], c["sm_scale"])
    dq, dk, dv, dc = oracle.backward(c["q"], c["k"], c["v"], c["coords"], c["dout"],
                                     c["W"], c["H"], c["sm_scale"], with_dcoords=True)
    tol = PIN_TOL[c["dtype"]]
    assert rel_err(out, c["out"]) < tol
    assert rel_err(dq, c["dq"]) < tol
    assert rel_err(dk, c["dk"]) < tol
    assert rel_err(dv, c["dv"]) < tol
    # the reference keeps coordinates in fp32 whatever the storage type of q/k/v
    assert rel_err(dc, c["dcoords"]) < 2e-5
    assert torch.isfinite(lse).all()


def test_golden_set_is_complete():
    names = golden_names()
    assert len(names) >= 10
    kinds = {str(load_golden(n)["dtype"]) for n in names}
    assert {"torch.float32", "torch.bfloat16"} <= kinds


def test_range_calls_agree_with_whole_call(oracle):
    c = load_golden("oob_f32")
    args = (c["q"], c["k"], c["v"], c["coords"], c["W"], c["H"], c["sm_scale"])
    out, lse = oracle.forward(*args)
    B, V, Hh, L, D = c["q"].shape
    qh = B * V * Hh * L
    a, _ = oracle.forward(*args, qh_range=(0, qh // 3))
    b, _ = oracle.forward(*args, qh_range=(qh // 3, qh))
    assert torch.equal(a + b, out)
    dq, dk, dv, _ = oracle.backward(c["q"], c["k"], c["v"], c["coords"], c["dout"], c["W"], c["H"], c["sm_scale"])
    parts = [oracle.backward(c["q"], c["k"], c["v"], c["coords"], c["dout"], c["W"], c["H"], c["sm_scale"],
                             bh_range=(i, i + 1)) for i in range(B * Hh)]
    assert torch.equal(sum(p[0] for p in parts), dq)
    assert torch.equal(sum(p[1] for p in parts), dk)
    assert torch.equal(sum(p[2] for p in parts), dv)

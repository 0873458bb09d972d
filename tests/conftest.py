"""Shared pytest plumbing: markers, repository paths, golden-vector loading."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def golden_names():
    return sorted(p.stem for p in GOLDEN_DIR.glob("*.npz"))


def load_golden(name):
    """Return the case as a dict of torch tensors (fp32) plus W, H, sm_scale, dtype."""
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    case = {}
    for key in ("q", "k", "v", "coords", "dout", "out", "dq", "dk", "dv", "dcoords"):
        case[key] = torch.from_numpy(z[key].copy())
    case["W"] = int(z["W"])
    case["H"] = int(z["H"])
    case["sm_scale"] = float(z["sm_scale"])
    case["dtype"] = getattr(torch, str(z["dtype"]))
    case["name"] = name
    return case


def rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """max|a - ref| / max|ref|: the norm-relative error every parity test uses
    (an elementwise relative error is meaningless next to zero)."""
    a = a.detach().double().cpu()
    ref = ref.detach().double().cpu()
    denom = ref.abs().max().item()
    if denom == 0.0:
        return (a - ref).abs().max().item()
    return (a - ref).abs().max().item() / denom


# Tolerances stated for the path: 1e-4 relative for fp32 storage, 2e-2 for 16-bit
# storage with fp32 accumulation.
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    orc.build()
    return orc


@pytest.fixture(autouse=True)
def _no_kernel_gave_up(request):
    """After every GPU test: no kernel recorded a timed-out wait or, in the checked build, an
    index out of range.  (Tests that provoke such a record on purpose read it themselves first.)"""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import ops
    cabi = ops.backend.cabi
    cabi.check(cabi.lib().dsdpa_device_error(0))

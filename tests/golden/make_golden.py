"""Generate the golden vectors under tests/golden/ from the REFERENCE implementation.

Run by hand in a container that has the reference checkout (it is not available
where the GPU tests run, which is why the vectors are committed):

    python tests/golden/make_golden.py /path/to/reference

The script imports the reference's pure-PyTorch path (``ops/torch.py``,
``deform_sdpa_torch``) under a private module name, runs it on small seeded inputs
on the CPU, obtains dq/dk/dv (and the coordinate gradient) from autograd, and
writes one ``.npz`` per case with inputs and outputs.  Nothing here is used by the
product; the vectors pin the CPU oracle and the CUDA path to the reference.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference(root: Path):
    spec = importlib.util.spec_from_file_location("_reference_ops_torch", root / "ops" / "torch.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.deform_sdpa_torch


def query_centres(W, H):
    ls = torch.arange(W * H)
    cx = (ls % W).float() / max(W - 1, 1)
    cy = (ls // W).float() / max(H - 1, 1)
    return torch.stack([cx, cy], -1)  # [L, 2]


def make_coords(kind, B, V, L, S, W, H, gen):
    shape = (B, V, L, V, S, 2)
    if kind == "uniform":
        return torch.rand(shape, generator=gen)
    if kind == "oob":
        return torch.rand(shape, generator=gen) * 1.6 - 0.3
    if kind == "far_oob":
        c = torch.rand(shape, generator=gen) * 1.6 - 0.3
        c[..., 0, :] = torch.tensor([-3.0, 0.5])   # far outside on one axis
        c[..., 1 % S, :] = torch.tensor([7.0, 9.0])  # far outside on both: logit 0, value 0
        return c
    if kind == "edges":
        # exact grid points, the two borders, and the middle of cells
        gx = torch.randint(0, W, shape[:-1], generator=gen).float() / max(W - 1, 1)
        gy = torch.randint(0, H, shape[:-1], generator=gen).float() / max(H - 1, 1)
        c = torch.stack([gx, gy], -1)
        c[..., 0, :] = 0.0
        c[..., 1 % S, :] = 1.0
        if S > 2:
            c[..., 2, 0] = 1.0
            c[..., 2, 1] = 0.0
        return c
    if kind == "clustered":
        ctr = query_centres(W, H).view(1, 1, L, 1, 1, 2)
        return (ctr + 0.05 * torch.randn(shape, generator=gen)).clamp(0, 1)
    if kind == "mixed":
        ctr = query_centres(W, H).view(1, 1, L, 1, 1, 2)
        near = (ctr + 0.02 * torch.randn(shape, generator=gen)).clamp(0, 1)
        uni = torch.rand(shape, generator=gen)
        pick = torch.rand(shape[:-1], generator=gen) < 0.5
        return torch.where(pick.unsqueeze(-1), uni, near)
    raise ValueError(kind)


CASES = [
    # name, B, V, Hh, W, H, D, S, sm_scale, dtype, coords kind, seed
    ("tiny_f32_uniform", 1, 2, 2, 5, 4, 16, 3, 0.5, "float32", "uniform", 11),
    ("oob_f32", 2, 3, 2, 6, 5, 32, 5, 32 ** -0.5, "float32", "oob", 12),
    ("far_oob_f32", 1, 2, 2, 4, 4, 32, 4, 0.25, "float32", "far_oob", 13),
    ("edges_f32", 1, 2, 1, 4, 3, 16, 4, 0.5, "float32", "edges", 14),
    ("nonsquare_d64_f32", 1, 2, 2, 9, 3, 64, 4, 0.125, "float32", "mixed", 15),
    ("clustered_f32", 1, 2, 2, 8, 8, 32, 8, 32 ** -0.5, "float32", "clustered", 16),
    ("quickstart_like_f32", 1, 3, 2, 14, 14, 32, 6, 0.5, "float32", "uniform", 17),
    ("bf16_d64_uniform", 1, 2, 2, 7, 7, 64, 8, 0.125, "bfloat16", "uniform", 18),
    ("bf16_d64_clustered", 2, 2, 2, 8, 8, 64, 8, 0.125, "bfloat16", "clustered", 19),
    ("bf16_d32_oob", 1, 3, 2, 6, 5, 32, 5, 32 ** -0.5, "bfloat16", "oob", 20),
    ("single_pixel_row_f32", 1, 2, 1, 6, 1, 16, 3, 0.5, "float32", "oob", 21),
    ("d128_f32", 1, 2, 1, 4, 4, 128, 3, 128 ** -0.5, "float32", "uniform", 22),
    ("d16_f16", 1, 2, 2, 5, 5, 16, 4, 0.25, "float16", "oob", 23),
]


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference>")
    root = Path(sys.argv[1])
    ref = load_reference(root)
    torch.set_num_threads(max(1, torch.get_num_threads()))
    for name, B, V, Hh, W, H, D, S, sm_scale, dtype, kind, seed in CASES:
        gen = torch.Generator().manual_seed(seed)
        L = W * H
        dt = getattr(torch, dtype)
        q = torch.randn(B, V, Hh, L, D, generator=gen).to(dt)
        k = torch.randn(B, V, Hh, L, D, generator=gen).to(dt)
        v = torch.randn(B, V, Hh, L, D, generator=gen).to(dt)
        dout = torch.randn(B, V, Hh, L, D, generator=gen).to(dt)
        coords = make_coords(kind, B, V, L, S, W, H, gen)
        q_, k_, v_ = (t.clone().requires_grad_(True) for t in (q, k, v))
        c_ = coords.clone().requires_grad_(True)
        out = ref(q_, k_, v_, c_, W, H, sm_scale)
        assert out.dtype == dt
        out.backward(dout)
        arrays = dict(
            q=q.float().numpy(), k=k.float().numpy(), v=v.float().numpy(),
            coords=coords.numpy(), dout=dout.float().numpy(),
            out=out.detach().float().numpy(),
            dq=q_.grad.float().numpy(), dk=k_.grad.float().numpy(), dv=v_.grad.float().numpy(),
            dcoords=c_.grad.float().numpy(),
            W=np.int32(W), H=np.int32(H), sm_scale=np.float64(sm_scale),
            dtype=np.array(dtype), coords_kind=np.array(kind),
        )
        np.savez_compressed(HERE / f"{name}.npz", **arrays)
        nbytes = (HERE / f"{name}.npz").stat().st_size
        print(f"{name}: q{tuple(q.shape)} coords{tuple(coords.shape)} -> {nbytes / 1024:.0f} KiB")


if __name__ == "__main__":
    main()

"""The five benchmark shapes and their seeded synthetic inputs.

The reference measures on synthetic ``randn``/``rand`` tensors (reference
benchmark.py:108-114) and never sets a seed; here every batch element has its own
seed, so that any (batch, head) shard of a configuration reproduces exactly the data
the unsharded run sees, whatever the number of GPUs.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import torch


@dataclass(frozen=True)
class Config:
    name: str
    B: int
    V: int      # views
    S: int      # samples per (query, key view)
    Hh: int     # heads
    D: int
    W: int
    H: int
    sm_scale: float
    dtype: torch.dtype
    coords: str  # "uniform" | "oob" | "clustered" | "mixed"
    sigma: float = 0.0

    @property
    def L(self) -> int:
        return self.W * self.H

    @property
    def N(self) -> int:
        return self.V * self.S

    @property
    def query_heads(self) -> int:
        return self.B * self.V * self.Hh * self.L

    def elem_size(self) -> int:
        return 4 if self.dtype == torch.float32 else 2

    def gather_bytes_per_qh(self) -> int:
        """Bytes the forward gathers per query-head: 4 corners x (K, V) x one D-row per key."""
        return self.N * 8 * self.D * self.elem_size()

    def hbm_bytes_per_qh(self, backward: bool = False) -> float:
        """Compulsory HBM bytes per query-head: q, k, v, out once (+ dout, dq, dk, dv),
        coordinates once (shared by the heads) and the 4-byte log-sum-exp."""
        rows = 8 if backward else 4
        return rows * self.D * self.elem_size() + self.N * 8 / self.Hh + 4

    def with_batch(self, B: int) -> "Config":
        return replace(self, B=B)


CONFIGS = {
    "C1": Config("C1", B=2, V=8, S=32, Hh=16, D=32, W=14, H=14, sm_scale=0.5, dtype=torch.float32, coords="uniform"),
    "C2": Config("C2", B=2, V=6, S=16, Hh=8, D=32, W=18, H=18, sm_scale=32 ** -0.5, dtype=torch.float32, coords="oob"),
    "C3": Config("C3", B=4, V=6, S=64, Hh=8, D=64, W=32, H=32, sm_scale=0.125, dtype=torch.bfloat16,
                 coords="clustered", sigma=0.05),
    "C4": Config("C4", B=8, V=6, S=8, Hh=8, D=32, W=88, H=32, sm_scale=32 ** -0.5, dtype=torch.float32,
                 coords="mixed", sigma=0.02),
    "C5": Config("C5", B=32, V=8, S=32, Hh=16, D=64, W=28, H=28, sm_scale=0.125, dtype=torch.bfloat16,
                 coords="uniform"),
}

# Not benchmark configurations: the quick-start shape in the other storage types and head
# dimensions the reference accepts (ops/triton.py:367-375, 386), to put a number on those paths.
EXTRA_CONFIGS = {
    "X_f16_d128": Config("X_f16_d128", B=2, V=8, S=32, Hh=16, D=128, W=14, H=14, sm_scale=128 ** -0.5,
                         dtype=torch.float16, coords="uniform"),
    "X_f32_d256": Config("X_f32_d256", B=2, V=8, S=32, Hh=16, D=256, W=14, H=14, sm_scale=256 ** -0.5,
                         dtype=torch.float32, coords="uniform"),
    "X_bf16_d16": Config("X_bf16_d16", B=2, V=8, S=32, Hh=16, D=16, W=14, H=14, sm_scale=0.25,
                         dtype=torch.bfloat16, coords="uniform"),
}


def config(name: str) -> Config:
    """A benchmark configuration (C1..C5) or one of EXTRA_CONFIGS by name."""
    return CONFIGS[name] if name in CONFIGS else EXTRA_CONFIGS[name]


SEED0 = 20240607


def _centres(W: int, H: int) -> torch.Tensor:
    ls = torch.arange(W * H)
    cx = (ls % W).float() / max(W - 1, 1)
    cy = (ls // W).float() / max(H - 1, 1)
    return torch.stack([cx, cy], -1)


def make_coords(cfg: Config, gen: torch.Generator) -> torch.Tensor:
    """Coordinates of ONE batch element: [V, L, V, S, 2], fp32."""
    shape = (cfg.V, cfg.L, cfg.V, cfg.S, 2)
    if cfg.coords == "uniform":
        return torch.rand(shape, generator=gen)
    if cfg.coords == "oob":
        return torch.rand(shape, generator=gen) * 1.2 - 0.1
    ctr = _centres(cfg.W, cfg.H).view(1, cfg.L, 1, 1, 2)
    near = (ctr + cfg.sigma * torch.randn(shape, generator=gen)).clamp_(0, 1)
    if cfg.coords == "clustered":
        return near
    if cfg.coords == "mixed":
        uni = torch.rand(shape, generator=gen)
        pick = torch.rand(shape[:-1], generator=gen) < 0.5
        return torch.where(pick.unsqueeze(-1), uni, near)
    raise ValueError(cfg.coords)


def make_batch_element(cfg: Config, b: int, cfg_index: int = 0, with_dout: bool = True):
    """q, k, v, coords(, dout) of batch element ``b`` on the CPU.  q/k/v/dout are drawn
    in fp32 from N(0,1) and cast to the configuration's storage type."""
    gen = torch.Generator().manual_seed(SEED0 + 1000 * cfg_index + b)
    shape = (cfg.V, cfg.Hh, cfg.L, cfg.D)
    q = torch.randn(shape, generator=gen).to(cfg.dtype)
    k = torch.randn(shape, generator=gen).to(cfg.dtype)
    v = torch.randn(shape, generator=gen).to(cfg.dtype)
    coords = make_coords(cfg, gen)
    dout = torch.randn(shape, generator=gen).to(cfg.dtype) if with_dout else None
    return q, k, v, coords, dout


def make_inputs(cfg: Config, batch_range=None, with_dout: bool = True, pin: bool = False):
    """Inputs for batch elements ``batch_range`` (default: all) stacked on the CPU:
    ``q, k, v, dout [b, V, Hh, L, D]`` and ``coords [b, V, L, V, S, 2]``."""
    idx = list(CONFIGS).index(cfg.name) if cfg.name in CONFIGS else 9
    lo, hi = (0, cfg.B) if batch_range is None else batch_range
    parts = [make_batch_element(cfg, b, idx, with_dout) for b in range(lo, hi)]
    out = []
    for i in range(5):
        if parts[0][i] is None:
            out.append(None)
            continue
        t = torch.stack([p[i] for p in parts], 0)
        out.append(t.pin_memory() if pin else t)
    return tuple(out)

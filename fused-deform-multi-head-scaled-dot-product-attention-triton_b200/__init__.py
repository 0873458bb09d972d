"""B200 (sm_100a) fused deformable multi-head scaled-dot-product attention.

Drop-in for the reference's fused operator: ``deform_sdpa_triton`` keeps the
reference's name, positional signature and autograd contract
(reference ops/triton.py:466); the device work is hand-written CUDA in
``csrc/`` behind the C ABI of ``include/dsdpa.h``.
"""
from . import cabi  # noqa: F401
from . import inputs  # noqa: F401
from . import partition  # noqa: F401
from . import probes  # noqa: F401  (measurement tooling; loads its library on first use only)
from .host import HostPipeline  # noqa: F401
from .op import deform_sdpa, deform_sdpa_triton, forward_raw, backward_raw  # noqa: F401

__all__ = ["deform_sdpa_triton", "deform_sdpa", "forward_raw", "backward_raw", "cabi", "inputs", "partition", "HostPipeline"]

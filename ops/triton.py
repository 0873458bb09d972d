"""Drop-in for the reference's ``ops/triton.py``: same import path and operator name
(reference ops/triton.py:466), implemented by hand-written sm_100a CUDA.  No Triton."""
from . import backend as _backend

deform_sdpa_triton = _backend.deform_sdpa_triton

__all__ = ["deform_sdpa_triton"]

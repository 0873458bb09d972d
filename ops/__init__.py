"""Reference-facing import path.

The reference is used as ``from ops.triton import deform_sdpa_triton``
(reference README.md:24, benchmark.py:6).  This package keeps that import working and
routes it to the B200 implementation, whose directory name is not an importable
identifier and is therefore loaded here under the module name ``deform_sdpa_b200``.
"""
import importlib.util as _ilu
import sys as _sys
from pathlib import Path as _Path

_PKG_DIR = _Path(__file__).resolve().parent.parent / "fused-deform-multi-head-scaled-dot-product-attention-triton_b200"
_NAME = "deform_sdpa_b200"


def _load_backend():
    mod = _sys.modules.get(_NAME)
    if mod is not None:
        return mod
    spec = _ilu.spec_from_file_location(_NAME, _PKG_DIR / "__init__.py", submodule_search_locations=[str(_PKG_DIR)])
    mod = _ilu.module_from_spec(spec)
    _sys.modules[_NAME] = mod
    try:
        spec.loader.exec_module(mod)
    except BaseException:
        _sys.modules.pop(_NAME, None)
        raise
    return mod


backend = _load_backend()

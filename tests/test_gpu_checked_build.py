"""The checked debug build (libdeform_sdpa_checked.so, compiled with -DDSDPA_BOUNDS_CHECK): its
kernels test every pixel index, index-entry offset and work-list position they compute against
its range, record a violation in the error word and skip the access instead of faulting.

The parity tests on the golden vectors, the edge shapes and the five configurations are run once
more in a child process that loads this build (DSDPA_LIBRARY); the suite's own fixture asks
dsdpa_device_error() after every test, so an out-of-range index anywhere fails the run.  This
stands where a compute-sanitizer run would: the reference has no tests to mirror here.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CHECKED = ROOT / "fused-deform-multi-head-scaled-dot-product-attention-triton_b200" / "libdeform_sdpa_checked.so"


@pytest.mark.gpu
def test_parity_suite_on_the_checked_build():
    assert CHECKED.exists(), "build.py builds the checked library beside the normal one"
    env = dict(os.environ, DSDPA_LIBRARY=str(CHECKED))
    probe = subprocess.run([sys.executable, "-c",
                            "import ops; print(ops.backend.cabi.lib().dsdpa_build_is_checked())"],
                           cwd=ROOT, env=env, capture_output=True, text=True)
    assert probe.stdout.strip() == "1", probe.stderr[-2000:]
    res = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_parity.py", "-m", "gpu", "-x", "-q",
                          "-k", "golden or edge or configs or coordinate_gradient or large_map or huge_map",
                          "-p", "no:cacheprovider"],
                         cwd=ROOT, env=env, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-2000:]
    assert " passed" in res.stdout


def test_the_normal_build_is_not_the_checked_one():
    import ops
    assert ops.backend.cabi.lib().dsdpa_build_is_checked() == int(bool(os.environ.get("DSDPA_LIBRARY", "").endswith("_checked.so")))

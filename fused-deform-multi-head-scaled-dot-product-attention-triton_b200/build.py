"""Builds the shared libraries in-tree with nvcc for sm_100a.

    python build.py [--force] [--jobs N]

Every translation unit under csrc/ is compiled to csrc/_build/*.o in parallel and the
objects are linked into libdeform_sdpa.so (the C-ABI library, the product) beside this
file; csrc/probes/*.cu become libdsdpa_probes.so, the bandwidth probes the benchmark uses
for its roofline denominators (not linked into, or needed by, the product library).  The same
sources compiled with -DDSDPA_BOUNDS_CHECK give libdeform_sdpa_checked.so, the debug build
whose kernels range-check every index they compute (the tests run it on the small cases;
DSDPA_LIBRARY=<path> makes the Python binding load it).  Nothing is installed outside the
source tree.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = CSRC / "_build"
LIB = HERE / "libdeform_sdpa.so"
PROBES_LIB = HERE / "libdsdpa_probes.so"
CHECKED_LIB = HERE / "libdeform_sdpa_checked.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (cand == "nvcc" or Path(cand).exists()):
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.inc"))
    hdrs.append(HERE.parent / "include" / "dsdpa.h")
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: Path, force: bool, hdr_time: float, checked: bool = False) -> Path:
    out_dir = OBJ / "checked" if checked else OBJ
    obj = out_dir / (src.stem + ".o")
    # -DNAME=value pairs for experiments and for the checked debug build
    if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_time):
        return obj
    extra = os.environ.get("DSDPA_NVCC_EXTRA", "").split()   # e.g. -DDSDPA_FWD_UNROLL=4, for experiments
    if checked:
        extra = extra + ["-DDSDPA_BOUNDS_CHECK"]
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (out_dir / (src.stem + ".ptxas.log")).write_text(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    return obj


def _link(lib: Path, objs: list[Path], force: bool) -> None:
    if force or not lib.exists() or lib.stat().st_mtime < max(o.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-shared", "-o", str(lib), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")


def build(force: bool = False, jobs: int | None = None, checked: bool = True) -> Path:
    (OBJ / "checked").mkdir(parents=True, exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    probe_srcs = sorted((CSRC / "probes").glob("*.cu"))
    hdr_time = _newest_header()
    work = [(s, False) for s in srcs + probe_srcs] + ([(s, True) for s in srcs] if checked else [])
    jobs = jobs or min(len(work), os.cpu_count() or 4)
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        objs = list(pool.map(lambda w: _compile(w[0], force, hdr_time, w[1]), work))
    n, m = len(srcs), len(srcs) + len(probe_srcs)
    _link(LIB, objs[:n], force)
    _link(PROBES_LIB, objs[n:m], force)
    if checked:
        _link(CHECKED_LIB, objs[m:], force)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--no-checked", action="store_true", help="skip the bounds-checked debug build")
    a = ap.parse_args()
    print(build(a.force, a.jobs, not a.no_checked))

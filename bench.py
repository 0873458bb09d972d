#!/usr/bin/env python
"""Benchmark of the fused deformable SDPA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config C5] [--mode fwdbwd|fwd]

One "step" is one pass of the hot path over the workload: forward and backward
(dq, dk, dv) of the operator through the C ABI.  The workload at every N is the
scaling configuration C5 (B=32, V=8, S=32, heads=16, D=64, 28x28 map, bf16, uniform
coordinates), the total split by batch over the N ranks ("strong" scaling) with the
results landing on rank 0 inside the timed region (by default the kernels store them
there themselves as they produce them; the environment variable BENCH_GATHER selects the
other ways, see main).  Rank 0 prints ONE JSON line.

`--impl reference` times the CPU implementation of the same path (the C oracle port of
the reference's ops/torch.py, all host threads) on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from dataclasses import replace
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "query-heads/sec (forward+backward)"
METRIC_FWD = "query-heads/sec (forward)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="C5")
    ap.add_argument("--mode", default="fwdbwd", choices=["fwdbwd", "fwd"])
    ap.add_argument("--batch", type=int, default=0,
                    help="override the configuration's batch size (e.g. 4: what one rank of an 8-GPU run of C5 holds)")
    ap.add_argument("--flags", type=lambda x: int(x, 0), default=0,
                    help="DSDPA_FLAG_* bits for every call (e.g. 0x10, rounded weights; 0x8, the scatter backward)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--sweep", action="store_true",
                    help="the reference's own sweep instead of the benchmark line: views x samples in {2..12}, "
                         "forward and backward latency and peak memory (reference benchmark.py:16-57)")
    ap.add_argument("--probes", action="store_true",
                    help="measure the roofline denominators only: L2 read, shared-memory access patterns, "
                         "L1-hit row gather; one JSON line")
    ap.add_argument("--profile-case", default=None, metavar="CFG:B:MODE[:FLAGS]",
                    help="run a small case of a configuration (e.g. C5:2:bwd) twice through the C ABI and exit: "
                         "the command the committed ncu captures were taken with")
    return ap.parse_args()


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", os.environ.get("BENCH_CLOCK_MS", "200")], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for n, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------
# CPU arm (the reference's path restated in C, test infrastructure)
# --------------------------------------------------------------------------------------
def host_threads():
    """Host cores this process may use.  (Not OpenMP's default: torch.distributed.run sets
    OMP_NUM_THREADS=1 for its workers, which would silently time the CPU arm on one core.)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return max(1, os.cpu_count() or 1)


def cpu_sample(cfg, mode, steps, warmup, target_s=15.0):
    """Times the oracle on a bounded sample of the workload: whole batch elements (all
    their heads), as many as keep one step near `target_s` seconds on this host."""
    from oracle import oracle as orc
    import ops
    inp = ops.backend.inputs
    threads = host_threads()
    per_batch_qh = cfg.V * cfg.Hh * cfg.L

    def run(q, k, v, coords, dout):
        t0 = time.perf_counter()
        orc.forward(q, k, v, coords, cfg.W, cfg.H, cfg.sm_scale, nthreads=threads)
        if mode == "fwdbwd":
            orc.backward(q, k, v, coords, dout, cfg.W, cfg.H, cfg.sm_scale, nthreads=threads)
        return time.perf_counter() - t0

    # calibration: enough batch elements to give every thread a (batch, head) slice
    nb_cal = max(1, min(cfg.B, (threads + cfg.Hh - 1) // cfg.Hh))
    cal = inp.make_inputs(replace(cfg, B=nb_cal))
    t_cal = run(*cal)
    nb = max(nb_cal, min(cfg.B, int(nb_cal * target_s / max(t_cal, 1e-3))))
    data = cal if nb == nb_cal else inp.make_inputs(replace(cfg, B=nb))
    for _ in range(warmup):
        run(*data)
    times = [run(*data) for _ in range(steps)]
    t = sum(times) / len(times)
    qh = nb * per_batch_qh
    return {
        "value": qh / t, "ms_per_step": t * 1e3, "cores": threads, "kind": "port",
        "unit": "query-heads/sec",
        "sample": f"{nb} of {cfg.B} batch elements of {cfg.name} ({nb * cfg.Hh} (batch, head) slices, "
                  f"{qh} query-heads per step), {'forward+backward' if mode == 'fwdbwd' else 'forward'}",
    }


REF_TORCH = ROOT / "baseline" / "_ref" / "ops" / "torch.py"


def reference_torch_sample(cfg, mode, n_slices=4):
    """Times the reference's own pure-PyTorch path, unmodified (its ops/torch.py, kept out of
    the repository's history under baseline/_ref/), on the host cores: `n_slices` (batch, head)
    slices of the workload, one call each (a slice is the largest piece that function can take
    at the larger configurations: it materialises every sampled key), forward and, through
    autograd, backward.  Slices are independent and equal-sized, so the figure extrapolates
    linearly to the whole workload."""
    if not REF_TORCH.exists():
        return {"unavailable": f"{REF_TORCH.relative_to(ROOT)} is not present (it is copied from the reference by "
                               "__graft_entry__.build() where the reference is mounted)"}
    try:
        import torch
        import ops
        ref_fn = _load_reference_torch()
    except Exception as exc:  # noqa: BLE001  (e.g. einops missing on this host)
        return {"unavailable": f"the reference's ops/torch.py does not import here: {exc!r}"}
    threads = host_threads()
    torch.set_num_threads(threads)
    q, k, v, coords, dout = ops.backend.inputs.make_inputs(replace(cfg, B=1))
    n_slices = max(1, min(n_slices, cfg.Hh))
    t_total = 0.0
    for h in range(n_slices):
        qs, ks, vs, ds = (t[:, :, h:h + 1].clone() for t in (q, k, v, dout))
        qs.requires_grad_(True), ks.requires_grad_(True), vs.requires_grad_(True)
        t0 = time.perf_counter()
        out = ref_fn(qs, ks, vs, coords, cfg.W, cfg.H, cfg.sm_scale)
        if mode == "fwdbwd":
            out.backward(ds)
        t_total += time.perf_counter() - t0
    qh = n_slices * cfg.V * cfg.L
    return {"value": qh / t_total, "unit": "query-heads/sec", "cores": threads, "kind": "reference",
            "sample": f"{n_slices} of {cfg.B * cfg.Hh} (batch, head) slices of {cfg.name}, one call of the reference's "
                      f"deform_sdpa_torch each ({qh} query-heads), "
                      f"{'forward+backward' if mode == 'fwdbwd' else 'forward'}, extrapolated linearly"}


def run_reference_arm(args):
    import ops
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = ops.backend.inputs.config(args.config)
    # one CPU step takes about 15 s: at most three timed steps and one warm-up, whatever was asked
    steps = max(1, min(args.steps, 3))
    warm = 1 if args.warmup > 0 else 0
    r = cpu_sample(cfg, args.mode, steps, warm)
    ref = reference_torch_sample(cfg, args.mode)
    line = {
        "impl": "reference",
        "metric": METRIC if args.mode == "fwdbwd" else METRIC_FWD,
        "value": r["value"], "unit": "query-heads/sec", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if cfg.elem_size() == 2 else "f32", "data": "synthetic (seeded)",
        "config": config_dict(cfg, args, 1),
        "cpu_baseline": {"value": r["value"], "unit": r["unit"], "cores": r["cores"], "kind": r["kind"],
                         "sample": r["sample"]},
        "cpu_baseline_reference": ref,
        "steps_note": f"requested steps={args.steps} warmup={args.warmup}; run with steps={steps} warmup={warm} "
                      "(a CPU step takes about 15 s)",
        "e2e": {"value": r["value"], "unit": "query-heads/sec", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def config_dict(cfg, args, world):
    # q, k, v, dout and the coordinates of the whole job
    in_gb = (4 * cfg.query_heads * cfg.D * cfg.elem_size() + cfg.B * cfg.V * cfg.L * cfg.N * 8) / 1e9
    return {
        "workload": f"{cfg.name}: B={cfg.B} V={cfg.V} S={cfg.S} heads={cfg.Hh} D={cfg.D} map={cfg.W}x{cfg.H} "
                    f"sm_scale={cfg.sm_scale:g} {str(cfg.dtype).replace('torch.', '')} coords={cfg.coords}",
        "step": "forward+backward (dq, dk, dv)" if args.mode == "fwdbwd" else "forward",
        "sharding": f"batch over {world} rank(s), outputs gathered to rank 0" if world > 1 else "single GPU",
        "l2": ("inputs (%.2f GB per step) are larger than L2; no explicit flush" % (in_gb,) if in_gb > 0.252 else
               "inputs (%.0f MB) fit L2: a 256 MB buffer is written between timed steps" % (in_gb * 1e3,)),
    }


# --------------------------------------------------------------------------------------
# the reference's sweep (role of its benchmark.py)
# --------------------------------------------------------------------------------------
def _load_reference_torch():
    if not REF_TORCH.exists():
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("_reference_ops_torch", REF_TORCH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.deform_sdpa_torch


def run_sweep():
    """Views x samples sweep with the reference's defaults (benchmark.py:16-20, 29-31: batch 2,
    32 heads, head dim 32, 18x18 map, fp32, sm_scale 0.5, V and S in {2,4,...,12}), forward and
    backward latency (CUDA events, median of 20 after at least 5 warm-ups and 50 ms) and peak
    device memory of one call.  One JSON line per (provider, mode, V, S).  As in the reference's script
    (benchmark.py:73-88) the second provider is the reference's own PyTorch path on the same GPU
    (its ops/torch.py, unmodified, where baseline/_ref/ holds it): timed on the diagonal V = S and
    on the V = 12 row, backward through autograd with the graph retained."""
    import torch
    import ops
    be = ops.backend
    dev = torch.device("cuda", 0)
    B, Hh, D, W = 2, 32, 32, 18
    L = W * W
    gen = torch.Generator(device=dev).manual_seed(1)
    ref_fn = _load_reference_torch()
    if ref_fn is None:
        print(json.dumps({"sweep_reference": "unavailable", "why": f"{REF_TORCH.relative_to(ROOT)} is not present"}),
              flush=True)

    def measure(fn, warm, reps):
        # warm-up: at least `warm` calls and at least 50 ms of them (allocations of the previous
        # point leave the GPU idle for a moment, and its clocks take a while to come back)
        t0 = time.perf_counter()
        n = 0
        while n < warm or time.perf_counter() - t0 < 0.05:
            fn()
            n += 1
            if n % 8 == 0:
                torch.cuda.synchronize()
        times = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); b.synchronize()
            times.append(a.elapsed_time(b))
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats(dev)
        base = torch.cuda.memory_allocated(dev)
        fn()
        torch.cuda.synchronize()
        return statistics.median(times), (torch.cuda.max_memory_allocated(dev) - base) / 1e6

    for V in (2, 4, 6, 8, 10, 12):
        for S in (2, 4, 6, 8, 10, 12):
            q, k, v, do = (torch.randn(B, V, Hh, L, D, device=dev, generator=gen) for _ in range(4))
            coords = torch.rand(B, V, L, V, S, 2, device=dev, generator=gen)
            out, lse = be.forward_raw(q, k, v, coords, W, W, 0.5)
            row = {"V": V, "S": S, "B": B, "heads": Hh, "D": D, "map": f"{W}x{W}", "dtype": "f32"}

            def fwd():
                return be.forward_raw(q, k, v, coords, W, W, 0.5)

            def bwd():
                return be.backward_raw(q, k, v, coords, out, lse, do, W, W, 0.5)

            for mode, fn in (("fwd", fwd), ("bwd", bwd)):
                ms, peak = measure(fn, 5, 20)
                print(json.dumps(dict(row, sweep=mode, provider="b200", latency_ms=ms, peak_extra_MB=peak)), flush=True)
            if ref_fn is None or not (V == S or V == 12):
                continue
            qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))

            def rfwd():
                with torch.no_grad():
                    return ref_fn(q, k, v, coords, W, W, 0.5)

            ms, peak = measure(rfwd, 2, 5)
            print(json.dumps(dict(row, sweep="fwd", provider="reference_torch", latency_ms=ms, peak_extra_MB=peak)),
                  flush=True)
            o = ref_fn(qr, kr, vr, coords, W, W, 0.5)

            def rbwd():
                o.backward(do, retain_graph=True)

            ms, peak = measure(rbwd, 2, 5)
            print(json.dumps(dict(row, sweep="bwd", provider="reference_torch", latency_ms=ms, peak_extra_MB=peak)),
                  flush=True)
            del o, qr, kr, vr
            torch.cuda.empty_cache()


def measure_peaks(dev_index):
    """Roofline denominators measured on this device by libdsdpa_probes.so (GB/s)."""
    import torch
    import ops
    pr = ops.backend.probes
    dev = torch.device("cuda", dev_index)
    buf = torch.empty(32 << 20, dtype=torch.uint8, device=dev)
    small = torch.zeros(64 << 10, dtype=torch.uint8, device=dev)
    torch.cuda.synchronize(dev)
    peaks = {"l2_read": pr.l2_read(buf.data_ptr(), buf.numel(), dev_index),
             "l1_row_gather": pr.l1_row_gather(small.data_ptr(), dev_index),
             "shared": {k: pr.shared_pattern(k, dev_index) for k in pr.SHARED_PATTERNS}}
    torch.cuda.set_device(dev)
    return peaks


def run_probes():
    import ops
    pr = ops.backend.probes
    peaks = measure_peaks(0)
    print(json.dumps({"probes": {"l2_read_GBps": peaks["l2_read"], "l1_row_gather_GBps": peaks["l1_row_gather"],
                                 "shared_GBps": {pr.SHARED_PATTERNS[k]: v for k, v in peaks["shared"].items()}}}),
          flush=True)


def run_profile_case(spec):
    """Forward (and backward) of configuration CFG with batch B, twice, for ncu to capture.
    MODE is fwd or bwd (= forward + backward); FLAGS are DSDPA_FLAG_* bits."""
    import torch
    import ops
    be = ops.backend
    parts = spec.split(":")
    cfg = replace(be.inputs.config(parts[0]), B=int(parts[1]))
    mode = parts[2] if len(parts) > 2 else "fwd"
    flags = int(parts[3], 0) if len(parts) > 3 else 0
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(1)
    shape = (cfg.B, cfg.V, cfg.Hh, cfg.L, cfg.D)
    q, k, v, do = (torch.randn(shape, device=dev, generator=gen).to(cfg.dtype) for _ in range(4))
    one = replace(cfg, B=1)
    coords = torch.stack([be.inputs.make_coords(one, torch.Generator().manual_seed(b)) for b in range(cfg.B)]).to(dev)
    for _ in range(2):
        out, lse = be.forward_raw(q, k, v, coords, cfg.W, cfg.H, cfg.sm_scale, flags=flags)
        if mode != "fwd":
            be.backward_raw(q, k, v, coords, out, lse, do, cfg.W, cfg.H, cfg.sm_scale, flags=flags)
    torch.cuda.synchronize()
    be.cabi.check(be.cabi.lib().dsdpa_device_error(0))
    print("ok")


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.sweep:
        run_sweep()
        return
    if args.profile_case:
        run_profile_case(args.profile_case)
        return
    if args.probes:
        run_probes()
        return

    import torch
    import torch.distributed as dist
    import ops
    be = ops.backend
    cabi, inp, part = be.cabi, be.inputs, be.partition

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path "
                         "(use --impl reference for the CPU arm)")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # The result gathers share the GPU with kernels that fill every SM: give NCCL's stream
        # priority, or its CTAs only run in the gaps between kernels and the gather falls behind.
        opts = dist.ProcessGroupNCCL.Options()
        opts.is_high_priority_stream = True
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)

    cfg = inp.config(args.config)
    if args.batch > 0:
        cfg = replace(cfg, B=args.batch)
    plan = part.shard_plan(cfg.B, cfg.Hh, world)
    shard = plan[rank]
    nb = shard.b1 - shard.b0
    nh = shard.h1 - shard.h0
    lib = cabi.lib()
    fwd_only = args.mode == "fwd"

    # ---- synthetic inputs of this rank's shard, drawn on the device (seeded per batch element)
    def draw(b):
        g = torch.Generator(device=dev).manual_seed(inp.SEED0 + 4000 + b)
        shape = (cfg.V, cfg.Hh, cfg.L, cfg.D)
        q = torch.randn(shape, generator=g, device=dev).to(cfg.dtype)
        k = torch.randn(shape, generator=g, device=dev).to(cfg.dtype)
        v = torch.randn(shape, generator=g, device=dev).to(cfg.dtype)
        do = torch.randn(shape, generator=g, device=dev).to(cfg.dtype)
        cs = (cfg.V, cfg.L, cfg.V, cfg.S, 2)
        if cfg.coords == "uniform":
            c = torch.rand(cs, generator=g, device=dev)
        elif cfg.coords == "oob":
            c = torch.rand(cs, generator=g, device=dev) * 1.2 - 0.1
        else:
            ls = torch.arange(cfg.L, device=dev)
            ctr = torch.stack([(ls % cfg.W).float() / max(cfg.W - 1, 1), (ls // cfg.W).float() / max(cfg.H - 1, 1)], -1)
            near = (ctr.view(1, cfg.L, 1, 1, 2) + cfg.sigma * torch.randn(cs, generator=g, device=dev)).clamp_(0, 1)
            if cfg.coords == "clustered":
                c = near
            else:
                uni = torch.rand(cs, generator=g, device=dev)
                pick = torch.rand(cs[:-1], generator=g, device=dev) < 0.5
                c = torch.where(pick.unsqueeze(-1), uni, near)
        sl = slice(shard.h0, shard.h1)
        return q[:, sl], k[:, sl], v[:, sl], do[:, sl], c

    parts = [draw(b) for b in range(shard.b0, shard.b1)]
    q, k, v, dout = (torch.stack([p[i] for p in parts]).contiguous() for i in range(4))
    coords = torch.stack([p[4] for p in parts]).contiguous()
    del parts
    full_shape = (cfg.B, cfg.V, cfg.Hh, cfg.L, cfg.D)

    n_results = 1 if fwd_only else 4

    # How the results reach rank 0 (inside the timed region in every mode but "none"):
    #   mirror     the kernels store every result row a second time, into rank 0's tensors, which
    #              every rank has mapped through CUDA IPC (default; needs all ranks on one box)
    #   nccl_sync  dist.gather after the step's kernels, on their stream
    #   nccl       the same on a side stream, free to overlap the next step's kernels
    #   peer       device-to-device copies into the mapped tensors on a side stream (copy engines)
    #   none       no gather (to measure what the gather costs)
    gather_mode = os.environ.get("BENCH_GATHER", "mirror") if world > 1 else "none"

    def gather(t, slot=0):
        if world == 1 or gather_mode == "none":
            return t
        return part.gather_to_root(t, plan, full_shape, root=0, out=dest[slot])

    peer = None
    if gather_mode in ("peer", "mirror"):
        try:
            peer = part.PeerGather([(full_shape, cfg.dtype)] * n_results, plan, dev)
        except Exception as exc:  # noqa: BLE001  (ranks that cannot share memory gather with NCCL)
            if rank == 0:
                print(f"rank 0's result tensors cannot be mapped by the other ranks ({exc!r}); using NCCL",
                      file=sys.stderr)
            gather_mode = "nccl_sync"
    side = torch.cuda.Stream(dev) if gather_mode == "nccl" else None
    # (NCCL modes: rank 0 receives into the same preallocated tensors every step)
    dest = [torch.empty(full_shape, dtype=cfg.dtype, device=dev) for _ in range(n_results)] \
        if gather_mode in ("nccl", "nccl_sync") and rank == 0 else [None] * n_results
    views = peer.shard_views() if gather_mode == "mirror" else None
    last_local = []

    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    fwd_ms, bwd_ms = [], []

    def step(record):
        e0, e1, e2 = ev(), ev(), ev()
        e0.record()
        out, lse = be.forward_raw(q, k, v, coords, cfg.W, cfg.H, cfg.sm_scale, flags=args.flags,
                                  out_mirror=views[0] if views and fwd_only else None)
        e1.record()
        res = [out]
        if not fwd_only:
            # (with mirrors the backward's first pass, which reads out anyway, sends it along)
            mir = dict(zip(("out", "dq", "dk", "dv"), views)) if views else None
            dq, dk, dv, _ = be.backward_raw(q, k, v, coords, out, lse, dout, cfg.W, cfg.H, cfg.sm_scale,
                                            flags=args.flags, mirrors=mir)
            e2.record()
            res += [dq, dk, dv]
        last_local[:] = res
        if views is not None:
            gathered = res
        elif peer is not None:
            for i, t in enumerate(res):
                peer.push(i, t)
            gathered = res
        elif side is None:
            gathered = [gather(t, i) for i, t in enumerate(res)]
        else:
            # The gathers to rank 0 run on their own stream, behind this step's kernels, and may
            # overlap the next step's kernels; the barrier + synchronize that close the timed
            # region wait for all of them.
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for t in res:
                    t.record_stream(side)
                gathered = [gather(t, i) for i, t in enumerate(res)]
        if record:
            fwd_ms.append((e0, e1))
            if not fwd_only:
                bwd_ms.append((e1, e2))
        return gathered

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Inputs smaller than twice the L2 would be served from it on the second step: such
    # configurations are timed step by step with a 256 MB write between the steps.
    in_bytes = sum(t.numel() * t.element_size() for t in (q, k, v, coords, dout))
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if in_bytes < (252 << 20) else None

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn(False)
        barrier()
        if flush_buf is not None:
            pairs = []
            for _ in range(steps):
                flush_buf.fill_(1)
                a, b = ev(), ev()
                a.record()
                fn(True)
                if peer is not None:
                    peer.wait()
                elif side is not None:
                    torch.cuda.current_stream(dev).wait_stream(side)
                b.record()
                pairs.append((a, b))
            barrier()
            ms = torch.tensor([sum(a.elapsed_time(b) for a, b in pairs)], device=dev)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return ms.item()
        a, b = ev(), ev()
        a.record()
        for _ in range(steps):
            fn(True)
        if peer is not None:
            peer.wait()
        elif side is not None:
            # the last steps' gathers belong to the timed region
            torch.cuda.current_stream(dev).wait_stream(side)
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    launches0 = lib.dsdpa_kernel_launches()
    sampler = ClockSampler(local_rank) if rank == 0 and os.environ.get("BENCH_CLOCK_MS", "200") != "0" else None
    if sampler:
        sampler.start()
    total_ms = timed(step, args.steps, max(args.warmup, 3))
    clocks = sampler.stop() if sampler else None
    launches_all = lib.dsdpa_kernel_launches() - launches0

    # did the last step's results reach rank 0?  every rank sends the results it computed (one more
    # step, outside the timed region) to rank 0 over NCCL, and rank 0 compares them element by
    # element with the matching slices of what the timed path delivered
    gather_ok = None
    if world > 1 and gather_mode != "none":
        last = step(False)
        if peer is not None:
            peer.wait()
        elif side is not None:
            torch.cuda.current_stream(dev).wait_stream(side)
        barrier()
        gather_ok = True
        full = (peer.results if peer is not None else last) if rank == 0 else None
        for i, t in enumerate(last_local):
            for src, sh in enumerate(plan):
                shape = (sh.b1 - sh.b0, cfg.V, sh.h1 - sh.h0, cfg.L, cfg.D)
                if rank == 0:
                    got = t if src == 0 else torch.empty(shape, dtype=cfg.dtype, device=dev)
                    if src != 0:
                        dist.recv(got, src=src)
                    want = full[i][sh.b0:sh.b1, :, sh.h0:sh.h1]
                    gather_ok = gather_ok and bool(torch.equal(got, want))
                elif rank == src:
                    dist.send(t.contiguous(), dst=0)
        barrier()
    cabi.check(lib.dsdpa_device_error(local_rank))
    # launches inside the timed region only (warm-up steps launch the same kernels)
    steps_run = args.steps + max(args.warmup, 3)
    launches = launches_all * args.steps // steps_run

    ms_step = total_ms / args.steps
    value = cfg.query_heads / (ms_step * 1e-3)
    f_ms = statistics.mean(a.elapsed_time(b) for a, b in fwd_ms)
    b_ms = statistics.mean(a.elapsed_time(b) for a, b in bwd_ms) if bwd_ms else None

    # ---- forward only (extra, same timing rules)
    fwd_value = None
    if not fwd_only:
        def fstep(_record):
            out, _lse = be.forward_raw(q, k, v, coords, cfg.W, cfg.H, cfg.sm_scale, flags=args.flags,
                                       out_mirror=views[0] if views else None)
            if views is not None:
                return out
            if peer is not None:
                peer.push(0, out)
                return out
            if side is None:
                return gather(out)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                out.record_stream(side)
                return gather(out)
        fwd_total = timed(fstep, args.steps, 3)
        fwd_value = cfg.query_heads / (fwd_total / args.steps * 1e-3)

    # ---- end to end: pinned host inputs in, results back out, through the operator's API
    e2e = None
    if not args.no_e2e:
        sizes = [int(x) for x in os.environ["BENCH_E2E_SIZES"].split(",")] if os.environ.get("BENCH_E2E_SIZES") else None

        class Leg:
            """Pinned host tensors of a batch range and the operator's front end for them: chunks
            of batch elements on copy-in, compute and copy-out streams; every byte crosses PCIe
            inside the timed region."""

            def __init__(self, tensors, n_elements, head_parts):
                self.nb = n_elements
                self.hq, self.hk, self.hv, self.hdo, self.hc = (t.cpu().pin_memory() for t in tensors)
                self.h_out = [torch.empty_like(self.hq).pin_memory() for _ in range(1 if fwd_only else 4)]
                ins = (self.hq, self.hk, self.hv, self.hc) if fwd_only else (self.hq, self.hk, self.hv, self.hc, self.hdo)
                self.h2d = sum(t.numel() * t.element_size() for t in ins)
                self.d2h = sum(t.numel() * t.element_size() for t in self.h_out)
                self.pipe = be.HostPipeline(dev, cfg.W, cfg.H, cfg.sm_scale, sizes=sizes,
                                            compute_streams=int(os.environ.get("BENCH_E2E_STREAMS", "2")),
                                            head_parts=head_parts,
                                            chunk=max(1, min(int(os.environ.get("BENCH_E2E_CHUNK", "8")), n_elements)))

            def step(self, _record):
                o = self.h_out
                if fwd_only:
                    self.pipe.run(self.hq, self.hk, self.hv, self.hc, out=o[0])
                else:
                    self.pipe.run(self.hq, self.hk, self.hv, self.hc, self.hdo, out=o[0], dq=o[1], dk=o[2], dv=o[3])

        head_parts = int(os.environ.get("BENCH_E2E_HEAD_PARTS", "1"))
        leg = Leg((q, k, v, dout, coords), nb, head_parts)
        # Several ranks: the GPUs of a box need not sit behind equally fast host links (measured
        # here: with all eight ranks transferring, four get half the rate of the other four).  The
        # leg calibrates itself: every rank times its pipeline over its even share, the times per
        # batch element become weights, and the batch is split again in their proportion (like
        # ranks share a weight, so a box of equal links keeps the even split).  A rank whose copies
        # take longer than its kernels also cuts its first and last element into head groups.
        shares, costs = None, None
        if world > 1 and cfg.B >= world and os.environ.get("BENCH_E2E_BALANCE", "1") != "0":
            for _ in range(2):
                leg.step(False)
            torch.cuda.synchronize()
            barrier()
            a, b = ev(), ev()
            a.record()
            for _ in range(2):
                leg.step(False)
            b.record()
            torch.cuda.synchronize()
            mine = a.elapsed_time(b) / 2 / nb
            costs = [None] * world
            dist.all_gather_object(costs, mine)
            weights = be.host.weights_from_costs(costs)
            if os.environ.get("BENCH_E2E_WEIGHTS"):      # a given split, to try the uneven path anywhere
                weights = [float(x) for x in os.environ["BENCH_E2E_WEIGHTS"].split(",")]
            kernels_ms = total_ms / args.steps * world / cfg.B
            if "BENCH_E2E_HEAD_PARTS" not in os.environ and mine > 1.3 * kernels_ms and cfg.Hh >= 4:
                head_parts = 4
            e_plan = part.shard_plan(cfg.B, cfg.Hh, world, weights=weights)
            shares = [s.b1 - s.b0 for s in e_plan]
            if e_plan[rank] != shard or head_parts != leg.pipe.head_parts:
                del leg
                parts = [draw(b) for b in range(e_plan[rank].b0, e_plan[rank].b1)]
                tensors = [torch.stack([p[i] for p in parts]).contiguous() for i in (0, 1, 2, 3, 4)]
                del parts
                leg = Leg(tensors, shares[rank], head_parts)
                del tensors
        if world > 1:
            moved = torch.tensor([leg.h2d, leg.d2h], dtype=torch.int64, device=dev)
            dist.all_reduce(moved)
            h2d_all, d2h_all = (int(x) for x in moved.tolist())
        else:
            h2d_all, d2h_all = leg.h2d, leg.d2h
        pipe, estep, e_nb = leg.pipe, leg.step, leg.nb

        e_total = timed(estep, max(2, min(args.steps, 5)), 3)
        e_ms = e_total / max(2, min(args.steps, 5))
        # what the copies of one more step (outside the timed region) sustained on every rank
        pipe.time_transfers = True
        estep(False)
        torch.cuda.synchronize()
        rates = pipe.transfer_rates()
        per_rank = [None] * world
        if world > 1:
            dist.all_gather_object(per_rank, rates)
        else:
            per_rank = [rates]
        # bytes of the whole job (summed over the ranks)
        e2e = {"value": cfg.query_heads / (e_ms * 1e-3), "unit": "query-heads/sec", "ms_per_step": e_ms,
               "h2d_bytes_per_step": h2d_all, "d2h_bytes_per_step": d2h_all,
               "chunks": [b1 - b0 if (h0, h1) == (0, cfg.Hh) else f"{h1 - h0}/{cfg.Hh} heads"
                          for b0, b1, h0, h1 in pipe.schedule(e_nb, cfg.Hh)],
               "transfers_per_rank": per_rank}
        if shares is not None:
            e2e["batch_elements_per_rank"] = shares
            e2e["calibration_ms_per_batch_element"] = [round(c, 2) for c in costs]
        del leg, pipe, estep

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the forward kernel and of the backward
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    hbm_peak, hbm_src = 6650.0, "fallback"
    if peaks_file.exists():
        try:
            hbm_peak = float(json.loads(peaks_file.read_text())["hbm_gbs"])
            hbm_src = "measured"
        except (KeyError, ValueError):
            pass
    peaks = measure_peaks(local_rank)
    l2_peak, smem_rows_peak, l1_rows_peak = peaks["l2_read"], peaks["shared"][1], peaks["l1_row_gather"]
    qh_rank = nb * cfg.V * nh * cfg.L
    gather_b = qh_rank * cfg.gather_bytes_per_qh()
    hbm_f = qh_rank * cfg.hbm_bytes_per_qh(False)
    hbm_b = qh_rank * cfg.hbm_bytes_per_qh(True)
    dt = {torch.float32: cabi.F32, torch.bfloat16: cabi.BF16, torch.float16: cabi.F16}[cfg.dtype]
    prob = cabi.Problem(nb, cfg.V, nh, cfg.W, cfg.H, cfg.D, cfg.S, cfg.sm_scale, dt, args.flags)
    plan_text = cabi.describe_plan(prob)
    staged = plan_text.startswith("fwd[staged")
    gather_gbs = gather_b / (f_ms * 1e-3) / 1e9
    # The binding roof of a row gather: the shared-memory pipe where the maps are staged (one
    # 128-byte wavefront per cycle and SM whatever the pattern), else the L1 data path, which
    # the same probe pattern reaches when its rows hit L1.  Both measured in this run.
    gather_peak = smem_rows_peak if staged else l1_rows_peak
    roofline = {
        "kernel": "fwd_kernel (forward, one launch per step)",
        "bound": "shared_memory" if staged else "l1",
        "achieved": gather_gbs, "peak": gather_peak, "unit": "GB/s", "frac": gather_gbs / gather_peak,
        "algorithmic_bytes": "K/V gather bytes: query-heads x V*S keys x 8 rows x D x elem_size",
        "peak_source": ("shared-memory read bandwidth measured in this run with the kernel's access pattern (every group "
                        "of 8 lanes reads an unrelated 128-byte row; contiguous and 256-byte patterns measure the same)"
                        if staged else
                        "row gather from a 64 KB global buffer that stays in L1, measured in this run (the ceiling when "
                        "every row hits L1; rows that miss are served by L2 at l2_read_peak)"),
        # dram__bytes_read.sum + dram__bytes_write.sum of the forward kernel, NOT measured in this run:
        # from the committed ncu capture of a B=2 case of this configuration, scaled to this launch
        # by its query-heads (the traffic grows in proportion to the batch)
        "traffic": (119.2e6 / 200704) * qh_rank if cfg.name == "C5" else None,
        "traffic_source": "profiles/c5_b2_kernels_full_set.md (ncu, B=2 case, scaled by query-heads)" if cfg.name == "C5" else None,
        "l2_read_peak": l2_peak,
        "shared_patterns_GBps": {str(k_): v_ for k_, v_ in peaks["shared"].items()},
        "hbm": {"bound": "hbm", "achieved": hbm_f / (f_ms * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                "frac": hbm_f / (f_ms * 1e-3) / 1e9 / hbm_peak, "peak_source": f"MEASURED_PEAKS.json ({hbm_src})",
                "algorithmic_bytes": "compulsory HBM bytes: q,k,v,out once + coords once + lse"},
        "ms_per_launch": f_ms,
    }
    if b_ms is not None:
        # first pass: the forward's gathers again; gather pass: per sample two entries (one per map
        # row of its footprint), each a q row, a dout row, a 16-byte entry and an 8-byte scalar pair
        pass2_b = qh_rank * cfg.N * 2 * (2 * cfg.D * cfg.elem_size() + 24)
        two_pass = "bwd_gather" in plan_text
        on_chip_b = gather_b + (pass2_b if two_pass else 0)
        roofline["backward"] = {
            "ms": b_ms, "bound": roofline["bound"], "peak": gather_peak, "unit": "GB/s",
            "achieved": on_chip_b / (b_ms * 1e-3) / 1e9, "frac": on_chip_b / (b_ms * 1e-3) / 1e9 / gather_peak,
            "algorithmic_bytes": ("first pass: the forward's gather bytes; gather pass: query-heads x V*S x 2 entries x "
                                  "(2 rows + 24 bytes)" if two_pass else "the forward's gather bytes (scatter form)"),
            "kernels": "index build, first pass, gather pass: shares in profiles/bench_c5_launch_list.md",
            "hbm_GBps": hbm_b / (b_ms * 1e-3) / 1e9, "hbm_frac": hbm_b / (b_ms * 1e-3) / 1e9 / hbm_peak,
        }
        roofline["step"] = {"frac": (gather_b + on_chip_b) / ((f_ms + b_ms) * 1e-3) / 1e9 / gather_peak,
                            "what": "forward + backward on-chip gather bytes over their summed kernel time"}

    cpu, cpu_ref = None, None
    if not args.no_cpu_baseline and world == 1:
        cpu = cpu_sample(cfg, args.mode, 1, 0)
        cpu = {"value": cpu["value"], "unit": cpu["unit"], "cores": cpu["cores"], "kind": cpu["kind"],
               "sample": cpu["sample"]}
        cpu_ref = reference_torch_sample(cfg, args.mode)

    line = {
        "metric": METRIC if not fwd_only else METRIC_FWD,
        "value": value, "unit": "query-heads/sec", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16" if cfg.dtype == torch.bfloat16 else str(cfg.dtype).replace("torch.", ""),
        "data": "synthetic (seeded, drawn on the device)",
        "config": config_dict(cfg, args, world),
        "fwd": {"value": fwd_value, "unit": "query-heads/sec", "kernel_ms": f_ms} if fwd_value else None,
        "bwd_ms": b_ms,
        "roofline": roofline,
        "cpu_baseline": cpu,
        "cpu_baseline_reference": cpu_ref,
        "e2e": e2e,
        "gpu_launches": int(launches),
        "clocks": clocks,
        "plan": plan_text,
        "flags": args.flags,
        "gather": (None if world == 1 else
                   {"how": {"mirror": "the kernels store each result row also into rank 0's tensors over NVLink "
                                      "(CUDA IPC mapping)",
                            "peer": "device-to-device copies into rank 0's tensors (CUDA IPC mapping, copy engines)",
                            "nccl": "dist.gather over NCCL on a side stream",
                            "nccl_sync": "dist.gather over NCCL after each step's kernels",
                            "none": "no gather"}[gather_mode],
                    "verified": gather_ok}),
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

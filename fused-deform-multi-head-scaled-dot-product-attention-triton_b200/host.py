"""Host-buffer front end: the operator for callers whose tensors live in (pinned) host memory.

The reference keeps everything on the device, and so does ``deform_sdpa_triton``.  A caller
that starts from host tensors pays a host->device copy of q, k, v, coords (and dout) and a
device->host transfer of the results around the kernels.  Batch elements are independent
(reference ops/triton.py:47-51), so this front end cuts the batch into chunks and overlaps the
PCIe traffic of one chunk with the kernels of another: inputs by copies on their own stream,
results by stores of the kernels themselves into pinned host memory (or by copies on a third
stream when the result tensors are pageable).  Results are identical to the one-shot call: the
chunks are whole batch elements.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .op import backward_raw, forward_raw


def chunk_schedule(B: int, chunk: int):
    """Batch ranges of the pipeline.  The first chunks are small (1, 2, 4, ... batch elements) so
    that the kernels start after a short first copy, the last ones shrink the same way so that
    little is left to copy out when the last kernel ends, and the middle runs ``chunk`` elements
    at a time (large launches are the efficient ones)."""
    chunk = max(1, int(chunk))
    if B <= 8:
        # a short batch (a rank's share of a job spread over many GPUs): one element at a time keeps
        # the first copy in and the last copy out shortest, and with chunks alternating between two
        # compute streams the small launches cost little (measured best for 4 and 8 elements)
        return [(b, b + 1) for b in range(B)]
    ramp, size = [], 1
    while size < chunk:
        ramp.append(size)
        size *= 2
    while ramp and 2 * sum(ramp) > B:
        ramp.pop()
    middle = B - 2 * sum(ramp)
    sizes = list(ramp)
    while middle > 0:
        n = min(chunk, middle)
        sizes.append(n)
        middle -= n
    sizes += reversed(ramp)
    out, b0 = [], 0
    for n in sizes:
        out.append((b0, b0 + n))
        b0 += n
    return out


def measure_link(device, nbytes: int = 64 << 20, reps: int = 4):
    """Host link of one GPU under load: copies ``nbytes`` of pinned memory in and out at the same
    time (two streams), ``reps`` times, and returns ``(h2d_GBps, d2h_GBps)``.  The ranks of a job
    call it together (after a barrier), so that each sees what it gets while the others transfer
    too; on some boxes the GPUs do not all sit behind equally fast links, and ``balance_weights``
    turns the figures into a batch split."""
    dev = torch.device(device)
    h_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_out = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    torch.cuda.synchronize(dev)
    for timed in (False, True):                      # one untimed round first
        with torch.cuda.stream(s_in):
            ev[0].record()
            for _ in range(reps if timed else 1):
                d_in.copy_(h_in, non_blocking=True)
            ev[1].record()
        with torch.cuda.stream(s_out):
            ev[2].record()
            for _ in range(reps if timed else 1):
                h_out.copy_(d_out, non_blocking=True)
            ev[3].record()
        torch.cuda.synchronize(dev)
    return (reps * nbytes / (ev[0].elapsed_time(ev[1]) * 1e6),
            reps * nbytes / (ev[2].elapsed_time(ev[3]) * 1e6))


def balance_weights(links, in_bytes: float, out_bytes: float, compute_ms: float, tolerance: float = 1.15):
    """Batch-split weights for ``partition.shard_plan`` from every rank's ``measure_link`` result.

    A rank's pipeline runs at the pace of its slowest stage, so a batch element costs it
    ``max(compute_ms, in_bytes / h2d, out_bytes / d2h)`` (bytes per batch element, rates in GB/s)
    and its weight is the inverse.  Ranks within ``tolerance`` of one another get equal weights:
    an even split is not traded for measurement noise."""
    cost = [max(float(compute_ms), in_bytes / (h * 1e6), out_bytes / (d * 1e6)) for h, d in links]
    if max(cost) <= tolerance * min(cost):
        return [1.0] * len(cost)
    return [1.0 / c for c in cost]


class HostPipeline:
    """Forward (+ backward) of the operator on host tensors, chunked over the batch.

    Inputs travel by asynchronous copies on their own stream (q, k, v, coords ahead of dout, which
    only the backward needs), results by copies on a third stream (out as soon as the forward of
    its chunk is done).  With ``direct_results=True`` results that are PINNED host tensors are not
    copied: they are handed to the kernels as mirrors and the kernels store every result row into
    host memory over PCIe while they run.  That leaves nothing to copy out at the end, but the
    stores hold the kernels back (C5 on a B200: +4% kernel time), more than the short last copy
    of the tapered schedule costs, so it is not the default.
    """

    def __init__(self, device, W: int, H: int, sm_scale: float, chunk: int = 8, flags: Optional[int] = None,
                 direct_results: bool = False, sizes: Optional[Sequence[int]] = None, compute_streams: int = 2):
        self.device = torch.device(device)
        self.W, self.H, self.sm_scale = int(W), int(H), float(sm_scale)
        self.chunk = max(1, int(chunk))
        self.sizes = list(sizes) if sizes else None   # explicit chunk sizes (must add up to the batch)
        self.flags = flags
        self.direct_results = bool(direct_results)
        self.s_in = torch.cuda.Stream(self.device)
        # Chunks are independent, so consecutive chunks run on alternating compute streams: the last,
        # partly filled wave of one chunk's kernels then shares the GPU with the first wave of the
        # next chunk's instead of leaving SMs idle.
        self.s_comps = [torch.cuda.Stream(self.device) for _ in range(max(1, int(compute_streams)))]
        self.s_out = torch.cuda.Stream(self.device)
        # With ``time_transfers = True`` every run brackets its copies in and its copies out with
        # timing events; ``transfer_rates()`` then gives the bandwidth they reached.
        self.time_transfers = False
        self._marks = None

    def _to_device(self, hosts: Sequence[Optional[torch.Tensor]], b0: int, b1: int, s_comp):
        out = []
        for t in hosts:
            if t is None:
                out.append(None)
                continue
            d = t[b0:b1].to(self.device, non_blocking=True)
            d.record_stream(s_comp)
            out.append(d)
        return out

    def run(self, q, k, v, coords, dout=None, *, out, dq=None, dk=None, dv=None):
        """All arguments are host tensors (pinned for the copies to be asynchronous) with the
        operator's layouts; ``out`` (and ``dq, dk, dv`` when ``dout`` is given) receive the
        results.  Asynchronous with respect to the host; ordered after and before the work on
        the current stream of the device, like a kernel launch."""
        if q.is_cuda or out.is_cuda:
            raise ValueError("HostPipeline takes host tensors; use deform_sdpa_triton for device tensors")
        backward = dout is not None
        if backward and (dq is None or dk is None or dv is None):
            raise ValueError("dq, dk, dv host tensors are needed when dout is given")
        B = q.shape[0]
        results = {"out": out, "dq": dq, "dk": dk, "dv": dv} if backward else {"out": out}
        # a result the kernels can store to directly: pinned, contiguous, of the inputs' type
        direct = {n: self.direct_results and t.is_pinned() and t.is_contiguous() and t.dtype == q.dtype
                  and t.shape == q.shape for n, t in results.items()}
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, *self.s_comps, self.s_out):
            s.wait_event(start)
        marks = None
        if self.time_transfers:
            marks = {n: torch.cuda.Event(enable_timing=True) for n in ("in0", "in1", "out0", "out1")}
            marks["in0"].record(self.s_in)
            marks["bytes_in"] = sum(t.numel() * t.element_size() for t in (q, k, v, coords, dout) if t is not None)
            marks["bytes_out"] = sum(t.numel() * t.element_size() for n, t in results.items() if not direct[n])
            first_out = True
        if self.sizes is not None:
            if sum(self.sizes) != B or min(self.sizes) < 1:
                raise ValueError(f"chunk sizes {self.sizes} do not cover a batch of {B}")
            bounds = [sum(self.sizes[:i]) for i in range(len(self.sizes) + 1)]
            schedule = list(zip(bounds[:-1], bounds[1:]))
        else:
            schedule = chunk_schedule(B, self.chunk)
        for step, (b0, b1) in enumerate(schedule):
            s_comp = self.s_comps[step % len(self.s_comps)]
            with torch.cuda.stream(self.s_in):
                d_q, d_k, d_v, d_c = self._to_device((q, k, v, coords), b0, b1, s_comp)
                ready_fwd = torch.cuda.Event()
                ready_fwd.record(self.s_in)
                (d_do,) = self._to_device((dout,), b0, b1, s_comp)
                ready_bwd = torch.cuda.Event()
                ready_bwd.record(self.s_in)
            mirror = {n: results[n][b0:b1] for n in results if direct[n]}
            copies = []
            s_comp.wait_event(ready_fwd)
            with torch.cuda.stream(s_comp):
                o, lse = forward_raw(d_q, d_k, d_v, d_c, self.W, self.H, self.sm_scale, flags=self.flags,
                                     out_mirror=mirror.get("out"))
                if not direct["out"]:
                    fwd_done = torch.cuda.Event()
                    fwd_done.record(s_comp)
                    copies.append((fwd_done, out, o))
                if backward:
                    s_comp.wait_event(ready_bwd)
                    grads = backward_raw(d_q, d_k, d_v, d_c, o, lse, d_do, self.W, self.H, self.sm_scale,
                                         flags=self.flags,
                                         mirrors={n: t for n, t in mirror.items() if n != "out"} or None)
                    bwd_done = torch.cuda.Event()
                    bwd_done.record(s_comp)
                    copies += [(bwd_done, results[n], g) for n, g in zip(("dq", "dk", "dv"), grads) if not direct[n]]
            with torch.cuda.stream(self.s_out):
                for event, host, dev_t in copies:
                    self.s_out.wait_event(event)
                    if marks is not None and first_out:
                        marks["out0"].record(self.s_out)
                        first_out = False
                    dev_t.record_stream(self.s_out)
                    host[b0:b1].copy_(dev_t, non_blocking=True)
        if marks is not None:
            marks["in1"].record(self.s_in)
            marks["out1"].record(self.s_out)
            self._marks = marks
        for s in (*self.s_comps, self.s_out):
            end = torch.cuda.Event()
            end.record(s)
            cur.wait_event(end)
        return out

    def transfer_rates(self):
        """Of the last run with ``time_transfers`` set (synchronise first): bytes copied in / out
        over the time from the start of the first such copy to the end of the last one, in GB/s.
        The copies out wait for the kernels that produce their data, so that window also holds
        those waits: the figure is what the pipeline sustained, not the link's peak."""
        m = self._marks
        if m is None:
            return None
        t_in = m["in0"].elapsed_time(m["in1"]) * 1e-3
        rates = {"h2d_GBps": m["bytes_in"] / t_in / 1e9 if t_in > 0 else None, "h2d_window_ms": t_in * 1e3}
        if m["bytes_out"]:
            t_out = m["out0"].elapsed_time(m["out1"]) * 1e-3
            rates.update(d2h_GBps=m["bytes_out"] / t_out / 1e9 if t_out > 0 else None, d2h_window_ms=t_out * 1e3)
        return rates

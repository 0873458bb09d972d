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


def measure_link(device, nbytes: int = 64 << 20, reps: int = 8):
    """Host link of one GPU under load: copies ``nbytes`` of pinned memory in and out at the same
    time (two streams), ``reps`` times, and returns ``(h2d_GBps, d2h_GBps)``, each the median over
    the repetitions.  The ranks of a job call it together (after a barrier), so that each sees
    what it gets while the others transfer too; on some boxes the GPUs do not all sit behind
    equally fast links, and ``balance_weights`` turns the figures into a batch split."""
    dev = torch.device(device)
    h_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_out = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    torch.cuda.synchronize(dev)
    marks_in = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 2)]
    marks_out = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 2)]
    with torch.cuda.stream(s_in):
        for i in range(reps + 1):                    # the first repetition is not counted
            marks_in[i].record()
            d_in.copy_(h_in, non_blocking=True)
        marks_in[reps + 1].record()
    with torch.cuda.stream(s_out):
        for i in range(reps + 1):
            marks_out[i].record()
            h_out.copy_(d_out, non_blocking=True)
        marks_out[reps + 1].record()
    torch.cuda.synchronize(dev)

    def median_rate(marks):
        ms = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(1, reps + 1))
        mid = ms[len(ms) // 2] if len(ms) % 2 else 0.5 * (ms[len(ms) // 2 - 1] + ms[len(ms) // 2])
        return nbytes / (mid * 1e6)
    return median_rate(marks_in), median_rate(marks_out)


def _element_costs(links, in_bytes: float, out_bytes: float, compute_ms: float):
    return [max(float(compute_ms), in_bytes / (h * 1e6), out_bytes / (d * 1e6)) for h, d in links]


def weights_from_costs(costs: Sequence[float], tolerance: float = 1.25):
    """Batch-split weights for ``partition.shard_plan`` from what one batch element costs every
    rank (any unit; e.g. the time of a calibration run of its ``HostPipeline`` over its share,
    divided by the share).  The weight is the inverse cost.  Ranks whose costs lie within
    ``tolerance`` of one another form a group and share the group's mean cost: an even split is
    not traded for measurement noise, neither over the whole job nor inside a group."""
    cost = [float(c) for c in costs]
    if not cost or min(cost) <= 0.0:
        raise ValueError("costs must be positive")
    order = sorted(range(len(cost)), key=lambda r: cost[r])
    shared = [0.0] * len(cost)
    i = 0
    while i < len(order):
        j = i
        while j + 1 < len(order) and cost[order[j + 1]] <= tolerance * cost[order[i]]:
            j += 1
        group = order[i:j + 1]
        mean = sum(cost[r] for r in group) / len(group)
        for r in group:
            shared[r] = mean
        i = j + 1
    return [1.0 / c for c in shared]


def balance_weights(links, in_bytes: float, out_bytes: float, compute_ms: float, tolerance: float = 1.25):
    """The same from every rank's ``measure_link`` result, without running the operator: a rank's
    pipeline runs at the pace of its slowest stage, so a batch element costs it
    ``max(compute_ms, in_bytes / h2d, out_bytes / d2h)`` (bytes per batch element, rates in GB/s).
    A probe of bare copies does not see how the copies of a real run interleave with the kernels;
    where the job can afford a calibration step, ``weights_from_costs`` of measured step times is
    the better input."""
    return weights_from_costs(_element_costs(links, in_bytes, out_bytes, compute_ms), tolerance)


def suggest_head_parts(link, in_bytes: float, out_bytes: float, compute_ms: float, heads: int, parts: int = 4) -> int:
    """``head_parts`` for a ``HostPipeline`` behind ``link`` (a ``measure_link`` result): cutting
    the first and last batch element into head groups pays when the copies of a batch element
    take longer than its kernels (measured: 8 ranks on a box with shared links, -3%), and costs
    a little when they do not (one rank on a fast link, +0.3%)."""
    if heads < parts:
        return 1
    return parts if _element_costs([link], in_bytes, out_bytes, compute_ms)[0] > float(compute_ms) else 1


def pipeline_schedule(B: int, Hh: int, *, chunk: int = 8, sizes: Optional[Sequence[int]] = None, head_parts: int = 1):
    """Chunks of a ``HostPipeline`` run as (b0, b1, h0, h1): ``chunk_schedule`` (or the given batch
    ``sizes``) over the batch, with the first and the last chunk, when they are single batch
    elements, cut into ``head_parts`` groups of heads (as even as the head count allows)."""
    if sizes is not None:
        if sum(sizes) != B or min(sizes) < 1:
            raise ValueError(f"chunk sizes {list(sizes)} do not cover a batch of {B}")
        bounds = [sum(sizes[:i]) for i in range(len(sizes) + 1)]
        batches = list(zip(bounds[:-1], bounds[1:]))
    else:
        batches = chunk_schedule(B, chunk)
    parts = min(max(1, int(head_parts)), Hh)
    chunks = []
    for i, (b0, b1) in enumerate(batches):
        if parts > 1 and b1 - b0 == 1 and i in (0, len(batches) - 1):
            cuts = [Hh * j // parts for j in range(parts + 1)]
            chunks += [(b0, b1, h0, h1) for h0, h1 in zip(cuts[:-1], cuts[1:]) if h1 > h0]
        else:
            chunks.append((b0, b1, 0, Hh))
    return chunks


class HostPipeline:
    """Forward (+ backward) of the operator on host tensors, chunked over the batch.

    Inputs travel by asynchronous copies on their own stream (q, k, v, coords ahead of dout, which
    only the backward needs), results by copies on a third stream (out as soon as the forward of
    its chunk is done).  With ``direct_results=True`` results that are PINNED host tensors are not
    copied: they are handed to the kernels as mirrors and the kernels store every result row into
    host memory over PCIe while they run.  That leaves nothing to copy out at the end, but the
    stores hold the kernels back (C5 on a B200: +4% kernel time), more than the short last copy
    of the tapered schedule costs, so it is not the default.

    ``head_parts`` > 1 cuts the first and the last batch element further, into that many groups of
    heads ((batch, head) slices are independent too): the kernels start after a copy of a fraction
    of an element and only as much is left to copy out when they end.  It pays where the host link
    is slow against the kernels (several ranks sharing a box's links); a head group of one element
    is V separate blocks of every tensor, so it costs V small copies per tensor and direction.
    """

    def __init__(self, device, W: int, H: int, sm_scale: float, chunk: int = 8, flags: Optional[int] = None,
                 direct_results: bool = False, sizes: Optional[Sequence[int]] = None, compute_streams: int = 2,
                 head_parts: int = 1):
        self.device = torch.device(device)
        self.head_parts = max(1, int(head_parts))
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

    def _heads_to_device(self, hosts: Sequence[Optional[torch.Tensor]], b: int, h0: int, h1: int, s_comp):
        """Heads h0..h1 of batch element b as compact device tensors [1, V, h1-h0, L, D]: one copy
        per view (each view's run of heads is contiguous on both sides)."""
        out = []
        for t in hosts:
            if t is None:
                out.append(None)
                continue
            d = torch.empty((1, t.shape[1], h1 - h0) + tuple(t.shape[3:]), dtype=t.dtype, device=self.device)
            for view in range(t.shape[1]):
                d[0, view].copy_(t[b, view, h0:h1], non_blocking=True)
            d.record_stream(s_comp)
            out.append(d)
        return out

    def schedule(self, B: int, Hh: int):
        """Chunks as (b0, b1, h0, h1)."""
        return pipeline_schedule(B, Hh, chunk=self.chunk, sizes=self.sizes,
                                 head_parts=1 if self.direct_results else self.head_parts)

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
        Hh = q.shape[2]
        kept_coords = (None, None)       # (batch element, its coordinates on the device): shared by head groups
        for step, (b0, b1, h0, h1) in enumerate(self.schedule(B, Hh)):
            s_comp = self.s_comps[step % len(self.s_comps)]
            whole = h0 == 0 and h1 == Hh
            with torch.cuda.stream(self.s_in):
                if whole:
                    d_q, d_k, d_v, d_c = self._to_device((q, k, v, coords), b0, b1, s_comp)
                else:
                    d_q, d_k, d_v = self._heads_to_device((q, k, v), b0, h0, h1, s_comp)
                    if kept_coords[0] != b0:
                        kept_coords = (b0, self._to_device((coords,), b0, b1, s_comp)[0])
                    d_c = kept_coords[1]
                    d_c.record_stream(s_comp)
                ready_fwd = torch.cuda.Event()
                ready_fwd.record(self.s_in)
                if whole:
                    (d_do,) = self._to_device((dout,), b0, b1, s_comp)
                else:
                    (d_do,) = self._heads_to_device((dout,), b0, h0, h1, s_comp)
                ready_bwd = torch.cuda.Event()
                ready_bwd.record(self.s_in)
            mirror = {n: results[n][b0:b1] for n in results if direct[n]} if whole else {}
            copies = []
            s_comp.wait_event(ready_fwd)
            with torch.cuda.stream(s_comp):
                o, lse = forward_raw(d_q, d_k, d_v, d_c, self.W, self.H, self.sm_scale, flags=self.flags,
                                     out_mirror=mirror.get("out"))
                if "out" not in mirror:
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
                    copies += [(bwd_done, results[n], g) for n, g in zip(("dq", "dk", "dv"), grads) if n not in mirror]
            with torch.cuda.stream(self.s_out):
                for event, host, dev_t in copies:
                    self.s_out.wait_event(event)
                    if marks is not None and first_out:
                        marks["out0"].record(self.s_out)
                        first_out = False
                    dev_t.record_stream(self.s_out)
                    if whole:
                        host[b0:b1].copy_(dev_t, non_blocking=True)
                    else:
                        for view in range(dev_t.shape[1]):
                            host[b0, view, h0:h1].copy_(dev_t[0, view], non_blocking=True)
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

"""(batch, head) partitioner: shards the operator over the GPUs of one box.

The reference has no multi-device code.  Every (batch, head) slice of the operator is
independent -- it reads only ``q, k, v[b, :, h]`` and ``coords[b]`` and writes only
``out/dq/dk/dv[b, :, h]`` (reference ops/triton.py:47-51, 97, 246-257) -- so the work is
split with no communication on the compute path; the only exchange is the final
gather of the outputs onto one rank.

Batch is split first: with the [B, V, Hh, L, D] layout a batch shard of every tensor
(coordinates included) is one contiguous block.  Heads are split only when there are
fewer batch elements than ranks; a head shard needs the whole coords[b].
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    """Half-open ranges of batch elements and heads owned by one rank."""
    b0: int
    b1: int
    h0: int
    h1: int

    @property
    def empty(self) -> bool:
        return self.b1 <= self.b0 or self.h1 <= self.h0

    def units(self) -> int:
        return max(0, self.b1 - self.b0) * max(0, self.h1 - self.h0)


def _split(n: int, parts: int) -> List[range]:
    base, extra = divmod(n, parts)
    out, lo = [], 0
    for i in range(parts):
        hi = lo + base + (1 if i < extra else 0)
        out.append(range(lo, hi))
        lo = hi
    return out


def _split_weighted(n: int, weights: Sequence[float]) -> List[range]:
    """Contiguous ranges of ``n`` items in proportion to ``weights`` (largest remainders first;
    every part with a positive weight gets at least one item when there are enough)."""
    w = [max(0.0, float(x)) for x in weights]
    total = sum(w)
    if total <= 0.0:
        raise ValueError("weights must have a positive sum")
    ideal = [n * x / total for x in w]
    counts = [int(x) for x in ideal]
    if n >= sum(1 for x in w if x > 0.0):
        counts = [max(c, 1) if x > 0.0 else 0 for c, x in zip(counts, w)]
    # hand out what is left (or take back what the minimum of one overspent) by remainder
    order = sorted(range(len(w)), key=lambda i: ideal[i] - counts[i], reverse=True)
    i = 0
    while sum(counts) < n:
        counts[order[i % len(order)]] += 1
        i += 1
    i = 0
    while sum(counts) > n:
        j = order[-1 - (i % len(order))]
        if counts[j] > 1:
            counts[j] -= 1
        i += 1
    out, lo = [], 0
    for c in counts:
        out.append(range(lo, lo + c))
        lo += c
    return out


def shard_plan(B: int, Hh: int, world: int, weights: Optional[Sequence[float]] = None) -> List[Shard]:
    """One Shard per rank.  Batch-major; heads are split only when B < world.

    ``weights`` (one positive number per rank, e.g. each rank's measured throughput) splits the
    batch in their proportion instead of evenly -- for boxes whose GPUs do not all sit behind
    equally fast host links.  It needs B >= world."""
    if B <= 0 or Hh <= 0 or world <= 0:
        raise ValueError("B, Hh and world must be positive")
    if weights is not None:
        if len(weights) != world:
            raise ValueError("one weight per rank")
        if B < world:
            raise ValueError("a weighted plan splits the batch only: it needs B >= world")
        return [Shard(r.start, r.stop, 0, Hh) for r in _split_weighted(B, weights)]
    if B >= world:
        return [Shard(r.start, r.stop, 0, Hh) for r in _split(B, world)]
    # fewer batch elements than ranks: give each batch element a group of ranks that
    # split its heads
    groups = _split(world, B)          # ranks per batch element
    plan: List[Optional[Shard]] = [None] * world
    for b, ranks in enumerate(groups):
        heads = _split(Hh, len(ranks))
        for r, hr in zip(ranks, heads):
            plan[r] = Shard(b, b + 1, hr.start, hr.stop)
    return [s if s is not None else Shard(0, 0, 0, 0) for s in plan]


def slice_inputs(shard: Shard, q, k, v, coords, *more):
    """Views of the full tensors for one shard ([B, V, Hh, L, D] and coords [B, ...])."""
    sl = (slice(shard.b0, shard.b1), slice(None), slice(shard.h0, shard.h1))
    extra = tuple(t[sl] if t is not None else None for t in more)
    return (q[sl], k[sl], v[sl], coords[shard.b0:shard.b1]) + extra


def gather_to_root(local: torch.Tensor, plan: Sequence[Shard], full_shape, root: int = 0,
                   group=None, out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Gather every rank's ``[b, V, h, L, D]`` shard into the full tensor on ``root``.

    Returns the full tensor on ``root`` and ``None`` elsewhere.  ``out`` (root only) is an
    optional preallocated result, for callers that gather every step.  Equal batch shards go
    through one ``dist.gather`` straight into views of the preallocated result (batch
    shards are contiguous blocks of it); anything else uses point-to-point copies.
    """
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    if len(plan) != world:
        raise ValueError("plan does not match the process group")
    full = None
    if rank == root:
        if out is not None:
            if tuple(out.shape) != tuple(full_shape) or out.dtype != local.dtype or not out.is_contiguous():
                raise ValueError("out does not match the full tensor")
            full = out
        else:
            full = torch.empty(full_shape, dtype=local.dtype, device=local.device)
    Hh = full_shape[2]
    batch_only = all(s.h0 == 0 and s.h1 == Hh for s in plan)
    equal = batch_only and len({s.b1 - s.b0 for s in plan}) == 1
    local = local.contiguous()
    if equal:
        views = [full[s.b0:s.b1] for s in plan] if rank == root else None
        dist.gather(local, views, dst=root, group=group)
        return full
    if rank == root:
        reqs = []
        staging = []
        for r, s in enumerate(plan):
            if s.empty:
                continue
            dst = full[s.b0:s.b1, :, s.h0:s.h1]
            if r == root:
                dst.copy_(local)
                continue
            if dst.is_contiguous():
                reqs.append(dist.irecv(dst, src=r, group=group))
            else:
                tmp = torch.empty(dst.shape, dtype=dst.dtype, device=dst.device)
                staging.append((dst, tmp))
                reqs.append(dist.irecv(tmp, src=r, group=group))
        for req in reqs:
            req.wait()
        for dst, tmp in staging:
            dst.copy_(tmp)
        return full
    if not plan[rank].empty:
        dist.send(local, dst=root, group=group)
    return None


def run_sharded(fn: Callable, q, k, v, coords, *, plan: Sequence[Shard], rank: int):
    """Apply ``fn(q, k, v, coords)`` to this rank's shard of full-size inputs."""
    s = plan[rank]
    if s.empty:
        return None
    qs, ks, vs, cs = slice_inputs(s, q, k, v, coords)
    return fn(qs.contiguous(), ks.contiguous(), vs.contiguous(), cs.contiguous())


class ShardError(RuntimeError):
    """A shard of a sharded call failed on some rank.  ``failures`` maps rank -> message."""

    def __init__(self, failures):
        self.failures = dict(failures)
        detail = "; ".join(f"rank {r}: {m}" for r, m in sorted(self.failures.items()))
        super().__init__(f"sharded call failed on {len(self.failures)} rank(s): {detail}")


def run_sharded_checked(fn: Callable, q, k, v, coords, *, plan: Sequence[Shard], rank: int, group=None,
                        after: Optional[Callable] = None):
    """``run_sharded`` for jobs that go on to a collective (the gather of the results): every rank
    learns whether any shard failed BEFORE anybody enters that collective.

    ``fn`` runs under try/except; ``after``, if given, runs next on the ranks whose ``fn``
    succeeded (e.g. a check of the device's error record, which needs a synchronise and is
    therefore optional).  The ranks then exchange one small status object.  If any rank failed,
    every rank raises :class:`ShardError` naming the failed ranks and their messages, so that no
    rank is left waiting in a gather for a peer that has given up; otherwise the local result is
    returned as from ``run_sharded``."""
    failure = None
    local = None
    try:
        local = run_sharded(fn, q, k, v, coords, plan=plan, rank=rank)
        if after is not None:
            after(local)
    except Exception as exc:  # noqa: BLE001  (reported to every rank below)
        failure = f"{type(exc).__name__}: {exc}"
    world = dist.get_world_size(group)
    statuses = [None] * world
    dist.all_gather_object(statuses, failure, group=group)
    failures = {r: m for r, m in enumerate(statuses) if m is not None}
    if failures:
        raise ShardError(failures)
    return local


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


class _DeviceBytes:
    """A run of device memory, described the way ``torch.as_tensor`` understands."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _alias_device_memory(ptr: int, nbytes: int, devices) -> torch.Tensor:
    """A uint8 tensor over ``[ptr, ptr + nbytes)``.  torch attributes a mapped block either to the
    device it was mapped on or to the one that owns the memory; naming the wrong one makes
    ``as_tensor`` copy, so the candidates are tried until the tensor's address is the block's."""
    for dev in devices:
        try:
            t = torch.as_tensor(_DeviceBytes(ptr, nbytes), device=dev)
        except Exception:  # noqa: BLE001  (a device torch does not accept for this pointer)
            continue
        if t.data_ptr() == ptr:
            return t
    raise RuntimeError("torch does not alias the mapped block")


class PeerGather:
    """The root's result tensors, mapped into every rank of the box.

    The root allocates the full result tensors once and shares them with the other ranks through
    CUDA IPC handles (all ranks must be processes on one machine with peer access between their
    GPUs).  ``shard_views()`` returns this rank's batch slice of each of them, in the root's
    memory: passed as mirrors to ``forward_raw`` / ``backward_raw`` they make the kernels store
    their rows there as they produce them, so that the job's final gather costs no pass of its
    own -- the kernels of this library fill every SM, and a gather made of NCCL send/recv kernels
    beside them is starved of SMs, one behind them adds its full time.  The peer mapping is only
    ever written, never read.

    ``push(index, shard)`` is the other way to fill the root's tensors: a device-to-device copy on
    this object's own stream (copy engines, no SM), ``wait()`` makes the current stream wait for it.
    Either way a barrier after the last step tells the root that everybody's data has landed in
    ``results`` (root only).
    """

    def __init__(self, specs, plan: Sequence[Shard], device, root: int = 0, group=None):
        import ctypes
        from . import cabi
        self.rank = dist.get_rank(group)
        self.root = root
        self.plan = plan
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(self.device)
        self.group = group
        self._mapped = None
        Hh = specs[0][0][2]
        if not all(s.h0 == 0 and s.h1 == Hh for s in plan):
            raise ValueError("PeerGather handles batch shards (every rank owns all heads)")
        # one flat block holds all result tensors: one export, one mapping per process
        sizes = [(_numel(shape) * torch.empty(0, dtype=dtype).element_size() + 255) // 256 * 256 for shape, dtype in specs]
        total = sum(sizes)
        L = cabi.lib()
        payload, flat, failure = None, None, None
        if self.rank == root:
            try:
                flat = torch.empty(total, dtype=torch.uint8, device=self.device)
                handle = ctypes.create_string_buffer(cabi.PEER_HANDLE_BYTES)
                offset = ctypes.c_size_t()
                cabi.check(L.dsdpa_peer_export(ctypes.c_void_p(flat.data_ptr()), self.device.index, handle,
                                               ctypes.byref(offset)))
                payload = (handle.raw, offset.value, self.device.index)
            except Exception as exc:  # noqa: BLE001  (reported to every rank below)
                failure = exc
        box = [payload]
        dist.broadcast_object_list(box, src=root, group=group)
        if self.rank != root and box[0] is not None:
            try:
                handle, offset, root_device = box[0]
                ptr = ctypes.c_void_p()
                # mapped with THIS rank's device current: its kernels are the ones that store there
                cabi.check(L.dsdpa_peer_import(handle, offset, self.device.index, ctypes.byref(ptr)))
                self._mapped = (ptr.value, offset)
                flat = _alias_device_memory(ptr.value, total, (self.device, torch.device("cuda", root_device)))
            except Exception as exc:  # noqa: BLE001
                failure = exc
        # all ranks succeed or all raise (nobody is left waiting in a later collective)
        ok = torch.tensor([0 if (failure is not None or flat is None) else 1], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if ok.item() == 0:
            self.close()
            raise RuntimeError(f"the root's result block could not be shared with every rank: {failure!r}")
        self._flat = flat
        self.targets, lo = [], 0
        for (shape, dtype), nbytes in zip(specs, sizes):
            n = _numel(shape) * torch.empty(0, dtype=dtype).element_size()
            self.targets.append(flat[lo:lo + n].view(dtype).view(shape))
            lo += nbytes
        self.results = self.targets if self.rank == root else None
        dist.barrier(group)

    def close(self) -> None:
        """Unmap the root's block (non-root ranks).  The views handed out become invalid."""
        if self._mapped is not None:
            from . import cabi
            ptr, offset = self._mapped
            self._mapped = None
            self.targets = self._flat = None
            cabi.lib().dsdpa_peer_release(ptr, offset, self.device.index)

    def shard_views(self):
        """This rank's batch slice of every result tensor of the root (contiguous views)."""
        s = self.plan[self.rank]
        return [t[s.b0:s.b1] for t in self.targets]

    def push(self, index: int, shard: torch.Tensor) -> None:
        s = self.plan[self.rank]
        if s.empty:
            return
        cur = torch.cuda.current_stream(self.device)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            shard.record_stream(self.stream)
            self.targets[index][s.b0:s.b1].copy_(shard, non_blocking=True)

    def wait(self) -> None:
        torch.cuda.current_stream(self.device).wait_stream(self.stream)

"""The (batch, head) partitioner on CPU: plan arithmetic, and a world_size-2 gloo run in
which every rank computes its shard with the CPU oracle (standing in for the GPU kernels)
and the root gathers the result, which must equal the unsharded computation."""
import os
import socket
import sys
from dataclasses import replace
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import ops

ROOT = Path(__file__).resolve().parent.parent
part = ops.backend.partition


def test_plan_batch_first():
    plan = part.shard_plan(32, 16, 8)
    assert [(s.b0, s.b1, s.h0, s.h1) for s in plan] == [(4 * r, 4 * r + 4, 0, 16) for r in range(8)]
    plan = part.shard_plan(5, 8, 2)
    assert [(s.b0, s.b1) for s in plan] == [(0, 3), (3, 5)]
    assert sum(s.units() for s in plan) == 5 * 8


def test_plan_splits_heads_only_when_batches_run_out():
    plan = part.shard_plan(2, 16, 8)
    assert sum(s.units() for s in plan) == 2 * 16
    assert all(s.b1 - s.b0 == 1 for s in plan)
    covered = set()
    for s in plan:
        for b in range(s.b0, s.b1):
            for h in range(s.h0, s.h1):
                assert (b, h) not in covered
                covered.add((b, h))
    assert len(covered) == 32
    plan = part.shard_plan(1, 2, 4)     # more ranks than units: some ranks stay empty
    assert sum(s.units() for s in plan) == 2
    assert sum(1 for s in plan if s.empty) == 2


def test_weighted_plan_splits_the_batch_in_proportion():
    sizes = lambda plan: [s.b1 - s.b0 for s in plan]
    assert sizes(part.shard_plan(32, 16, 8, weights=[1.0] * 8)) == [4] * 8
    # four ranks behind links of half the rate: 1/6.2 against 1/3.8 per batch element
    plan = part.shard_plan(32, 16, 8, weights=[1 / 6.2] * 4 + [1 / 3.8] * 4)
    assert sizes(plan) == [3, 3, 3, 3, 5, 5, 5, 5]
    assert [s.b0 for s in plan] == [0, 3, 6, 9, 12, 17, 22, 27] and plan[-1].b1 == 32
    assert all(s.h0 == 0 and s.h1 == 16 for s in plan)
    # nobody with a positive weight is left without work while there is enough of it
    assert sizes(part.shard_plan(8, 4, 8, weights=[1, 1, 1, 1, 9, 9, 9, 9])) == [1] * 8
    assert sum(sizes(part.shard_plan(9, 4, 8, weights=[1, 1, 1, 1, 9, 9, 9, 9]))) == 9
    assert sizes(part.shard_plan(32, 4, 2, weights=[1, 3])) == [8, 24]
    with pytest.raises(ValueError):
        part.shard_plan(2, 16, 8, weights=[1.0] * 8)       # a weighted plan never splits heads
    with pytest.raises(ValueError):
        part.shard_plan(8, 16, 2, weights=[1.0] * 3)
    with pytest.raises(ValueError):
        part.shard_plan(8, 16, 2, weights=[0.0, 0.0])


def test_balance_weights_follow_the_slowest_stage():
    host = ops.backend.host
    sizes = lambda w: [s.b1 - s.b0 for s in part.shard_plan(32, 16, len(w), weights=w)]
    # (h2d, d2h) GB/s per rank; 64 MB in and 51 MB out per batch element, 3.75 ms of kernels
    links = [(11.7, 8.2)] * 4 + [(21.3, 13.5)] * 4
    w = host.balance_weights(links, 64.2e6, 51.4e6, 3.75)
    assert w[0] == pytest.approx(1 / (51.4 / 8.2), rel=1e-6)        # copy-out bound
    assert w[4] == pytest.approx(1 / (51.4 / 13.5), rel=1e-6)
    assert sizes(w) == [3, 3, 3, 3, 5, 5, 5, 5]
    # like links measured with some noise form groups that share one weight: the split inside a
    # group stays even (figures of a run on an 8-GPU box)
    noisy = [(10.9, 8.3), (9.5, 7.2), (9.5, 7.2), (9.4, 7.1), (15.2, 11.6), (16.2, 12.3), (16.2, 12.5), (16.3, 12.4)]
    w = host.balance_weights(noisy, 64.2e6, 51.4e6, 3.75)
    assert len(set(w[:4])) == 1 and len(set(w[4:])) == 1 and w[4] > w[0]
    assert sizes(w) == [3, 3, 3, 3, 5, 5, 5, 5]
    # an outlier falls out of its group but the slow links still get the smaller shares
    noisy = [(8.6, 9.1), (10.5, 11.1), (10.6, 11.1), (10.9, 11.4), (14.4, 15.9), (15.5, 17.1), (13.4, 14.5), (14.7, 16.1)]
    shares = sizes(host.balance_weights(noisy, 64.2e6, 51.4e6, 3.75))
    assert sum(shares) == 32 and max(shares[:4]) <= min(shares[4:]) and shares[4:] == [5, 5, 5, 5]
    # alike within the tolerance: an even split; fast links: the kernels set the pace for everybody
    for links in ([(20.0, 13.0), (21.0, 13.5)], [(50.0, 50.0), (25.0, 25.0)]):
        w = host.balance_weights(links, 64.2e6, 51.4e6, 3.75)
        assert w[0] == w[1] and sizes(w) == [16, 16]
    # head groups at the ends of the batch only behind a link that is slower than the kernels
    assert host.suggest_head_parts((9.5, 7.2), 64.2e6, 51.4e6, 3.75, 16) == 4
    assert host.suggest_head_parts((53.0, 50.0), 64.2e6, 51.4e6, 3.6, 16) == 1
    assert host.suggest_head_parts((9.5, 7.2), 64.2e6, 51.4e6, 3.75, 2) == 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, Hh, result_path, weights=None):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import ops as _ops
    from oracle import oracle as orc
    inp, prt = _ops.backend.inputs, _ops.backend.partition
    cfg = replace(inp.CONFIGS["C2"], B=B, Hh=Hh, V=2, S=4, W=6, H=5)
    q, k, v, coords, _ = inp.make_inputs(cfg)
    plan = prt.shard_plan(cfg.B, cfg.Hh, world, weights=weights)

    def fn(qs, ks, vs, cs):
        return orc.forward(qs, ks, vs, cs, cfg.W, cfg.H, cfg.sm_scale, nthreads=1)[0]

    local = prt.run_sharded(fn, q, k, v, coords, plan=plan, rank=rank)
    if local is None:
        s = plan[rank]
        local = torch.empty(0, cfg.V, max(s.h1 - s.h0, 0), cfg.L, cfg.D)
    full = prt.gather_to_root(local, plan, tuple(q.shape), root=0)
    if rank == 0:
        ref = orc.forward(q, k, v, coords, cfg.W, cfg.H, cfg.sm_scale, nthreads=1)[0]
        torch.save({"equal": bool(torch.equal(full, ref)), "shape": tuple(full.shape)}, result_path)
    else:
        assert full is None
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("B,Hh", [(4, 2), (3, 2), (1, 4)])
def test_two_rank_sharded_run_matches_unsharded(tmp_path, B, Hh):
    from oracle import oracle as orc
    orc.build()
    result = tmp_path / "result.pt"
    mp.spawn(_worker, args=(2, _free_port(), B, Hh, str(result)), nprocs=2, join=True)
    out = torch.load(result)
    assert out["equal"], "gathered sharded output differs from the unsharded one"
    assert out["shape"][0] == B and out["shape"][2] == Hh


def test_two_rank_run_with_a_weighted_plan_matches_unsharded(tmp_path):
    from oracle import oracle as orc
    orc.build()
    result = tmp_path / "result.pt"
    mp.spawn(_worker, args=(2, _free_port(), 4, 2, str(result), [1.0, 3.0]), nprocs=2, join=True)
    out = torch.load(result)
    assert out["equal"], "gathered output of the 1 + 3 split differs from the unsharded one"


def _failing_worker(rank, world, port, result_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    import ops as _ops
    inp, prt = _ops.backend.inputs, _ops.backend.partition
    cfg = replace(inp.CONFIGS["C2"], B=2, Hh=2, V=2, S=2, W=4, H=3)
    q, k, v, coords, _ = inp.make_inputs(cfg)
    plan = prt.shard_plan(cfg.B, cfg.Hh, world)

    def fn(qs, ks, vs, cs):
        if rank == 1:
            raise ValueError("injected failure of this shard")
        return qs.clone()

    outcome = {"raised": False, "failed_ranks": None, "entered_gather": False}
    try:
        local = prt.run_sharded_checked(fn, q, k, v, coords, plan=plan, rank=rank)
        outcome["entered_gather"] = True
        prt.gather_to_root(local, plan, tuple(q.shape), root=0)
    except prt.ShardError as err:
        outcome["raised"] = True
        outcome["failed_ranks"] = sorted(err.failures)
        outcome["message"] = str(err)
    # nobody is stuck in a collective: the group still works for everybody afterwards
    dist.barrier()
    torch.save(outcome, os.path.join(result_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


def test_a_failed_shard_reaches_every_rank_before_the_gather(tmp_path):
    """One rank's shard raises: every rank gets a ShardError naming it, no rank enters the
    gather, and the process group is still usable afterwards (the barrier completes)."""
    mp.spawn(_failing_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        out = torch.load(tmp_path / f"rank{rank}.pt")
        assert out["raised"] and not out["entered_gather"]
        assert out["failed_ranks"] == [1]
        assert "injected failure" in out["message"] and "rank 1" in out["message"]

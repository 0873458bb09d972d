"""Two processes, two GPUs: the root's result block is mapped into the other rank, and that
rank's kernels store their results into it (mirrors) -- the gather of a sharded job.

Needs two GPUs with peer access; skipped elsewhere.  The host-side logic of the partitioner is
covered on CPU by test_partition_gloo.py.
"""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, failures) -> None:
    try:
        sys.path.insert(0, str(ROOT))
        sys.path.insert(0, str(ROOT / "tests"))
        import torch.distributed as dist
        import ops
        from conftest import load_golden
        be = ops.backend
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

        c = load_golden("bf16_d64_clustered")          # B = 2: one batch element per rank
        dt = c["dtype"]
        full_shape = tuple(c["q"].shape)
        plan = be.partition.shard_plan(full_shape[0], full_shape[2], world)
        s = plan[rank]
        q, k, v, dout = (c[n][s.b0:s.b1].to(dev, dt).contiguous() for n in ("q", "k", "v", "dout"))
        coords = c["coords"][s.b0:s.b1].to(dev).contiguous()
        args = (c["W"], c["H"], c["sm_scale"])

        peer = be.partition.PeerGather([(full_shape, dt)] * 4, plan, dev)
        # 1. copy engines first: the mapping is right if a plain copy lands in the root's tensor
        marker = torch.full_like(q, float(rank + 1))
        peer.push(0, marker)
        peer.wait()
        torch.cuda.synchronize(dev)
        dist.barrier()
        if rank == 0:
            for r, sh in enumerate(plan):
                assert torch.all(peer.results[0][sh.b0:sh.b1] == float(r + 1)), f"copy of rank {r} did not land"
        dist.barrier()

        # 2. the kernels store into the root's block
        m_out, m_dq, m_dk, m_dv = peer.shard_views()
        out, lse = be.forward_raw(q, k, v, coords, *args)
        dq, dk, dv, _ = be.backward_raw(q, k, v, coords, out, lse, dout, *args,
                                        mirrors={"out": m_out, "dq": m_dq, "dk": m_dk, "dv": m_dv})
        torch.cuda.synchronize(dev)
        be.cabi.check(be.cabi.lib().dsdpa_device_error(rank))
        dist.barrier()
        # every rank sends its local results the ordinary way; the root compares bit for bit
        for i, t in enumerate((out, dq, dk, dv)):
            ref = be.partition.gather_to_root(t, plan, full_shape, root=0)
            if rank == 0:
                assert torch.equal(ref, peer.results[i]), f"result {i} differs from its mirror"
        if rank == 0:
            from conftest import TOL, rel_err
            assert rel_err(peer.results[0], c["out"]) < TOL[dt]
            assert rel_err(peer.results[2], c["dk"]) < TOL[dt]
        dist.barrier()
        peer.close()
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001  (reported to the parent, which fails the test)
        import traceback
        failures.put((rank, "".join(traceback.format_exception(exc))))
        raise


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_kernels_store_into_the_roots_mapped_block():
    if not (torch.cuda.can_device_access_peer(0, 1) and torch.cuda.can_device_access_peer(1, 0)):
        pytest.skip("the two GPUs cannot reach each other")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, failures)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            msgs.append(("parent", "a worker did not finish"))
    assert not msgs, msgs
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]

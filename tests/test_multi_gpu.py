"""One operator call spread over two GPUs (needs two visible devices; skipped otherwise).

Child processes, one per GPU, NCCL between them: the hybrid plan splits one batch entry's
queries over both ranks and sums grad_value with an all-reduce (or a reduce-scatter by key);
the batch plan gives each rank whole entries and needs no collective. Results are stitched
together on rank 0 and compared with the float64 oracle on the unsharded problem.
"""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, B, scatter, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    from drivingsdk_b200 import dist as sdist
    from drivingsdk_b200 import workloads
    from tests import parity
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        w = workloads.WORKLOADS["toy"].with_batch(B).with_queries(600)
        inp = workloads.make_inputs(w, torch.float32)
        # a long kernel and a tiny gradient: the planner splits queries whenever it may
        cost = sdist.CostModel(entry_seconds=1.0, entry_grad_bytes=1.0)
        p = sdist.plan(w.B, w.Q, world, cost=cost, scatter=scatter)
        groups = sdist.make_groups(p)
        group = groups.get(p.group_of(rank))
        value, loc, attn, go = sdist.shard_operands(p, rank, inp["value"], inp["loc"], inp["attn"],
                                                    inp["grad_out"])
        value = value.to(dev).contiguous().requires_grad_(True)
        loc = loc.to(dev).contiguous().requires_grad_(True)
        attn = attn.to(dev).contiguous().requires_grad_(True)
        shapes, starts = inp["shapes"].to(dev), inp["starts"].to(dev)
        out = sdist.multi_scale_deformable_attn_sharded(value, shapes, starts, loc, attn, p,
                                                        group=group, rank=rank)
        out.backward(go.to(dev).contiguous())
        torch.cuda.synchronize()
        pieces = [None] * world
        dist.all_gather_object(pieces, tuple(t.detach().cpu() for t in
                                             (out, value.grad, loc.grad, attn.grad)))
        if rank == 0:
            if p.kind == "batch":
                full = [torch.cat([pc[i] for pc in pieces]) for i in range(4)]
            else:
                cat_q = lambda i: torch.cat([pieces[r][i] for r in p.groups[0]], dim=1)
                gv = sum(pieces[r][1] for r in p.groups[0]) if p.scatter else pieces[0][1]
                full = [cat_q(0), gv, cat_q(2), cat_q(3)]
            errs = parity.compare_all(inp, full, torch.float32)
            out_q.put((p.kind, errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("B,scatter,kind", [(1, False, "hybrid"), (1, True, "hybrid"),
                                            (2, False, "batch")])
def test_two_gpus_match_the_oracle(B, scatter, kind):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, B, scatter, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=300)
        assert pr.exitcode == 0
    got_kind, errs = q.get(timeout=10)
    assert got_kind == kind
    assert errs["out"] < 1e-4

"""Shard planner and the N>1 path on CPU ranks (gloo); no GPU involved."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from drivingsdk_b200 import dist as sdist
from drivingsdk_b200 import workloads


def test_plan_prefers_batch_split():
    p = sdist.plan(B=6, Q=2500, world=2)
    assert p.kind == "batch" and p.ranges == ((0, 3), (3, 6)) and not p.needs_allreduce
    p = sdist.plan(B=6, Q=2500, world=4)
    assert p.kind == "batch" and [hi - lo for lo, hi in p.ranges] == [2, 2, 1, 1]
    assert abs(p.efficiency_ceiling() - 0.75) < 1e-12
    p = sdist.plan(B=8, Q=20000, world=8)
    assert p.kind == "batch" and all(hi - lo == 1 for lo, hi in p.ranges)


def test_plan_falls_back_to_query_split():
    p = sdist.plan(B=6, Q=2500, world=8)
    assert p.kind == "query" and p.needs_allreduce
    assert p.ranges[0] == (0, 313) and p.ranges[-1][1] == 2500
    assert sum(hi - lo for lo, hi in p.ranges) == 2500
    p = sdist.plan(B=1, Q=20000, world=8)
    assert p.kind == "query" and all(hi - lo == 2500 for lo, hi in p.ranges)


def test_plan_rejects_impossible_splits():
    with pytest.raises(ValueError):
        sdist.plan(B=1, Q=3, world=8)
    with pytest.raises(ValueError):
        sdist.plan(B=0, Q=3, world=1)


def test_ranges_cover_without_overlap():
    for n in (1, 5, 6, 7, 2500):
        for parts in (1, 2, 3, 4, 8):
            rs = [sdist.query_range(n, parts, r) for r in range(parts)]
            assert rs[0][0] == 0 and rs[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(rs, rs[1:]))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, B, mode, out_q):
    """One CPU rank. The compute stand-in is the PyTorch restatement of the reference's
    golden (it is differentiable and runs on CPU); the code under test is the planner, the
    operand slicing, the gradient all-reduce and the result gathering."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import golden_torch
        torch.set_num_threads(1)
        w = workloads.Workload("t", B, 24, 4, 8, ((6, 5), (3, 2)), 3, (-0.1, 1.1), 77)
        inp = workloads.make_inputs(w)
        shapes, starts = inp["shapes"], inp["starts"]
        op = lambda v, s, st, l, a: golden_torch.msda_forward(v, s, l, a)
        p = sdist.plan(w.B, w.Q, world)
        assert p.kind == mode
        value, loc, attn, go = sdist.shard_operands(p, rank, inp["value"].double(),
                                                    inp["loc"].double(), inp["attn"].double(),
                                                    inp["grad_out"].double())
        value = value.clone().requires_grad_(True)
        loc = loc.clone().requires_grad_(True)
        attn = attn.clone().requires_grad_(True)
        out = sdist.multi_scale_deformable_attn_sharded(value, shapes, starts, loc, attn, p, op=op)
        out.backward(go)
        full_out = sdist.gather_result(p, out.detach())
        full_gl = sdist.gather_result(p, loc.grad)
        full_ga = sdist.gather_result(p, attn.grad)
        full_gv = value.grad if p.kind == "query" else sdist.gather_result(p, value.grad)
        if rank == 0:
            ref = golden_torch.msda_forward_backward(inp["value"].double(), shapes,
                                                     inp["loc"].double(), inp["attn"].double(),
                                                     inp["grad_out"].double())
            errs = [float((a - b).abs().max()) for a, b in
                    zip((full_out, full_gv, full_gl, full_ga), ref)]
            out_q.put(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,mode", [(2, "batch"), (3, "batch"), (1, "query")])
def test_two_ranks_match_unsharded(B, mode):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, B, mode, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=180)
        assert pr.exitcode == 0
    errs = q.get(timeout=10)
    assert max(errs) < 1e-12, errs


def _failing_rank(rank, world, port, out_q):
    """Rank 1 never joins the collective: rank 0 must get an error from the process group's
    timeout, not hang."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        out_q.put(("rank1", "left"))
        out_q.close()
        out_q.join_thread()
        os._exit(0)   # leaves between steps, nothing in flight
    t = torch.ones(4, dtype=torch.float64).requires_grad_(True)
    y = sdist.sum_grad_across_ranks(t).sum()
    try:
        y.backward()
        out_q.put(("rank0", "no error"))
    except Exception as exc:  # gloo reports the lost peer / timeout
        out_q.put(("rank0", type(exc).__name__))
    out_q.close()
    out_q.join_thread()
    os._exit(0)


def test_missing_rank_is_an_error_not_a_hang():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_rank, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=120)
    got = dict(q.get(timeout=10) for _ in range(2))
    assert got["rank1"] == "left"
    assert got["rank0"] != "no error"

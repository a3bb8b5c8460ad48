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


# cost models in the spirit of the measured ones: BEVFormer-base fp32 on B200 (about 80 us per
# camera, 31.6 MB of grad_value per camera) and the D = 128 bf16 stress shape (about 0.9 ms
# per batch entry, 30.6 MB of grad_value)
BEV = sdist.CostModel(entry_seconds=80e-6, entry_grad_bytes=31.6e6)
STRESS = sdist.CostModel(entry_seconds=900e-6, entry_grad_bytes=30.6e6)


def test_plan_needs_a_cost_model_once_a_collective_is_in_play():
    with pytest.raises(ValueError, match="CostModel"):
        sdist.plan(B=6, Q=2500, world=8)


def test_plan_never_picks_something_slower_than_one_gpu():
    """BEVFormer-base on 8 GPUs: reducing 190 MB of fp32 grad_value costs more than the whole
    operator, so the plan keeps six ranks on whole cameras and leaves two idle."""
    p = sdist.plan(B=6, Q=2500, world=8, cost=BEV)
    assert p.kind == "batch" and not p.needs_allreduce
    assert [hi - lo for lo, hi in p.ranges] == [1, 1, 1, 1, 1, 1, 0, 0]
    assert p.is_idle(7) and not p.is_idle(0)
    assert p.predicted_seconds <= p.predicted_single_gpu_seconds
    for B in (1, 2, 3, 4, 6):
        for world in (2, 4, 8):
            for cost in (BEV, STRESS):
                q = sdist.plan(B, 2500, world, cost=cost)
                if q.predicted_seconds is not None:
                    assert q.predicted_seconds <= q.predicted_single_gpu_seconds * (1 + 1e-9)


def test_plan_takes_the_hybrid_split_when_the_reduction_is_cheap_enough():
    """Stress shape, one batch entry on 8 GPUs (the query-sharded variant of the benchmark's
    large-head-dim configuration): the kernel dominates, so the queries are split 8 ways and
    the one entry's grad_value is reduced over all ranks."""
    p = sdist.plan(B=1, Q=20000, world=8, cost=STRESS)
    assert p.kind == "hybrid" and p.needs_allreduce and p.groups == (tuple(range(8)),)
    assert all(r == (0, 1) for r in p.ranges)
    assert all(hi - lo == 2500 for lo, hi in p.query_ranges)
    # two entries on 8 GPUs: each entry's queries 4 ways, reduction inside its 4-rank group
    p = sdist.plan(B=2, Q=20000, world=8, cost=STRESS)
    assert p.kind == "hybrid" and p.groups == ((0, 1, 2, 3), (4, 5, 6, 7))
    assert p.ranges[3] == (0, 1) and p.ranges[4] == (1, 2)
    assert p.query_ranges[5] == (5000, 10000)
    # the same two entries with a BEVFormer-sized kernel: not worth a collective
    assert sdist.plan(B=2, Q=2500, world=8, cost=BEV).kind == "batch"


def test_reduce_scatter_halves_the_modelled_wire_time():
    c = sdist.CostModel(1e-3, 100e6, bus_bytes_per_s=500e9, latency_s=0.0)
    assert abs(c.reduce_seconds(100e6, 8) - 2 * 7 / 8 * 100e6 / 500e9) < 1e-12
    assert abs(c.reduce_seconds(100e6, 8, scatter=True) - 7 / 8 * 100e6 / 500e9) < 1e-12
    assert c.reduce_seconds(100e6, 1) == 0.0
    lo, hi = sdist.key_block(30825, 4, 3)
    assert (lo, hi) == (3 * 7707, 30825)


def test_estimate_cost_uses_the_roofline_byte_counts():
    c = sdist.estimate_cost(K=30825, H=8, D=32, L=4, Q=2500, P=8, elem_size=4,
                            achieved_bytes_per_s=1e12)
    assert abs(c.entry_seconds - 737126400 / 6 / 1e12) < 1e-12
    assert c.entry_grad_bytes == 4 * 30825 * 8 * 32


def test_plan_rejects_impossible_splits():
    with pytest.raises(ValueError):
        sdist.plan(B=0, Q=3, world=1)
    # too few queries to split: the batch plan (with idle ranks) is all that is left
    assert sdist.plan(B=1, Q=3, world=8, cost=STRESS).kind == "batch"


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


def _gather_hybrid(p, rank, w, out, gv, gl, ga):
    """Stitches a hybrid plan's results together on every rank (test tooling): all ranks
    exchange their pieces; grad_value of an entry is taken from its group (after an
    all-reduce every member holds it; after a reduce-scatter each member holds its block of
    keys and zeros elsewhere, so the members' tensors are added)."""
    pieces = [None] * p.world
    dist.all_gather_object(pieces, (out, gv, gl, ga))
    B = w.B
    full_out = torch.cat([torch.cat([pieces[r][0] for r in p.groups[b]], dim=1) for b in range(B)])
    full_gl = torch.cat([torch.cat([pieces[r][2] for r in p.groups[b]], dim=1) for b in range(B)])
    full_ga = torch.cat([torch.cat([pieces[r][3] for r in p.groups[b]], dim=1) for b in range(B)])
    if p.scatter:
        full_gv = torch.cat([sum(pieces[r][1] for r in p.groups[b]) for b in range(B)])
    else:
        full_gv = torch.cat([pieces[p.groups[b][0]][1] for b in range(B)])
    return full_out, full_gv, full_gl, full_ga


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
        scatter = mode.endswith("+scatter")
        kind = mode.split("+")[0].rstrip("!")
        # a long kernel and a tiny gradient: splitting queries always pays in this model;
        # "!": a short kernel and a huge gradient, so that leaving ranks idle beats any
        # collective
        cost = sdist.CostModel(entry_seconds=1.0, entry_grad_bytes=1.0)
        if mode.endswith("!"):
            cost = sdist.CostModel(entry_seconds=1e-6, entry_grad_bytes=1e12)
        p = sdist.plan(w.B, w.Q, world, cost=cost, scatter=scatter)
        assert p.kind == kind, (p.kind, kind)
        groups = sdist.make_groups(p)
        group = groups.get(p.group_of(rank))
        value, loc, attn, go = sdist.shard_operands(p, rank, inp["value"].double(),
                                                    inp["loc"].double(), inp["attn"].double(),
                                                    inp["grad_out"].double())
        value = value.clone().requires_grad_(True)
        loc = loc.clone().requires_grad_(True)
        attn = attn.clone().requires_grad_(True)
        out = sdist.multi_scale_deformable_attn_sharded(value, shapes, starts, loc, attn, p,
                                                        group=group, op=op, rank=rank)
        out.backward(go)
        if p.kind == "hybrid":
            full_out, full_gv, full_gl, full_ga = _gather_hybrid(p, rank, w, out.detach(),
                                                                 value.grad, loc.grad, attn.grad)
        else:
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


@pytest.mark.parametrize("world,B,mode", [(2, 2, "batch"), (2, 3, "batch"), (2, 1, "hybrid"),
                                          (2, 1, "hybrid+scatter"), (4, 2, "hybrid"),
                                          (4, 2, "hybrid+scatter"), (4, 3, "batch!")])
def test_ranks_match_unsharded(world, B, mode):
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

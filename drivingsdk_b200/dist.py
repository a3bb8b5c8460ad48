"""Multi-GPU sharding of multi-scale deformable attention: one process per GPU.

The operator is independent across the batch dimension (value row offsets are
``b*K*H*D``-based in forward and backward, kernels/multi_scale_deformable_attn/op_kernel/
msda.h:358-359, 414-426), so the natural split is by batch and needs no collective: each
rank holds its slice of every operand and produces its slice of every result. A batch entry
can also be split by queries: every rank of the entry's group holds that entry's whole
``value`` and a contiguous slice of its queries; ``output``, ``grad_sampling_loc`` and
``grad_attn_weight`` are sliced the same way and need nothing, but ``grad_value`` is a
partial sum on every rank of the group and is summed over the group (NCCL on GPUs) — the
only collective on this path — either everywhere (all-reduce) or to one owner per block of
keys (reduce-scatter, half the bytes on the wire, for consumers that can take grad_value
sharded by key).

Three kinds of plan:
  batch   min(B, world) ranks take whole batch entries; with B < world the other ranks idle
  hybrid  world is a multiple of B: world/B ranks share each entry's queries and reduce that
          entry's grad_value among themselves (B == 1 is the pure query split)
  query   every rank takes a slice of every entry's queries and all of grad_value is
          reduced over all ranks
``plan`` picks the fastest by a cost model (kernel time scales with the work a rank holds;
a reduction over g ranks moves 2*(g-1)/g of the bytes — (g-1)/g for reduce-scatter — at the
measured bus bandwidth plus a latency), and never returns a plan it predicts to be slower
than one GPU doing everything. The reference library has no collective of its own (its
models use data parallelism around the operator, model_examples/BEVFormer/README.md:208-215);
this module is what that usage looks like when one operator call is spread over the GPUs of
a node.
"""
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def _even_ranges(n: int, parts: int) -> List[Tuple[int, int]]:
    """``parts`` contiguous ranges covering [0, n), sizes differing by at most one (larger
    ones first); ranges are empty when parts > n."""
    base, extra = divmod(n, parts)
    out, lo = [], 0
    for r in range(parts):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def batch_range(B: int, world: int, rank: int) -> Tuple[int, int]:
    return _even_ranges(B, world)[rank]


def query_range(Q: int, world: int, rank: int) -> Tuple[int, int]:
    return _even_ranges(Q, world)[rank]


@dataclass(frozen=True)
class CostModel:
    """What ``plan`` needs to compare plans: seconds one GPU takes for forward + backward of
    ONE batch entry, bytes of one entry's grad_value, how much of the entry's time does not
    shrink when its queries are split (zero-fill and 16-bit conversion of grad_value, launch
    gaps), and the collective's cost: bus bandwidth (bytes/s) plus a latency per ring step
    (2(n-1) steps for an all-reduce over n ranks, n-1 for a reduce-scatter). The defaults are
    NCCL all-reduces of 30.6 MB measured on 2, 4 and 8 B200s over NVLink (88 / 129 / 166 us);
    messages of ~190 MB reach 550-600 GB/s."""
    entry_seconds: float
    entry_grad_bytes: float
    bus_bytes_per_s: float = 420e9
    latency_s: float = 3e-6
    fixed_seconds: float = 0.0

    def reduce_seconds(self, nbytes: float, ranks: int, scatter: bool = False) -> float:
        if ranks <= 1:
            return 0.0
        passes = 1.0 if scatter else 2.0
        return (passes * (ranks - 1) * self.latency_s +
                passes * (ranks - 1) / ranks * nbytes / self.bus_bytes_per_s)

    def split_seconds(self, share: float) -> float:
        """One entry's time on a rank that works `share` of its queries."""
        fixed = min(self.fixed_seconds, self.entry_seconds)
        return fixed + share * (self.entry_seconds - fixed)


def fixed_entry_seconds(K: int, H: int, D: int, elem_size: int, hbm_bytes_per_s: float = 6.4e12,
                        launch_gaps_s: float = 15e-6) -> float:
    """The part of one entry's forward + backward that a split of its queries does not
    shrink: the zero-fill of grad_value (for 16-bit tensors of its fp32 accumulation copy,
    plus the conversion pass: 4 + 4 + 2 bytes per element) at HBM speed, and the gaps between
    the call's launches."""
    per_elem = 4 if elem_size == 4 else 10
    return per_elem * K * H * D / hbm_bytes_per_s + launch_gaps_s


def estimate_cost(K: int, H: int, D: int, L: int, Q: int, P: int, elem_size: int,
                  achieved_bytes_per_s: float = 1.8e12, **kw) -> CostModel:
    """Cost model from the operand sizes alone: one entry's forward + backward algorithmic
    bytes (every operand once, every result once) over the bandwidth the kernels reach on
    one GPU (default: what they measure at the BEVFormer shape)."""
    v, s, o = K * H * D, Q * H * L * P, Q * H * D
    step_bytes = elem_size * (3 * v + 9 * s + 2 * o)
    kw.setdefault("fixed_seconds", fixed_entry_seconds(K, H, D, elem_size))
    return CostModel(step_bytes / achieved_bytes_per_s, float(elem_size * v), **kw)


@dataclass(frozen=True)
class ShardPlan:
    kind: str                                   # "batch", "hybrid" or "query"
    world: int
    ranges: Tuple[Tuple[int, int], ...]         # per rank [lo, hi): batch entries ("batch",
                                                # "hybrid") or queries ("query")
    query_ranges: Tuple[Tuple[int, int], ...] = ()   # "hybrid": per rank [lo, hi) of queries
    groups: Tuple[Tuple[int, ...], ...] = ()    # sets of ranks that sum grad_value together
    scatter: bool = False                       # reduce-scatter (by key) instead of all-reduce
    predicted_seconds: Optional[float] = None
    predicted_single_gpu_seconds: Optional[float] = None

    @property
    def needs_allreduce(self) -> bool:
        return any(len(g) > 1 for g in self.groups)

    def group_of(self, rank: int) -> Tuple[int, ...]:
        for g in self.groups:
            if rank in g:
                return g
        return (rank,)

    def is_idle(self, rank: int) -> bool:
        lo, hi = self.ranges[rank]
        return hi <= lo

    def efficiency_ceiling(self) -> float:
        """Best possible parallel efficiency of this split: mean share / largest share."""
        if self.kind == "hybrid":
            sizes = [(hi - lo) * (qh - ql) for (lo, hi), (ql, qh) in
                     zip(self.ranges, self.query_ranges)]
        else:
            sizes = [hi - lo for lo, hi in self.ranges]
        return (sum(sizes) / len(sizes)) / max(sizes) if max(sizes) > 0 else 0.0


def _batch_plan(B: int, world: int) -> ShardPlan:
    return ShardPlan("batch", world, tuple(_even_ranges(B, world)),
                     groups=tuple((r,) for r in range(world)))


def _hybrid_plan(B: int, Q: int, world: int, scatter: bool) -> ShardPlan:
    g = world // B
    ranges, qranges, groups = [], [], []
    for b in range(B):
        groups.append(tuple(range(b * g, (b + 1) * g)))
        for lo, hi in _even_ranges(Q, g):
            ranges.append((b, b + 1))
            qranges.append((lo, hi))
    return ShardPlan("hybrid", world, tuple(ranges), tuple(qranges), tuple(groups), scatter)


def _query_plan(Q: int, world: int, scatter: bool) -> ShardPlan:
    return ShardPlan("query", world, tuple(_even_ranges(Q, world)),
                     groups=(tuple(range(world)),), scatter=scatter)


def predict_seconds(p: ShardPlan, B: int, Q: int, cost: CostModel) -> float:
    """Predicted time of one forward + backward under plan ``p`` (slowest rank)."""
    if p.kind == "batch":
        return max(hi - lo for lo, hi in p.ranges) * cost.entry_seconds
    if p.kind == "hybrid":
        g = len(p.groups[0])
        share = max(qh - ql for ql, qh in p.query_ranges) / Q
        return cost.split_seconds(share) + cost.reduce_seconds(cost.entry_grad_bytes, g,
                                                               p.scatter)
    share = max(hi - lo for lo, hi in p.ranges) / Q
    return B * cost.split_seconds(share) + cost.reduce_seconds(B * cost.entry_grad_bytes,
                                                               p.world, p.scatter)


def candidate_plans(B: int, Q: int, world: int, scatter: bool = False) -> List[ShardPlan]:
    out = [_batch_plan(B, world)]
    if world > B and world % B == 0 and Q >= world // B:
        out.append(_hybrid_plan(B, Q, world, scatter))
    if world > 1 and Q >= world and not (B == 1):      # B == 1: hybrid is the query split
        out.append(_query_plan(Q, world, scatter))
    return out


def plan(B: int, Q: int, world: int, cost: Optional[CostModel] = None,
         scatter: bool = False) -> ShardPlan:
    """The fastest of the candidate plans under ``cost``. Without a cost model: batch split
    whenever B >= world (no collective, nothing to weigh); otherwise the collective's cost
    decides and a model is required — ``estimate_cost`` builds one from the operand sizes."""
    if world < 1 or B < 1 or Q < 1:
        raise ValueError("plan(): B, Q and world must be positive")
    if B >= world:
        return _batch_plan(B, world)
    cands = candidate_plans(B, Q, world, scatter)
    if cost is None:
        raise ValueError(
            f"B={B} < world={world}: a split of the queries needs a collective; pass a "
            "CostModel (see estimate_cost) so that the plan can weigh it")
    single = B * cost.entry_seconds
    best, best_t = None, None
    for c in cands:
        t = predict_seconds(c, B, Q, cost)
        if best_t is None or t < best_t:
            best, best_t = c, t
    return ShardPlan(best.kind, best.world, best.ranges, best.query_ranges, best.groups,
                     best.scatter, best_t, single)


# ---------------------------------------------------------------------------
# running a plan
# ---------------------------------------------------------------------------
def shard_operands(p: ShardPlan, rank: int, value, loc, attn, grad_out=None):
    """This rank's views of the operands (no copies beyond what slicing needs)."""
    lo, hi = p.ranges[rank]
    if p.kind == "batch":
        parts = (value[lo:hi], loc[lo:hi], attn[lo:hi])
        return parts + ((grad_out[lo:hi],) if grad_out is not None else ())
    if p.kind == "hybrid":
        ql, qh = p.query_ranges[rank]
        parts = (value[lo:hi], loc[lo:hi, ql:qh], attn[lo:hi, ql:qh])
        return parts + ((grad_out[lo:hi, ql:qh],) if grad_out is not None else ())
    parts = (value, loc[:, lo:hi], attn[:, lo:hi])
    return parts + ((grad_out[:, lo:hi],) if grad_out is not None else ())


def make_groups(p: ShardPlan) -> Dict[Tuple[int, ...], object]:
    """Process groups for the plan's reduction groups. Collective: every rank of the default
    group must call it, once, with the same plan (torch.distributed.new_group's rule)."""
    out: Dict[Tuple[int, ...], object] = {}
    for g in p.groups:
        if len(g) > 1 and len(g) < p.world:
            out[g] = dist.new_group(list(g))
        elif len(g) > 1:
            out[g] = None   # the default group
    return out


class _SumGradAcrossRanks(torch.autograd.Function):
    """Identity in forward; in backward the incoming gradient (this rank's partial
    grad_value) is summed over the process group, in place."""

    @staticmethod
    def forward(ctx, tensor, group):
        ctx.group = group
        return tensor.view_as(tensor)

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=ctx.group)
        return grad, None


class _ScatterGradAcrossRanks(torch.autograd.Function):
    """Identity in forward; in backward the partial grad_value [b, K, H, D] is reduce-
    scattered over the group along K: this rank's block of keys receives the sum, the rest of
    the returned gradient is zero (the consumer reads only its own block, see
    ``key_block``)."""

    @staticmethod
    def forward(ctx, tensor, group, rank_in_group, group_size):
        ctx.group, ctx.r, ctx.g = group, rank_in_group, group_size
        return tensor.view_as(tensor)

    @staticmethod
    def backward(ctx, grad):
        g, r = ctx.g, ctx.r
        K = grad.shape[1]
        block = (K + g - 1) // g
        padded = grad.new_zeros((grad.shape[0], block * g) + tuple(grad.shape[2:]))
        padded[:, :K].copy_(grad)
        # [b, g, block, ...] -> [g, b, block, ...] so that rank i's block is contiguous
        send = padded.view(grad.shape[0], g, block, *grad.shape[2:]).transpose(0, 1).contiguous()
        recv = torch.empty_like(send[0])
        send = send.view(g * grad.shape[0], block, *grad.shape[2:])   # rank blocks along dim 0
        dist.reduce_scatter_tensor(recv, send, op=dist.ReduceOp.SUM, group=ctx.group)
        out = torch.zeros_like(grad)
        lo, hi = r * block, min(K, (r + 1) * block)
        if hi > lo:
            out[:, lo:hi].copy_(recv[:, :hi - lo])
        return out, None, None, None


def key_block(K: int, group_size: int, rank_in_group: int) -> Tuple[int, int]:
    """Keys [lo, hi) whose grad_value a rank owns after a reduce-scatter plan's backward."""
    block = (K + group_size - 1) // group_size
    return min(K, rank_in_group * block), min(K, (rank_in_group + 1) * block)


def sum_grad_across_ranks(tensor: torch.Tensor, group=None) -> torch.Tensor:
    return _SumGradAcrossRanks.apply(tensor, group)


def multi_scale_deformable_attn_sharded(value, value_spatial_shapes, value_level_start_index,
                                        sampling_locations, attention_weights, shard: ShardPlan,
                                        group=None, op: Optional[Callable] = None,
                                        rank: Optional[int] = None):
    """Runs this rank's share of one operator call. The operands passed in are already this
    rank's shares (see ``shard_operands``). Where the plan splits queries, ``value`` is the
    whole entry (or tensor) on every rank of the group and its gradient is summed over
    ``group`` during backward (``make_groups`` gives the group of a hybrid plan; None is the
    default group); with a batch split this is exactly the plain operator. ``op`` defaults
    to the CUDA operator of this package. ``rank`` (default: this process's rank) is needed
    only by reduce-scatter plans."""
    if op is None:
        from drivingsdk_b200 import multi_scale_deformable_attn as op
    if shard.needs_allreduce:
        if shard.scatter:
            me = dist.get_rank() if rank is None else rank
            members = shard.group_of(me)
            value = _ScatterGradAcrossRanks.apply(value, group, members.index(me), len(members))
        else:
            value = sum_grad_across_ranks(value, group)
    return op(value, value_spatial_shapes, value_level_start_index, sampling_locations,
              attention_weights)


def gather_result(p: ShardPlan, local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers a sliced result (output, grad_sampling_loc, grad_attn_weight — or
    grad_value of a batch split) of a batch or query plan back into the full tensor, for
    checks and tooling; the operator itself never needs it."""
    if p.kind == "hybrid":
        raise ValueError("gather_result handles batch and query plans; gather a hybrid plan's "
                         "results per entry group")
    dim = 0 if p.kind == "batch" else 1
    sizes = [hi - lo for lo, hi in p.ranges]
    biggest = max(sizes)
    pad_shape = list(local.shape)
    pad_shape[dim] = biggest
    padded = local.new_zeros(pad_shape)
    padded.narrow(dim, 0, local.shape[dim]).copy_(local)
    bucket = [torch.empty_like(padded) for _ in range(p.world)]
    dist.all_gather(bucket, padded, group=group)
    return torch.cat([b.narrow(dim, 0, n) for b, n in zip(bucket, sizes)], dim=dim)

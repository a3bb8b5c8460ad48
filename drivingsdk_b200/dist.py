"""Multi-GPU sharding of multi-scale deformable attention: one process per GPU.

The operator is independent across the batch dimension (value row offsets are
``b*K*H*D``-based in forward and backward), so the natural split is by batch and needs
no collective: each rank holds its slice of every operand and produces its slice of
every result. When there are fewer batch entries than ranks the queries are split
instead: every rank holds the whole ``value`` and a contiguous slice of the queries;
``output``, ``grad_sampling_loc`` and ``grad_attn_weight`` are sliced the same way and
need nothing, but ``grad_value`` is a partial sum on every rank and is all-reduced
(NCCL on GPUs) — the only collective on this path. The reference library has no
collective of its own (its models use data parallelism around the operator,
model_examples/BEVFormer/README.md:208-215); this module is what that usage looks like
when one operator call is spread over the GPUs of a node.
"""
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

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
class ShardPlan:
    kind: str                       # "batch" or "query"
    world: int
    ranges: Tuple[Tuple[int, int], ...]   # per rank, [lo, hi) along the sharded dimension

    @property
    def needs_allreduce(self) -> bool:
        return self.kind == "query" and self.world > 1

    def efficiency_ceiling(self) -> float:
        """Best possible parallel efficiency of this split: mean share / largest share."""
        sizes = [hi - lo for lo, hi in self.ranges]
        return (sum(sizes) / len(sizes)) / max(sizes) if max(sizes) > 0 else 0.0


def plan(B: int, Q: int, world: int) -> ShardPlan:
    """Batch split when every rank gets at least one batch entry, else query split."""
    if world < 1 or B < 1 or Q < 1:
        raise ValueError("plan(): B, Q and world must be positive")
    if B >= world:
        return ShardPlan("batch", world, tuple(_even_ranges(B, world)))
    if Q < world:
        raise ValueError(f"cannot shard B={B}, Q={Q} over {world} ranks")
    return ShardPlan("query", world, tuple(_even_ranges(Q, world)))


def shard_operands(p: ShardPlan, rank: int, value, loc, attn, grad_out=None):
    """This rank's views of the operands (no copies beyond what slicing needs)."""
    lo, hi = p.ranges[rank]
    if p.kind == "batch":
        parts = (value[lo:hi], loc[lo:hi], attn[lo:hi])
        return parts + ((grad_out[lo:hi],) if grad_out is not None else ())
    parts = (value, loc[:, lo:hi], attn[:, lo:hi])
    return parts + ((grad_out[:, lo:hi],) if grad_out is not None else ())


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


def sum_grad_across_ranks(tensor: torch.Tensor, group=None) -> torch.Tensor:
    return _SumGradAcrossRanks.apply(tensor, group)


def multi_scale_deformable_attn_sharded(value, value_spatial_shapes, value_level_start_index,
                                        sampling_locations, attention_weights, shard: ShardPlan,
                                        group=None, op: Optional[Callable] = None):
    """Runs this rank's share of one operator call. The operands passed in are already this
    rank's shares (see ``shard_operands``). With a query split ``value`` is the whole tensor
    on every rank and its gradient is all-reduced during backward; with a batch split this
    is exactly the plain operator. ``op`` defaults to the CUDA operator of this package."""
    if op is None:
        from drivingsdk_b200 import multi_scale_deformable_attn as op
    if shard.needs_allreduce:
        value = sum_grad_across_ranks(value, group)
    return op(value, value_spatial_shapes, value_level_start_index, sampling_locations,
              attention_weights)


def gather_result(p: ShardPlan, local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers a sliced result (output, grad_sampling_loc, grad_attn_weight — or
    grad_value of a batch split) back into the full tensor, for checks and tooling; the
    operator itself never needs it."""
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

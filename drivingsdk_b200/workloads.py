"""Seeded synthetic MSDA workloads with the tensor shapes of the benchmark configs.

No dataset is read: each workload takes the operand shapes and value
distributions of a model's deformable-attention call and draws them from a
seeded generator (value ~ N(0,1); locations uniform in a stated range;
attention weights = softmax of N(0,1) logits over levels*points; grad_output ~
N(0,1)). All tensors are created on the CPU in float32, rounded to the
requested dtype, and returned in float32 containers together with that dtype,
so that a float64 checker and the device run see exactly the same values.
"""
from dataclasses import dataclass
from typing import List, Tuple

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    Q: int
    H: int
    D: int
    levels: Tuple[Tuple[int, int], ...]   # (height, width) per level
    P: int
    loc_range: Tuple[float, float]
    seed: int

    @property
    def L(self) -> int:
        return len(self.levels)

    @property
    def K(self) -> int:
        return sum(h * w for h, w in self.levels)

    def with_batch(self, B: int) -> "Workload":
        return Workload(self.name, B, self.Q, self.H, self.D, self.levels, self.P,
                        self.loc_range, self.seed)

    def with_queries(self, Q: int) -> "Workload":
        return Workload(self.name, self.B, Q, self.H, self.D, self.levels, self.P,
                        self.loc_range, self.seed)


WORKLOADS = {
    # CPU-golden-runnable toy
    "toy": Workload("toy", 1, 1000, 8, 32, ((32, 32), (16, 16), (8, 8), (4, 4)), 4, (-0.1, 1.1), 1234),
    # Deformable-DETR encoder self-attention
    "deformable_detr": Workload("deformable_detr", 2, 17821, 8, 32,
                                ((100, 134), (50, 67), (25, 34), (13, 17)), 4, (0.0, 1.0), 1235),
    # BEVFormer-base spatial cross-attention: 6 cameras, 2500 queries per camera
    "bevformer_sca": Workload("bevformer_sca", 6, 2500, 8, 32,
                              ((116, 200), (58, 100), (29, 50), (15, 25)), 8, (-0.05, 1.05), 1236),
    # BEVFormer temporal self-attention: previous and current BEV stacked
    "bevformer_tsa": Workload("bevformer_tsa", 2, 40000, 8, 32, ((200, 200),), 4, (0.0, 1.0), 1237),
    # large head_dim stress; level sizes sum to 14960 keys
    "stress_d128": Workload("stress_d128", 8, 20000, 8, 128,
                            ((64, 176), (32, 88), (16, 44), (8, 22)), 4, (-0.1, 1.1), 1238),
}


def level_tensors(levels) -> Tuple[torch.Tensor, torch.Tensor]:
    """(spatial_shapes [L,2] int64, level_start_index [L] int64)."""
    shapes = torch.tensor(list(levels), dtype=torch.int64).reshape(-1, 2)
    sizes = shapes[:, 0] * shapes[:, 1]
    starts = torch.cat([sizes.new_zeros(1), sizes.cumsum(0)[:-1]])
    return shapes, starts


def make_inputs(w: Workload, dtype: torch.dtype = torch.float32, seed_offset: int = 0):
    """Returns dict(shapes, starts, value, loc, attn, grad_out): float32 CPU tensors holding
    values representable in ``dtype``."""
    g = torch.Generator().manual_seed(w.seed + seed_offset)
    shapes, starts = level_tensors(w.levels)
    lo, hi = w.loc_range
    value = torch.randn(w.B, w.K, w.H, w.D, generator=g)
    loc = torch.rand(w.B, w.Q, w.H, w.L, w.P, 2, generator=g) * (hi - lo) + lo
    logits = torch.randn(w.B, w.Q, w.H, w.L * w.P, generator=g)
    attn = torch.softmax(logits, -1).reshape(w.B, w.Q, w.H, w.L, w.P)
    grad_out = torch.randn(w.B, w.Q, w.H * w.D, generator=g)
    rnd = lambda t: t.to(dtype).float()
    return {"shapes": shapes, "starts": starts, "value": rnd(value), "loc": rnd(loc),
            "attn": rnd(attn), "grad_out": rnd(grad_out)}


def compulsory_bytes(w: Workload, elem_size: int) -> Tuple[int, int]:
    """(forward, backward) algorithmic bytes: every operand read once, every result
    written once.
        forward  = e * (B*K*H*D + 3*B*Q*H*L*P + B*Q*H*D)
        backward = e * (2*B*K*H*D + 6*B*Q*H*L*P + B*Q*H*D)
    """
    v = w.B * w.K * w.H * w.D
    s = w.B * w.Q * w.H * w.L * w.P
    o = w.B * w.Q * w.H * w.D
    return elem_size * (v + 3 * s + o), elem_size * (2 * v + 6 * s + o)

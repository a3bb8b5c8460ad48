"""Parity of the fused operator (reference points + offsets + logits in) — needs a GPU.

Checker: the float64 composition of what the fused kernels absorb (location arithmetic and
softmax as mmcv's MultiScaleDeformableAttention.forward writes them) with the PyTorch
restatement of the reference's MSDA golden, differentiated by autograd."""
import numpy as np
import pytest
import torch

from drivingsdk_b200 import workloads
from drivingsdk_b200.ops.msda_fused import compose_unfused
from oracle import golden_torch
from tests import parity

pytestmark = pytest.mark.gpu


def _inputs(w, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    shapes, starts = workloads.level_tensors(w.levels)
    rnd = lambda t: t.to(dtype).float()
    return {
        "shapes": shapes, "starts": starts,
        "value": rnd(torch.randn(w.B, w.K, w.H, w.D, generator=g)),
        "ref": rnd(torch.rand(w.B, w.Q, w.L, 2, generator=g) * 1.1 - 0.05),
        "off": rnd(torch.randn(w.B, w.Q, w.H, w.L, w.P, 2, generator=g) * 2.0),
        "logits": rnd(torch.randn(w.B, w.Q, w.H, w.L, w.P, generator=g)),
        "grad_out": rnd(torch.randn(w.B, w.Q, w.H * w.D, generator=g)),
    }


def _golden(inp):
    d = {k: inp[k].double() for k in ("value", "ref", "off", "logits", "grad_out")}
    for k in ("value", "ref", "off", "logits"):
        d[k].requires_grad_()
    loc, attn = compose_unfused(d["ref"], d["off"], d["logits"], inp["shapes"])
    out = golden_torch.msda_forward(d["value"], inp["shapes"], loc, attn)
    out.backward(d["grad_out"])
    return (out.detach().numpy(), d["value"].grad.numpy(), d["ref"].grad.numpy(),
            d["off"].grad.numpy(), d["logits"].grad.numpy(), loc.detach().numpy())


def _run(inp, dtype):
    import drivingsdk_b200 as sdk
    dev = {k: inp[k].to("cuda", dtype).requires_grad_() for k in ("value", "ref", "off", "logits")}
    out = sdk.multi_scale_deformable_attn_fused(dev["value"], inp["shapes"].cuda(),
                                                inp["starts"].cuda(), dev["ref"], dev["off"],
                                                dev["logits"])
    out.backward(inp["grad_out"].to("cuda", dtype))
    return out.detach(), dev["value"].grad, dev["ref"].grad, dev["off"].grad, dev["logits"].grad


CASES = [
    ("toy_l4p4", workloads.Workload("f", 1, 300, 8, 32, ((32, 32), (16, 16), (8, 8), (4, 4)), 4, (0, 1), 1)),
    ("bev_l4p8", workloads.Workload("f", 2, 200, 8, 32, ((29, 50), (15, 25), (8, 13), (4, 7)), 8, (0, 1), 2)),
    ("tsa_l1p4", workloads.Workload("f", 2, 333, 8, 32, ((40, 40),), 4, (0, 1), 3)),
    ("odd_l3p5_d37", workloads.Workload("f", 1, 77, 3, 37, ((9, 7), (5, 4), (2, 3)), 5, (0, 1), 4)),
    ("l1p1_d128", workloads.Workload("f", 1, 129, 2, 128, ((6, 6),), 1, (0, 1), 5)),
]


@pytest.mark.parametrize("name,w", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_matches_float64_composition(name, w, dtype):
    inp = _inputs(w, dtype, seed=w.seed)
    want = _golden(inp)
    got = _run(inp, dtype)
    tol = parity.TOL[dtype]
    rnd = (lambda a: a) if dtype == torch.float32 else (
        lambda a: torch.from_numpy(a).to(dtype).double().numpy())
    parity.assert_close("output", got[0], rnd(want[0]), tol)
    parity.assert_close("grad_value", got[1], rnd(want[1]), tol)
    parity.assert_close("grad_logits", got[4], rnd(want[4]), tol)
    if dtype == torch.float32:
        # location gradients: skip samples that sit on a pixel boundary (one-sided derivative)
        from oracle import msda_oracle
        smooth = msda_oracle.kink_distance(inp["shapes"].numpy(), want[5].astype(np.float32)) > 1e-3
        # the mask may only ever hide a small share of the samples
        assert (~smooth).sum() <= max(4, 1e-2 * smooth.size), ((~smooth).sum(), smooth.size)
        parity.assert_close("grad_offsets", got[3], want[3], tol,
                            mask=np.broadcast_to(smooth[..., None], want[3].shape))
        # a reference point collects all heads and points of its level (a sum of H * P location
        # gradients that largely cancel, each carrying the float32 rounding of its location):
        # wider absolute tolerance, and only points whose samples are all away from boundaries
        ok = smooth.all(axis=(2, 4))                       # [B, Q, L]
        parity.assert_close("grad_reference_points", got[2], want[2], tol * 20,
                            mask=np.broadcast_to(ok[..., None], want[2].shape))
    else:
        # 16-bit: offsets / size is no longer exact, samples may change cells; check the bulk
        err = np.abs(got[3].double().cpu().numpy() - rnd(want[3]))
        assert np.mean(err > tol + tol * np.abs(rnd(want[3]))) < 0.02


def test_fused_equals_unfused_cuda_path_at_bevformer_size():
    import drivingsdk_b200 as sdk
    w = workloads.WORKLOADS["bevformer_sca"].with_batch(2)
    inp = _inputs(w, torch.float32, seed=9)
    got = _run(inp, torch.float32)
    dev = {k: inp[k].cuda().requires_grad_() for k in ("value", "ref", "off", "logits")}
    loc, attn = compose_unfused(dev["ref"], dev["off"], dev["logits"], inp["shapes"].cuda())
    out = sdk.multi_scale_deformable_attn(dev["value"], inp["shapes"].cuda(), inp["starts"].cuda(),
                                          loc, attn)
    out.backward(inp["grad_out"].cuda())
    torch.testing.assert_close(got[0], out.detach(), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(got[1], dev["value"].grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(got[4], dev["logits"].grad, rtol=1e-4, atol=1e-4)
    # the two paths round the location differently (fused: one rounding of ref + off / W);
    # a sample within that rounding of a pixel boundary may fall into the neighbouring cell
    bad = ((got[3] - dev["off"].grad).abs() > 1e-4 + 1e-4 * dev["off"].grad.abs()).float().mean()
    assert bad.item() < 1e-3


def test_fused_rejects_more_than_32_samples():
    import drivingsdk_b200 as sdk
    w = workloads.Workload("f", 1, 4, 2, 8, ((4, 4),) * 5, 7, (0, 1), 1)
    inp = _inputs(w, torch.float32, seed=1)
    with pytest.raises(RuntimeError, match="<= 32"):
        _run(inp, torch.float32)

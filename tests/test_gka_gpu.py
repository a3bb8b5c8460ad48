"""Parity of the geometric-kernel-attention CUDA path (needs a GPU)."""
import os
import zlib

import numpy as np
import pytest
import torch

from drivingsdk_b200 import workloads
from oracle import msda_oracle
from tests import parity
from tests.test_gka_oracle import NAMES, case

pytestmark = pytest.mark.gpu


def _run_python_api(inp, dtype, loc_dtype=None):
    import drivingsdk_b200 as sdk
    value = torch.from_numpy(inp["value"]).to("cuda", dtype).requires_grad_(True)
    attn = torch.from_numpy(inp["attn"]).to("cuda", dtype).requires_grad_(True)
    loc = torch.from_numpy(inp["loc"]).to("cuda")
    loc = loc.to(loc_dtype) if loc_dtype is not None else loc.to(dtype)
    shapes = torch.from_numpy(inp["shapes"]).to("cuda")
    starts = torch.from_numpy(inp["starts"]).to("cuda")
    out = sdk.geometric_kernel_attention(value, shapes, starts, loc, attn)
    out.backward(torch.from_numpy(inp["grad_out"]).to("cuda", dtype))
    return out.detach(), value.grad, attn.grad


def _run_c_abi(inp, dtype):
    from drivingsdk_b200 import capi
    lib = capi.load()
    dev = {k: torch.from_numpy(inp[k]).to("cuda", dtype) for k in ("value", "loc", "attn", "grad_out")}
    shapes = torch.from_numpy(inp["shapes"]).to("cuda", torch.int32)
    starts = torch.from_numpy(inp["starts"]).to("cuda", torch.int32)
    B, K, H, D = dev["value"].shape
    _, Q, _, L, P, _ = dev["loc"].shape
    out = torch.empty(B, Q, H * D, device="cuda", dtype=dtype)
    gv, ga = torch.empty_like(dev["value"]), torch.empty_like(dev["attn"])
    code = capi.dtype_code(dtype)
    stream = torch.cuda.current_stream().cuda_stream
    capi.check(lib.gka_sm100_forward(dev["value"].data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                     dev["loc"].data_ptr(), dev["attn"].data_ptr(), out.data_ptr(),
                                     B, K, H, D, L, Q, P, code, stream), "gka forward")
    nbytes = lib.msda_sm100_backward_workspace_bytes(B, K, H, D, code)
    ws = torch.empty(max(nbytes, 16), device="cuda", dtype=torch.uint8)
    capi.check(lib.gka_sm100_backward_ws(
        dev["value"].data_ptr(), shapes.data_ptr(), starts.data_ptr(), dev["loc"].data_ptr(),
        dev["attn"].data_ptr(), dev["grad_out"].data_ptr(), gv.data_ptr(), ga.data_ptr(),
        ws.data_ptr(), nbytes, B, K, H, D, L, Q, P, code, stream), "gka backward")
    torch.cuda.synchronize()
    return out, gv, ga


def _check(results, want, dtype):
    tol = parity.TOL[dtype]
    if dtype != torch.float32:
        want = [torch.from_numpy(w).to(dtype).double().numpy() for w in want]
    # the reference draws value in [0, 3) and grad_output in [0, 10): results reach the
    # hundreds, where the relative term of the tolerance carries the comparison
    for name, got, w in zip(("output", "grad_value", "grad_attn"), results, want):
        parity.assert_close(name, got, w, tol)


@pytest.mark.parametrize("name", NAMES)
def test_golden_fixture_c_abi_and_python_api(name):
    c = case(name)
    want = (c["out"], c["grad_value"], c["grad_attn"])
    _check(_run_c_abi(c, torch.float32), want, torch.float32)
    _check(_run_python_api(c, torch.float32), want, torch.float32)
    # integer location tensors, as mmcv-style callers may pass them
    _check(_run_python_api(c, torch.float32, loc_dtype=torch.int64), want, torch.float32)
    _check(_run_python_api(c, torch.float32, loc_dtype=torch.int32), want, torch.float32)


def _reference_style_inputs(shape, seed, levels_hw=(6, 10)):
    """Inputs drawn like the reference test's generator
    (tests/torch/test_geometric_kernel_attention.py:20-41)."""
    bs, nq, d, nh, nl, npnt = shape
    g = torch.Generator().manual_seed(seed)
    h, w = levels_hw
    shapes, starts = workloads.level_tensors([(h, w)] * nl)
    loc = torch.rand(bs, nq, nh, nl, npnt, 2, generator=g)
    loc[..., 0] = loc[..., 0] * (w + 6) - 3
    loc[..., 1] = loc[..., 1] * (h + 6) - 3
    return {
        "shapes": shapes.numpy().astype(np.int32), "starts": starts.numpy().astype(np.int32),
        "value": (torch.rand(bs, h * w * nl, nh, d, generator=g) * 3).numpy(),
        "loc": loc.long().float().numpy(),
        "attn": torch.rand(bs, nq, nh, nl, npnt, generator=g).numpy(),
        "grad_out": (torch.rand(bs, nq, nh * d, generator=g) * 10).numpy(),
    }


# [bs, num_queries, embed_dims, num_heads, num_levels, num_points]: the reference test's shape
# classes (:109-115) with reduced batch / query counts
SHAPES = [[4, 716, 64, 4, 1, 15], [6, 115, 64, 4, 1, 15], [2, 4, 16, 4, 2, 15],
          [2, 300, 32, 8, 4, 8], [1, 200, 128, 2, 2, 32], [2, 100, 8, 3, 4, 3],
          [1, 50, 256, 2, 1, 5]]


@pytest.mark.parametrize("shape", SHAPES, ids=["x".join(map(str, s)) for s in SHAPES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_reference_test_shapes(shape, dtype):
    inp = _reference_style_inputs(shape, seed=zlib.crc32(str(shape).encode()) % 1000,
                                  levels_hw=(15, 25) if shape[0] == 4 else (6, 10))
    rnd = lambda a: torch.from_numpy(a).to(dtype).float().numpy()
    for k in ("value", "attn", "grad_out"):
        inp[k] = rnd(inp[k])
    want_out = msda_oracle.gka_forward(inp["value"], inp["shapes"], inp["starts"], inp["loc"],
                                       inp["attn"])
    want_gv, want_ga = msda_oracle.gka_backward(inp["value"], inp["shapes"], inp["starts"],
                                                inp["loc"], inp["attn"], inp["grad_out"])
    _check(_run_python_api(inp, dtype), (want_out, want_gv, want_ga), dtype)
    _check(_run_c_abi(inp, dtype), (want_out, want_gv, want_ga), dtype)


def test_backward_requires_embed_dims_multiple_of_8():
    """The reference binding refuses other sizes
    (mx_driving/csrc/GeometricKernelAttentionFunc.cpp:96)."""
    inp = _reference_style_inputs([1, 10, 12, 2, 1, 3], seed=1)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        _run_python_api(inp, torch.float32)


def test_large_problem_identities():
    """BEVFormer-sized operands: <grad_out, out> == <grad_value, value> == <grad_attn, attn>
    (the operator is linear in value and in the weights)."""
    w = workloads.WORKLOADS["bevformer_sca"].with_batch(2)
    g = torch.Generator().manual_seed(3)
    shapes, starts = workloads.level_tensors(w.levels)
    loc = torch.empty(w.B, w.Q, w.H, w.L, w.P, 2)
    for l, (h, ww) in enumerate(w.levels):
        loc[:, :, :, l, :, 0] = torch.randint(-3, ww + 3, (w.B, w.Q, w.H, w.P), generator=g).float()
        loc[:, :, :, l, :, 1] = torch.randint(-3, h + 3, (w.B, w.Q, w.H, w.P), generator=g).float()
    inp = {"shapes": shapes.numpy().astype(np.int32), "starts": starts.numpy().astype(np.int32),
           "value": torch.randn(w.B, w.K, w.H, w.D, generator=g).numpy(), "loc": loc.numpy(),
           "attn": torch.rand(w.B, w.Q, w.H, w.L, w.P, generator=g).numpy(),
           "grad_out": torch.randn(w.B, w.Q, w.H * w.D, generator=g).numpy()}
    out, gv, ga = _run_python_api(inp, torch.float32)
    go = torch.from_numpy(inp["grad_out"]).cuda().double()
    lhs = (go * out.double()).sum().item()
    rhs_v = (gv.double() * torch.from_numpy(inp["value"]).cuda().double()).sum().item()
    rhs_a = (ga.double() * torch.from_numpy(inp["attn"]).cuda().double()).sum().item()
    scale = (go.abs() * out.double().abs()).sum().item()
    assert abs(lhs - rhs_v) <= 1e-5 * scale and abs(lhs - rhs_a) <= 1e-5 * scale
    # and a query slice against the oracle
    sub = dict(inp, loc=inp["loc"][:, ::50].copy(), attn=inp["attn"][:, ::50].copy())
    want = msda_oracle.gka_forward(sub["value"], sub["shapes"], sub["starts"], sub["loc"], sub["attn"])
    parity.assert_close("output[slice]", out[:, ::50], want, 1e-4)

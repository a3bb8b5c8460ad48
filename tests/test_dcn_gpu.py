"""Deformable / modulated deformable convolution on the GPU against the golden fixtures
(torchvision's CPU operator, tests/golden/make_dcn_golden.py) and against the oracle on
seeded inputs in the reference tests' value ranges (tests/torch/test_deformable_conv2d.py:60-64,
tests/torch/test_modulated_deformable_conv2d_grad.py:58-67). Tolerances: 1e-4 relative to the
largest magnitude of each tensor for the fp32 FMA products; the reference's own bars (1e-3
forward and input gradients, 1e-2 weight gradient) for the tensor-core products.
"""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import dcn_oracle  # noqa: E402

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(ROOT, "tests", "golden", "dcn_golden.npz"))
CASES = sorted({k.split("/")[0] for k in GOLDEN.files})


def close(got, want, tol, what):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = max(1.0, float(np.abs(want).max()))
    err = float(np.abs(got - want).max())
    assert err <= tol * scale, f"{what}: max error {err:.3e} > {tol:.1e} * {scale:.3e}"


def golden_case(name):
    get = lambda key: GOLDEN[f"{name}/{key}"] if f"{name}/{key}" in GOLDEN.files else None
    N, C, Co, H, W, k, s, p, d, g, dg, modulated, with_bias = (int(v) for v in get("cfg"))
    return get, dict(stride=s, padding=p, dilation=d, groups=g, deform_groups=dg)


def run_python_api(x, offset, mask, weight, bias, grad_out, conv):
    import mx_driving
    dev = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda().requires_grad_()
    xt, ot, mt, wt, bt = dev(x), dev(offset), dev(mask), dev(weight), dev(bias)
    args = (conv["stride"], conv["padding"], conv["dilation"], conv["groups"], conv["deform_groups"])
    if mask is None:
        out = mx_driving.deform_conv2d(xt, ot, wt, *args)
        if bias is not None:
            out = out + bt.view(1, -1, 1, 1)
    else:
        out = mx_driving.modulated_deform_conv2d(xt, ot, mt, wt, bt, *args)
    out.backward(torch.from_numpy(grad_out).cuda())
    cpu = lambda t: None if t is None or t.grad is None else t.grad.cpu().numpy()
    return out.detach().cpu().numpy(), cpu(xt), cpu(ot), cpu(mt), cpu(wt), cpu(bt)


@pytest.mark.parametrize("tensor_cores", [0, 1])
@pytest.mark.parametrize("name", CASES)
def test_golden_through_the_python_api(name, tensor_cores):
    from drivingsdk_b200 import _C
    get, conv = golden_case(name)
    old = _C.dcn_use_tensor_cores(tensor_cores)
    try:
        out, gx, goff, gmask, gw, gb = run_python_api(get("x"), get("offset"), get("mask"),
                                                      get("weight"), get("bias"), get("grad_out"), conv)
    finally:
        _C.dcn_use_tensor_cores(old)
    tol = 1e-4 if tensor_cores == 0 else 1e-3
    close(out, get("out"), tol, "out")
    close(gx, get("grad_x"), tol, "grad_x")
    close(goff, get("grad_offset"), tol, "grad_offset")
    close(gw, get("grad_weight"), tol if tensor_cores == 0 else 1e-2, "grad_weight")
    if get("mask") is not None:
        close(gmask, get("grad_mask"), tol, "grad_mask")
    if get("bias") is not None:
        close(gb, get("grad_bias"), tol, "grad_bias")


def nhwc(a):
    return np.ascontiguousarray(np.transpose(a, (0, 2, 3, 1)))


@pytest.mark.parametrize("name", CASES)
def test_golden_through_the_c_abi(name):
    """Raw device pointers into dcn_sm100_forward / dcn_sm100_backward (channels-last)."""
    from drivingsdk_b200 import capi
    lib = capi.load()
    get, conv = golden_case(name)
    N, C, Co, H, W, k, s, p, d, g, dg, modulated, with_bias = (int(v) for v in get("cfg"))
    Ho, Wo = get("out").shape[2:]
    shape = capi.DcnShape(N, H, W, C, Ho, Wo, Co, k, k, s, s, p, p, d, d, g, dg)
    dev = lambda a: None if a is None else torch.from_numpy(a).cuda()
    ptr = lambda t: None if t is None else t.data_ptr()
    x, off, w = dev(nhwc(get("x"))), dev(nhwc(get("offset"))), dev(nhwc(get("weight")))
    mask = dev(nhwc(get("mask"))) if modulated else None
    bias = dev(get("bias")) if with_bias else None
    go = dev(nhwc(get("grad_out")))
    col_bytes = lib.dcn_sm100_columns_bytes(ctypes.byref(shape))
    assert col_bytes == 4 * N * Ho * Wo * k * k * C
    cols = torch.empty(col_bytes // 4, device="cuda")
    out = torch.empty(N, Ho, Wo, Co, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    capi.check(lib.dcn_sm100_forward(ptr(x), ptr(off), ptr(mask), ptr(w), ptr(bias), ptr(out),
                                     ptr(cols), ctypes.byref(shape), stream), "dcn forward")
    close(out.cpu().numpy(), nhwc(get("out")), 1e-3, "out")
    want_cols = dcn_oracle.columns(get("x"), get("offset"), get("mask"), (k, k), s, p, d, dg)
    # oracle columns are [N, C, K, Ho, Wo]; ours [N*Ho*Wo, G, K, Cg]
    want_cols = want_cols.reshape(N, g, C // g, k * k, Ho, Wo).transpose(0, 4, 5, 1, 3, 2)
    close(cols.cpu().numpy().reshape(want_cols.shape), want_cols, 1e-5, "columns")

    ws_bytes = lib.dcn_sm100_backward_workspace_bytes(ctypes.byref(shape))
    ws = torch.empty(ws_bytes // 4 + 4, device="cuda")
    gx, goff, gw = torch.empty_like(x), torch.empty_like(off), torch.empty_like(w)
    gmask = torch.empty_like(mask) if modulated else None
    gb = torch.empty(Co, device="cuda") if with_bias else None
    capi.check(lib.dcn_sm100_backward(ptr(x), ptr(off), ptr(mask), ptr(w), ptr(cols), ptr(go),
                                      ptr(gx), ptr(goff), ptr(gmask), ptr(gw), ptr(gb), ptr(ws),
                                      ws_bytes, ctypes.byref(shape), stream), "dcn backward")
    close(gx.cpu().numpy(), nhwc(get("grad_x")), 1e-3, "grad_x")
    close(goff.cpu().numpy(), nhwc(get("grad_offset")), 1e-3, "grad_offset")
    close(gw.cpu().numpy(), nhwc(get("grad_weight")), 1e-2, "grad_weight")
    if modulated:
        close(gmask.cpu().numpy(), nhwc(get("grad_mask")), 1e-3, "grad_mask")
    if with_bias:
        close(gb.cpu().numpy(), get("grad_bias"), 1e-3, "grad_bias")
    # too small a workspace is refused before anything is launched
    assert lib.dcn_sm100_backward(ptr(x), ptr(off), ptr(mask), ptr(w), ptr(cols), ptr(go),
                                  ptr(gx), ptr(goff), ptr(gmask), ptr(gw), ptr(gb), ptr(ws),
                                  ws_bytes - 1, ctypes.byref(shape), stream) == -6


SEEDED = [
    # N, C, Co, H, W, k, stride, pad, dil, groups, dg, modulated
    (2, 64, 64, 13, 17, 3, 1, 1, 1, 1, 1, True),
    (1, 128, 64, 11, 9, 3, 1, 1, 1, 8, 1, False),
    (3, 32, 48, 10, 12, 3, 2, 1, 1, 1, 2, True),
    (1, 256, 256, 8, 10, 3, 1, 1, 1, 1, 1, True),
    (2, 12, 20, 9, 7, 3, 1, 2, 2, 1, 3, False),
    (1, 6, 5, 7, 8, 3, 1, 1, 1, 1, 1, True),       # channel count that is not a multiple of 4
]


@pytest.mark.parametrize("tensor_cores", [0, 1])
@pytest.mark.parametrize("cfg", SEEDED)
def test_seeded_inputs_against_the_oracle(cfg, tensor_cores):
    from drivingsdk_b200 import _C
    N, C, Co, H, W, k, s, p, d, g, dg, modulated = cfg
    rng = np.random.default_rng(sum((i + 1) * int(v) for i, v in enumerate(cfg)))
    Ho, Wo = dcn_oracle.out_size(H, k, s, p, d), dcn_oracle.out_size(W, k, s, p, d)
    u = lambda *shape: rng.uniform(-5, 5, shape).astype(np.float32)
    x, offset = u(N, C, H, W), u(N, dg * 2 * k * k, Ho, Wo)
    weight = (u(Co, C // g, k, k) * 0.01).astype(np.float32)
    mask = u(N, dg * k * k, Ho, Wo) if modulated else None
    grad_out = u(N, Co, Ho, Wo)
    conv = dict(stride=s, padding=p, dilation=d, groups=g, deform_groups=dg)
    old = _C.dcn_use_tensor_cores(tensor_cores)
    try:
        out, gx, goff, gmask, gw, _ = run_python_api(x, offset, mask, weight, None, grad_out, conv)
    finally:
        _C.dcn_use_tensor_cores(old)
    want_out = dcn_oracle.forward(x, offset, mask, weight, None, **conv)
    wx, woff, wmask, ww, _ = dcn_oracle.backward(x, offset, mask, weight, grad_out, **conv)
    tol = 1e-4 if tensor_cores == 0 else 1e-3
    close(out, want_out, tol, "out")
    close(gx, wx, tol, "grad_x")
    close(goff, woff, tol, "grad_offset")
    close(gw, ww, tol if tensor_cores == 0 else 1e-2, "grad_weight")
    if modulated:
        close(gmask, wmask, tol, "grad_mask")


def test_offsets_outside_the_image_and_nan_give_zeros():
    import mx_driving
    x = torch.randn(1, 8, 5, 6, device="cuda")
    w = torch.randn(4, 8, 3, 3, device="cuda")
    for bad in (1e4, -1e4, float("nan"), float("inf")):
        off = torch.full((1, 18, 5, 6), bad, device="cuda", requires_grad=True)
        xr = x.clone().requires_grad_()
        out = mx_driving.deform_conv2d(xr, off, w, 1, 1)
        assert torch.count_nonzero(out) == 0
        out.backward(torch.ones_like(out))
        assert torch.count_nonzero(xr.grad) == 0 and torch.count_nonzero(off.grad) == 0


def test_zero_offsets_reduce_to_a_plain_convolution():
    import mx_driving
    g = torch.Generator().manual_seed(7)
    x = torch.randn(2, 16, 9, 11, generator=g).cuda()
    w = (torch.randn(24, 8, 3, 3, generator=g) * 0.1).cuda()
    off = torch.zeros(2, 18, 9, 11, device="cuda")
    mask = torch.ones(2, 9, 9, 11, device="cuda")
    want = torch.nn.functional.conv2d(x, w, None, 1, 1, 1, 2)
    torch.testing.assert_close(mx_driving.deform_conv2d(x, off, w, 1, 1, 1, 2), want, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(mx_driving.modulated_deform_conv2d(x, off, mask, w, None, 1, 1, 1, 2),
                               want, rtol=1e-3, atol=1e-3)


def test_argument_checks():
    import mx_driving
    off = torch.zeros(1, 18, 5, 5, device="cuda")
    x = torch.randn(1, 8, 5, 5, device="cuda")
    w = torch.randn(4, 8, 3, 3, device="cuda")
    with pytest.raises(RuntimeError):                 # offset for the wrong output size
        mx_driving.deform_conv2d(x, torch.zeros(1, 18, 4, 5, device="cuda"), w, 1, 1)
    with pytest.raises(RuntimeError):                 # CPU tensors
        mx_driving.deform_conv2d(x.cpu(), off.cpu(), w.cpu(), 1, 1)


def test_full_size_identities_and_agreement_of_the_product_kernels():
    """The reference's unit-test shape (N=18, C=Co=512, 29x50; tests/torch/test_deformable_conv2d.py:59)
    is too large for the CPU oracle, so it is checked through properties that hold at any size:
    the operator is linear in x and in the weights for fixed offsets and masks, hence
    <grad_out, out> = <grad_x, x> = <grad_weight, weight> = <grad_mask, mask>; and the tensor-core
    products must agree with the fp32 FMA products."""
    import mx_driving
    from drivingsdk_b200 import _C
    N, C, Co, H, W = 18, 512, 512, 29, 50
    g = torch.Generator().manual_seed(11)
    u = lambda lo, hi, *shape: (torch.rand(*shape, generator=g) * (hi - lo) + lo).cuda()
    x, off, mask = u(-5, 5, N, C, H, W), u(-5, 5, N, 18, H, W), u(-5, 5, N, 9, H, W)
    w, go = u(-0.05, 0.05, Co, C, 3, 3), u(-1, 1, N, Co, H, W)
    results = {}
    for mode in (1, 0):
        old = _C.dcn_use_tensor_cores(mode)
        try:
            xt, ot, mt, wt = (t.clone().requires_grad_() for t in (x, off, mask, w))
            out = mx_driving.modulated_deform_conv2d(xt, ot, mt, wt, None, 1, 1, 1)
            out.backward(go)
            results[mode] = (out.detach(), xt.grad, ot.grad, mt.grad, wt.grad)
        finally:
            _C.dcn_use_tensor_cores(old)
    out, gx, goff, gmask, gw = results[1]
    dot = lambda a, b: (a.double() * b.double()).sum().item()
    ref = dot(go, out)
    # the inner products cancel heavily (13 M terms of either sign), so the bar is relative to
    # the norms of the factors, not to the result
    bar = 1e-5 * go.double().norm().item() * out.double().norm().item()
    for name, val in (("x", dot(gx, x)), ("weight", dot(gw, w)), ("mask", dot(gmask, mask))):
        assert abs(val - ref) <= bar, (name, val, ref, bar)
    for name, a, b in zip(("out", "grad_x", "grad_offset", "grad_mask", "grad_weight"), results[1], results[0]):
        scale = b.abs().max().item()
        err = (a - b).abs().max().item()
        assert err <= 1e-4 * scale, (name, err, scale)
    # linearity in x for fixed offsets and masks
    with torch.no_grad():
        o2 = mx_driving.modulated_deform_conv2d(2.5 * x, off, mask, w, None, 1, 1, 1)
    assert (o2 - 2.5 * out).abs().max().item() <= 1e-4 * out.abs().max().item()


def test_sixteen_bit_inputs_are_computed_in_fp32():
    """fp16 / bf16 tensors are converted, computed in fp32 and returned in their own dtype
    (the reference wraps the modulated operator in custom_fwd(cast_inputs=float32),
    mx_driving/ops/modulated_deform_conv2d.py:21-26)."""
    import mx_driving
    g = torch.Generator().manual_seed(5)
    u = lambda lo, hi, *shape: (torch.rand(*shape, generator=g) * (hi - lo) + lo).cuda()
    x, off, mask, w = u(-2, 2, 2, 16, 8, 9), u(-2, 2, 2, 18, 8, 9), u(0, 1, 2, 9, 8, 9), u(-0.2, 0.2, 8, 16, 3, 3)
    want = mx_driving.modulated_deform_conv2d(x, off, mask, w, None, 1, 1, 1)
    for dtype in (torch.float16, torch.bfloat16):
        xh, oh, mh, wh = (t.to(dtype).requires_grad_() for t in (x, off, mask, w))
        ref = mx_driving.modulated_deform_conv2d(xh.float(), oh.float(), mh.float(), wh.float(), None, 1, 1, 1)
        out = mx_driving.deform_conv2d(xh, oh, wh, 1, 1, 1)
        assert out.dtype == dtype
        with torch.autocast("cuda", dtype=dtype):
            outm = mx_driving.modulated_deform_conv2d(xh, oh, mh, wh, None, 1, 1, 1)
        assert outm.dtype == torch.float32          # cast_inputs=float32, as in the reference
        torch.testing.assert_close(outm, ref.detach(), rtol=1e-4, atol=1e-4)
        outm.sum().backward()
        assert xh.grad.dtype == dtype and wh.grad.dtype == dtype and mh.grad is not None
    assert torch.isfinite(want).all()

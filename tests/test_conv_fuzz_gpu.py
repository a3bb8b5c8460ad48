"""Seeded random shapes for the matrix product (both operand orders, all three modes) and for
the deformable convolution (against the oracle): tails in every dimension, strides with
padding, groups, dilation, stride, odd channel counts."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import dcn_oracle  # noqa: E402

pytestmark = pytest.mark.gpu


def _gemm_case(rng, row_contiguous):
    from drivingsdk_b200 import capi
    lib = capi.load()
    M, N = int(rng.integers(1, 700)), int(rng.integers(1, 700))
    K = int(rng.integers(1, 1500))
    if row_contiguous and rng.random() < 0.7:       # mostly shapes the tensor-core path takes
        M, N = 32 * int(rng.integers(1, 12)), 32 * int(rng.integers(1, 12))
    pad_a, pad_b = (int(4 * rng.integers(0, 3)) for _ in range(2))
    mode = int(rng.integers(0, 3))
    splits = int(rng.integers(1, 5))
    g = torch.Generator().manual_seed(int(rng.integers(1 << 30)))
    if row_contiguous:
        A = torch.randn(K, M + pad_a, generator=g).cuda()
        B = torch.randn(K, N + pad_b, generator=g).cuda()
        want = A[:, :M].double().t() @ B[:, :N].double()
    else:
        A = torch.randn(M, K + pad_a, generator=g).cuda()
        B = torch.randn(N, K + pad_b, generator=g).cuda()
        want = A[:, :K].double() @ B[:, :K].double().t()
    C = torch.full((M, N), float("nan"), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    old = lib.dcn_sm100_use_tensor_cores(mode)
    try:
        if row_contiguous:
            rc = lib.gemm_tn_sm100_f32(A.data_ptr(), M + pad_a, B.data_ptr(), N + pad_b, C.data_ptr(), N,
                                       M, N, K, splits, st)
        else:
            rc = lib.gemm_nt_sm100_f32(A.data_ptr(), K + pad_a, B.data_ptr(), K + pad_b, C.data_ptr(), N,
                                       None, M, N, K, splits, st)
    finally:
        lib.dcn_sm100_use_tensor_cores(old)
    capi.check(rc, "gemm")
    torch.cuda.synchronize()
    err = (C.double() - want).abs().max().item()
    scale = max(want.abs().max().item(), 1e-6)
    tol = {0: 2e-5, 1: 5e-5, 2: 4e-3}[mode]
    assert err <= tol * scale, dict(M=M, N=N, K=K, mode=mode, splits=splits, rc=row_contiguous,
                                    err=err, scale=scale)


@pytest.mark.parametrize("row_contiguous", [False, True])
def test_random_products(row_contiguous):
    from drivingsdk_b200 import capi
    rng = np.random.default_rng(2024 + int(row_contiguous))
    for _ in range(60):
        _gemm_case(rng, row_contiguous)
    assert capi.load().msda_sm100_device_status(1) == 0


def test_random_deformable_convolutions():
    import mx_driving
    from drivingsdk_b200 import _C, capi
    rng = np.random.default_rng(77)
    for case in range(24):
        groups = int(rng.choice([1, 1, 2, 4]))
        dg = int(rng.choice([1, 1, 2]))
        unit = int(np.lcm(groups, dg))
        C = unit * int(rng.integers(1, 9)) * int(rng.choice([1, 4]))
        Co = groups * int(rng.integers(1, 12))
        k = int(rng.choice([1, 3, 3, 5]))
        stride, dil = int(rng.choice([1, 1, 2])), int(rng.choice([1, 1, 2]))
        pad = int(rng.integers(0, 3))
        H, W = int(rng.integers(k * dil, 14)) + 1, int(rng.integers(k * dil, 14)) + 1
        Ho, Wo = dcn_oracle.out_size(H, k, stride, pad, dil), dcn_oracle.out_size(W, k, stride, pad, dil)
        if Ho < 1 or Wo < 1:
            continue
        N = int(rng.integers(1, 4))
        modulated = bool(rng.integers(0, 2))
        u = lambda *shape: rng.uniform(-3, 3, shape).astype(np.float32)
        x, off = u(N, C, H, W), u(N, dg * 2 * k * k, Ho, Wo)
        w = (u(Co, C // groups, k, k) * 0.1).astype(np.float32)
        mask = u(N, dg * k * k, Ho, Wo) if modulated else None
        go = u(N, Co, Ho, Wo)
        conv = dict(stride=stride, padding=pad, dilation=dil, groups=groups, deform_groups=dg)
        mode = case % 2
        old = _C.dcn_use_tensor_cores(mode)
        try:
            t = lambda a: None if a is None else torch.from_numpy(a).cuda().requires_grad_()
            xt, ot, mt, wt = t(x), t(off), t(mask), t(w)
            args = (stride, pad, dil, groups, dg)
            out = (mx_driving.modulated_deform_conv2d(xt, ot, mt, wt, None, *args) if modulated
                   else mx_driving.deform_conv2d(xt, ot, wt, *args))
            out.backward(torch.from_numpy(go).cuda())
        finally:
            _C.dcn_use_tensor_cores(old)
        want = dcn_oracle.forward(x, off, mask, w, None, **conv)
        gx, goff, gmask, gw, _ = dcn_oracle.backward(x, off, mask, w, go, **conv)
        info = dict(case=case, N=N, C=C, Co=Co, H=H, W=W, k=k, mode=mode, **conv)
        pairs = [("out", out, want), ("grad_x", xt.grad, gx), ("grad_offset", ot.grad, goff),
                 ("grad_weight", wt.grad, gw)]
        if modulated:
            pairs.append(("grad_mask", mt.grad, gmask))
        for name, got, ref in pairs:
            err = np.abs(got.detach().cpu().numpy() - ref).max()
            assert err <= 1e-4 * max(1.0, np.abs(ref).max()), (name, err, info)
    assert capi.load().msda_sm100_device_status(1) == 0

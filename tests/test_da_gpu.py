"""Parity of the deformable-aggregation CUDA path (needs a GPU)."""
import zlib

import numpy as np
import pytest
import torch

from oracle import msda_oracle
from tests import parity
from tests.test_da_oracle import NAMES, case

pytestmark = pytest.mark.gpu


def _run_python_api(c, dtype=torch.float32):
    import drivingsdk_b200 as sdk
    feat = torch.from_numpy(c["feat"]).to("cuda", dtype).requires_grad_(True)
    loc = torch.from_numpy(c["loc"]).to("cuda", dtype).requires_grad_(True)
    wts = torch.from_numpy(c["wts"]).to("cuda", dtype).requires_grad_(True)
    shapes = torch.from_numpy(c["shapes"]).cuda()
    starts = torch.from_numpy(c["starts"]).cuda()
    out = sdk.deformable_aggregation(feat, shapes, starts, loc, wts)
    out.backward(torch.from_numpy(c["grad_out"]).to("cuda", dtype))
    return out.detach(), feat.grad, loc.grad, wts.grad


def _run_c_abi(c, host_tables=False):
    from drivingsdk_b200 import capi
    lib = capi.load()
    dev = {k: torch.from_numpy(c[k]).cuda() for k in ("feat", "loc", "wts", "grad_out")}
    shapes = torch.from_numpy(c["shapes"]).to(torch.int32).contiguous()
    starts = torch.from_numpy(c["starts"]).to(torch.int32).contiguous()
    if not host_tables:
        shapes, starts = shapes.cuda(), starts.cuda()
    B, F, C = dev["feat"].shape
    _, A, Pts, cams, scales, G = dev["wts"].shape
    dims = (B, F, C, A, Pts, cams, scales, G)
    out = torch.empty(B, A, C, device="cuda")
    gf, gl, gw = (torch.empty_like(dev[k]) for k in ("feat", "loc", "wts"))
    stream = torch.cuda.current_stream().cuda_stream
    capi.check(lib.da_sm100_forward(dev["feat"].data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                    dev["loc"].data_ptr(), dev["wts"].data_ptr(), out.data_ptr(),
                                    *dims, stream), "da forward")
    capi.check(lib.da_sm100_backward(dev["feat"].data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                     dev["loc"].data_ptr(), dev["wts"].data_ptr(),
                                     dev["grad_out"].data_ptr(), gf.data_ptr(), gl.data_ptr(),
                                     gw.data_ptr(), *dims, stream), "da backward")
    torch.cuda.synchronize()
    return out, gf, gl, gw


def _check(c, results, tol=1e-4):
    want_out = msda_oracle.da_forward(c["feat"], c["shapes"], c["starts"], c["loc"], c["wts"])
    gf, gl, gw = msda_oracle.da_backward(c["feat"], c["shapes"], c["starts"], c["loc"], c["wts"],
                                         c["grad_out"])
    parity.assert_close("out", results[0], want_out, tol)
    parity.assert_close("grad_feat", results[1], gf, tol)
    parity.assert_close("grad_weights", results[3], gw, tol)
    # grad_loc sums W * weight * grad_out * (value differences) over all channels and scales:
    # its float32 rounding scales with that sum's terms, not with the result
    parity.assert_close("grad_loc", results[2], gl, tol * 10)


@pytest.mark.parametrize("name", NAMES)
def test_golden_fixture(name):
    c = case(name)
    res = _run_c_abi(c)
    parity.assert_close("out vs reference golden", res[0], c["out"].astype(np.float64), 1e-4)
    _check(c, res)
    _check(c, _run_c_abi(c, host_tables=True))
    _check(c, _run_python_api(c))


def _random_case(seed, B, C, A, Pts, G, maps):
    rng = np.random.default_rng(seed)
    cams, scales = len(maps), len(maps[0])
    shapes = np.array(maps, dtype=np.int32).reshape(cams, scales, 2)
    sizes = (shapes[..., 0] * shapes[..., 1]).reshape(-1)
    starts = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int32).reshape(cams, scales)
    return {"feat": rng.random((B, int(sizes.sum()), C), dtype=np.float32),
            "shapes": shapes, "starts": starts,
            "loc": (rng.random((B, A, Pts, cams, 2), dtype=np.float32) * 1.1 - 0.05).astype(np.float32),
            "wts": rng.random((B, A, Pts, cams, scales, G), dtype=np.float32),
            "grad_out": rng.standard_normal((B, A, C), dtype=np.float32)}


# the reference test's grid (tests/torch/test_deformable_aggregation.py:131-135): B in {1,5,10},
# C in {32,64}, groups in {8,16}, anchors in {10,13,18}, pts in {10,50,31}, one 32x88 map
REF_GRID = [(1, 32, 10, 10, 8), (5, 64, 13, 50, 16), (10, 32, 18, 31, 16), (5, 64, 10, 31, 8)]


@pytest.mark.parametrize("B,C,A,Pts,G", REF_GRID)
def test_reference_test_grid(B, C, A, Pts, G):
    c = _random_case(zlib.crc32(str((B, C, A, Pts, G)).encode()), B, C, A, Pts, G, [[(32, 88)]])
    _check(c, _run_python_api(c))


def test_sparse4d_shape():
    """Sparse4D-like call: 6 cameras x 4 scales, 256 channels in 8 groups, 13 points."""
    maps = [[(16, 44), (8, 22), (4, 11), (2, 6)]] * 6
    c = _random_case(5, 1, 256, 60, 13, 8, maps)
    _check(c, _run_c_abi(c))
    _check(c, _run_python_api(c))


@pytest.mark.parametrize("C,G", [(256, 1), (256, 2), (128, 1), (64, 1), (40, 2)])
def test_wide_channel_groups_through_c_abi(C, G):
    """Few groups over many channels (up to 256 channels in one group), which only the C ABI
    accepts (the Python wrapper wants a multiple of 8 groups): every group's dot product must
    cover all of its channels."""
    c = _random_case(zlib.crc32(str((C, G)).encode()), 2, C, 7, 5, G, [[(9, 14), (5, 7)]] * 2)
    _check(c, _run_c_abi(c))
    _check(c, _run_c_abi(c, host_tables=True))


def test_half_precision_inputs_round_trip():
    c = _random_case(9, 2, 64, 8, 6, 8, [[(6, 9), (3, 5)]] * 2)
    for k in ("feat", "loc", "wts", "grad_out"):
        c[k] = torch.from_numpy(c[k]).half().float().numpy()
    out, gf, gl, gw = _run_python_api(c, torch.float16)
    assert out.dtype == torch.float16 and gf.dtype == torch.float16
    want = msda_oracle.da_forward(c["feat"], c["shapes"], c["starts"], c["loc"], c["wts"])
    parity.assert_close("out", out, torch.from_numpy(want).half().double().numpy(), 1e-2)


def test_group_count_must_be_multiple_of_8():
    c = _random_case(1, 1, 32, 2, 2, 4, [[(4, 4)]])
    with pytest.raises(RuntimeError, match="multiple of 8"):
        _run_python_api(c)

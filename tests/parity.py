"""Shared helpers of the GPU parity tests: run the CUDA path, run the oracle, compare."""
import numpy as np
import torch

from oracle import msda_oracle

# tolerances of the acceptance contract: |a - b| <= atol + rtol * |b|
TOL = {torch.float32: 1e-4, torch.float16: 1e-2, torch.bfloat16: 1e-2}
# grad_sampling_loc is a one-sided derivative where a sample sits on a pixel
# boundary; float32 pixel coordinates (|x| up to a few hundred) resolve about
# 3e-5, so samples closer than this to a boundary are not compared.
# 16-bit locations times a level size are exact in float32, so the kernel and the
# oracle always pick the same cell and nothing needs masking there.
KINK_EPS = {torch.float32: 1e-4, torch.float16: -1.0, torch.bfloat16: -1.0}
# ... and no comparison may leave out more than this share of its samples (or 4 samples, for
# tiny cases): uniformly drawn locations put about 4e-4 of them that close to a boundary.
MAX_KINK_FRACTION = 2e-3


def oracle_all(inp):
    """float64 (out, grad_value, grad_loc, grad_attn) for a dict from workloads.make_inputs
    or a golden case (numpy or torch float32 containers)."""
    n = lambda k: inp[k].numpy() if isinstance(inp[k], torch.Tensor) else inp[k]
    out = msda_oracle.forward(n("value"), n("shapes"), n("starts"), n("loc"), n("attn"))
    gv, gl, ga = msda_oracle.backward(n("value"), n("shapes"), n("starts"), n("loc"), n("attn"),
                                      n("grad_out"))
    return out, gv, gl, ga


def to_device(inp, dtype, device="cuda"):
    t = lambda k: (torch.from_numpy(inp[k]) if not isinstance(inp[k], torch.Tensor) else inp[k])
    d = {k: t(k).to(device=device, dtype=dtype) for k in ("value", "loc", "attn", "grad_out")}
    d["shapes"] = t("shapes").to(device=device)
    d["starts"] = t("starts").to(device=device)
    return d


def run_python_api(dev):
    """Forward + backward through the public autograd function."""
    import drivingsdk_b200 as sdk
    value = dev["value"].clone().requires_grad_(True)
    loc = dev["loc"].clone().requires_grad_(True)
    attn = dev["attn"].clone().requires_grad_(True)
    out = sdk.multi_scale_deformable_attn(value, dev["shapes"], dev["starts"], loc, attn)
    out.backward(dev["grad_out"])
    return out.detach(), value.grad, loc.grad, attn.grad


def run_c_abi(dev, dtype, workspace=True, host_levels=False, lib=None):
    """Forward + backward through the C ABI with raw device pointers (``lib``: which build of
    the library, default the normal one)."""
    from drivingsdk_b200 import capi
    if lib is None:
        lib = capi.load()
    value, loc, attn, go = dev["value"], dev["loc"], dev["attn"], dev["grad_out"]
    B, K, H, D = value.shape
    _, Q, _, L, P, _ = loc.shape
    shapes = dev["shapes"].to(torch.int32).contiguous()
    starts = dev["starts"].to(torch.int32).contiguous()
    if host_levels:
        shapes, starts = shapes.cpu(), starts.cpu()
    out = torch.empty(B, Q, H * D, device=value.device, dtype=dtype)
    gv = torch.empty_like(value)
    gl = torch.empty_like(loc)
    ga = torch.empty_like(attn)
    code = capi.dtype_code(dtype)
    stream = torch.cuda.current_stream().cuda_stream
    dims = (B, K, H, D, L, Q, P)
    capi.check(lib.msda_sm100_forward(value.data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                      loc.data_ptr(), attn.data_ptr(), out.data_ptr(), *dims,
                                      code, stream), "forward")
    if workspace:
        nbytes = lib.msda_sm100_backward_workspace_bytes(B, K, H, D, code)
        ws = torch.empty(max(nbytes, 16), device=value.device, dtype=torch.uint8)
        capi.check(lib.msda_sm100_backward_ws(
            value.data_ptr(), shapes.data_ptr(), starts.data_ptr(), loc.data_ptr(), attn.data_ptr(),
            go.data_ptr(), gv.data_ptr(), gl.data_ptr(), ga.data_ptr(), ws.data_ptr(), nbytes,
            *dims, code, stream), "backward_ws")
    else:
        capi.check(lib.msda_sm100_backward(
            value.data_ptr(), shapes.data_ptr(), starts.data_ptr(), loc.data_ptr(), attn.data_ptr(),
            go.data_ptr(), gv.data_ptr(), gl.data_ptr(), ga.data_ptr(), *dims, code, stream),
            "backward")
    torch.cuda.synchronize()
    return out, gv, gl, ga


def assert_close(name, got, want, tol, mask=None):
    got = got.detach().double().cpu().numpy().reshape(want.shape)
    err = np.abs(got - want)
    bound = tol + tol * np.abs(want)
    bad = err > bound
    if mask is not None:
        bad &= mask
    if bad.any():
        i = np.unravel_index(np.argmax(np.where(bad, err - bound, -1)), bad.shape)
        raise AssertionError(
            f"{name}: {int(bad.sum())} of {bad.size} elements outside rtol=atol={tol}; worst at {i}: "
            f"got {got[i]!r}, want {want[i]!r}")
    return float(err.max())


def compare_all(inp, results, dtype):
    """Checks (out, grad_value, grad_loc, grad_attn) against the float64 oracle.
    The oracle's results are rounded to ``dtype`` first when it is a 16-bit type,
    as the reference test does for float16
    (tests/torch/test_multi_scale_deformable_attn.py:256-264)."""
    want = oracle_all(inp)
    if dtype != torch.float32:
        want = tuple(torch.from_numpy(w).to(dtype).double().numpy() for w in want)
    n = lambda k: inp[k].numpy() if isinstance(inp[k], torch.Tensor) else inp[k]
    dist = msda_oracle.kink_distance(n("shapes"), n("loc"))
    smooth = dist > KINK_EPS[dtype]
    tol = TOL[dtype]
    out, gv, gl, ga = results
    errs = {
        "out": assert_close("output", out, want[0], tol),
        "grad_value": assert_close("grad_value", gv, want[1], tol),
        "grad_attn": assert_close("grad_attn_weight", ga, want[3], tol),
        "grad_loc": assert_close("grad_sampling_loc", gl, want[2], tol,
                                 mask=np.broadcast_to(smooth[..., None], want[2].shape)),
    }
    errs["kink_masked"] = int((~smooth).sum())
    assert errs["kink_masked"] <= max(4, MAX_KINK_FRACTION * smooth.size), \
        f"{errs['kink_masked']} of {smooth.size} samples masked as boundary samples"
    return errs

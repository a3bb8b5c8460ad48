"""Parity of the CUDA path with the oracle and the reference's golden outputs (needs a GPU)."""
import zlib

import numpy as np
import pytest
import torch

from drivingsdk_b200 import workloads
from tests import parity
from tests.golden_cases import CASES, NAMES

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def _golden_check(case, results, dtype):
    tol = parity.TOL[dtype]
    want = [case[k] for k in ("out", "grad_value", "grad_loc", "grad_attn")]
    if dtype != torch.float32:
        want = [torch.from_numpy(w).to(dtype).double().numpy() for w in want]
    from oracle import msda_oracle
    smooth = msda_oracle.kink_distance(case["shapes"], case["loc"]) > parity.KINK_EPS[dtype]
    parity.assert_close("output", results[0], want[0], tol)
    parity.assert_close("grad_value", results[1], want[1], tol)
    parity.assert_close("grad_sampling_loc", results[2], want[2], tol,
                        mask=np.broadcast_to(smooth[..., None], want[2].shape))
    parity.assert_close("grad_attn_weight", results[3], want[3], tol)


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("stage", [0, 1, 2])
def test_golden_fixture_through_c_abi(name, stage):
    """CUDA kernels, called through the C ABI, against the reference golden's own outputs."""
    from drivingsdk_b200 import capi
    case = CASES[name]
    dtype = DTYPES[case["dtype"]]
    prev = capi.load().msda_sm100_tune(capi.TUNE_STAGE, stage)
    try:
        dev = parity.to_device(case, dtype)
        _golden_check(case, parity.run_c_abi(dev, dtype), dtype)
    finally:
        capi.load().msda_sm100_tune(capi.TUNE_STAGE, prev)
    assert capi.load().msda_sm100_device_status(1) == 0


@pytest.mark.parametrize("name", NAMES)
def test_golden_fixture_through_python_api(name):
    case = CASES[name]
    dtype = DTYPES[case["dtype"]]
    dev = parity.to_device(case, dtype)
    _golden_check(case, parity.run_python_api(dev), dtype)


@pytest.mark.parametrize("name", ["tiny_border", "toy_slice", "unaligned_d37"])
def test_host_level_arrays(name):
    """spatial_shapes / level_start_index given as host memory (passed by value)."""
    case = CASES[name]
    dev = parity.to_device(case, torch.float32)
    _golden_check(case, parity.run_c_abi(dev, torch.float32, host_levels=True), torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_toy_config_full(dtype):
    w = workloads.WORKLOADS["toy"]
    inp = workloads.make_inputs(w, dtype)
    dev = parity.to_device(inp, dtype)
    parity.compare_all(inp, parity.run_python_api(dev), dtype)
    parity.compare_all(inp, parity.run_c_abi(dev, dtype), dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_direct_16bit_accumulation(dtype):
    """msda_sm100_backward (no workspace): grad_value accumulated with 16-bit vector atomics.
    Every atomic add rounds the running sum to the 16-bit type, so the error of a grad_value
    row grows with the number of samples that hit it (about 75 here); this entry point is
    held to 1e-2 for float16 and 5e-2 for bfloat16 on grad_value, the other three results
    to the usual 1e-2. The workspace entry point (fp32 accumulation) has no such growth."""
    w = workloads.WORKLOADS["toy"].with_queries(200)
    inp = workloads.make_inputs(w, dtype)
    dev = parity.to_device(inp, dtype)
    out, gv, gl, ga = parity.run_c_abi(dev, dtype, workspace=False)
    want = [torch.from_numpy(x).to(dtype).double().numpy() for x in parity.oracle_all(inp)]
    parity.assert_close("output", out, want[0], 1e-2)
    parity.assert_close("grad_value", gv, want[1], 1e-2 if dtype == torch.float16 else 5e-2)
    parity.assert_close("grad_sampling_loc", gl, want[2], 1e-2)
    parity.assert_close("grad_attn_weight", ga, want[3], 1e-2)


# shapes of the reference's unit test, [bs, num_queries, embed_dims, num_heads, num_levels,
# num_points] (tests/torch/test_multi_scale_deformable_attn.py:156-264), with the query count
# and level size reduced so that the oracle finishes in seconds; the reference draws
# value*0.01, loc in [0,1), weights rand+1e-5 (not normalised) and grad_output*1e-3.
REFERENCE_TEST_SHAPES = [
    ("fast_mode", [2, 300, 32, 8, 1, 8], torch.float32),
    ("embed_32", [2, 300, 32, 8, 4, 4], torch.float32),
    ("embed_unaligned", [2, 200, 37, 4, 5, 3], torch.float32),
    ("embed_16", [1, 500, 16, 5, 3, 1], torch.float32),
    ("embed_64", [1, 300, 64, 6, 1, 2], torch.float32),
    ("fully_embed_64", [1, 100, 64, 8, 8, 8], torch.float32),
    ("fully_embed_128", [1, 100, 128, 8, 8, 8], torch.float32),
    ("fully_embed_256", [1, 100, 256, 8, 8, 8], torch.float32),
    ("fully_unaligned", [1, 100, 147, 7, 3, 21], torch.float32),
    ("point_16", [1, 150, 32, 7, 4, 16], torch.float32),
    ("fp16", [2, 300, 32, 8, 4, 4], torch.float16),
    ("bf16_d128", [1, 100, 128, 8, 4, 4], torch.bfloat16),
    ("bf16_d8", [1, 100, 8, 3, 2, 2], torch.bfloat16),
    ("fp16_unaligned", [1, 60, 37, 4, 5, 3], torch.float16),
]


def _reference_style_inputs(shape, dtype, seed):
    bs, nq, d, nh, nl, npnt = shape
    g = torch.Generator().manual_seed(seed)
    levels = [(12, 10)] * nl
    shapes, starts = workloads.level_tensors(levels)
    nk = 120 * nl
    rnd = lambda t: t.to(dtype).float()
    return {
        "shapes": shapes, "starts": starts,
        "value": rnd(torch.rand(bs, nk, nh, d, generator=g) * 0.01),
        "loc": rnd(torch.rand(bs, nq, nh, nl, npnt, 2, generator=g)),
        "attn": rnd(torch.rand(bs, nq, nh, nl, npnt, generator=g) + 1e-5),
        "grad_out": rnd(torch.rand(bs, nq, nh * d, generator=g) * 1e-3),
    }


@pytest.mark.parametrize("label,shape,dtype", REFERENCE_TEST_SHAPES,
                         ids=[s[0] for s in REFERENCE_TEST_SHAPES])
def test_reference_unit_test_shapes(label, shape, dtype):
    inp = _reference_style_inputs(shape, dtype, seed=zlib.crc32(label.encode()) % 1000)
    dev = parity.to_device(inp, dtype)
    parity.compare_all(inp, parity.run_python_api(dev), dtype)


@pytest.mark.parametrize("fill", [float("nan"), float("inf")])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_nonfinite_inputs_give_zeros(fill, dtype):
    """All-NaN and all-Inf operands give exact zeros in the output and all three gradients
    (tests/torch/test_multi_scale_deformable_attn.py:266-282)."""
    inp = _reference_style_inputs([2, 200, 32, 8, 4, 4], dtype, seed=5)
    for k in ("value", "loc", "attn", "grad_out"):
        inp[k].fill_(fill)
    dev = parity.to_device(inp, dtype)
    for res in parity.run_python_api(dev):
        assert torch.count_nonzero(res).item() == 0


def test_empty_inputs_raise():
    import drivingsdk_b200 as sdk
    shapes = torch.tensor([[2, 2]], device="cuda")
    starts = torch.tensor([0], device="cuda")
    with pytest.raises(Exception):
        sdk.multi_scale_deformable_attn(torch.empty(0, 4, 2, 8, device="cuda"), shapes, starts,
                                        torch.empty(0, 3, 2, 1, 2, 2, device="cuda"),
                                        torch.empty(0, 3, 2, 1, 2, device="cuda"))


def test_limits_raise():
    import drivingsdk_b200 as sdk
    shapes = torch.tensor([[2, 2]], device="cuda")
    starts = torch.tensor([0], device="cuda")
    with pytest.raises(RuntimeError, match="embedding dimensions"):
        sdk.multi_scale_deformable_attn(torch.zeros(1, 4, 2, 257, device="cuda"), shapes, starts,
                                        torch.zeros(1, 3, 2, 1, 2, 2, device="cuda"),
                                        torch.zeros(1, 3, 2, 1, 2, device="cuda"))
    with pytest.raises(RuntimeError, match="levels and the number of points"):
        sdk.multi_scale_deformable_attn(torch.zeros(1, 4, 2, 8, device="cuda"), shapes, starts,
                                        torch.zeros(1, 3, 2, 1, 65, 2, device="cuda"),
                                        torch.zeros(1, 3, 2, 1, 65, device="cuda"))
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        sdk.multi_scale_deformable_attn(torch.zeros(1, 4, 2, 8), shapes.cpu(), starts.cpu(),
                                        torch.zeros(1, 3, 2, 1, 2, 2), torch.zeros(1, 3, 2, 1, 2))


def test_autocast_casts_to_float32():
    """Under autocast the op runs in float32 (custom_fwd(cast_inputs=float32),
    mx_driving/ops/multi_scale_deformable_attn.py:20)."""
    import drivingsdk_b200 as sdk
    w = workloads.WORKLOADS["toy"].with_queries(64)
    inp = workloads.make_inputs(w, torch.float16)
    dev = parity.to_device(inp, torch.float16)
    with torch.autocast("cuda", dtype=torch.float16):
        out = sdk.multi_scale_deformable_attn(dev["value"], dev["shapes"], dev["starts"],
                                              dev["loc"], dev["attn"])
    assert out.dtype == torch.float32
    want = parity.oracle_all(inp)[0]
    parity.assert_close("output", out, want, 1e-4)


def test_non_contiguous_inputs():
    import drivingsdk_b200 as sdk
    w = workloads.WORKLOADS["toy"].with_queries(50)
    inp = workloads.make_inputs(w, torch.float32)
    dev = parity.to_device(inp, torch.float32)
    value_nc = dev["value"].permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    assert not value_nc.is_contiguous()
    out = sdk.multi_scale_deformable_attn(value_nc, dev["shapes"], dev["starts"], dev["loc"],
                                          dev["attn"])
    parity.assert_close("output", out, parity.oracle_all(inp)[0], 1e-4)


FULL_SIZE = [
    ("deformable_detr", torch.float32),
    ("bevformer_sca", torch.float32),
    ("bevformer_sca", torch.bfloat16),
    ("bevformer_tsa", torch.float32),
    ("bevformer_tsa", torch.bfloat16),
    ("stress_d128", torch.bfloat16),
]
# grad_sampling_loc samples that may be left out of the comparison because they sit on a
# cell boundary (see parity.KINK_EPS): at most this fraction of all samples.
MAX_KINK_FRACTION = 1e-3


@pytest.mark.parametrize("name,dtype", FULL_SIZE, ids=[f"{n}-{str(d)[6:]}" for n, d in FULL_SIZE])
def test_full_size_whole_tensor_parity(name, dtype):
    """Every element of output, grad_value, grad_sampling_loc and grad_attn_weight at the
    full benchmark sizes (stress at its full batch of 8) against the float64 oracle, as the
    reference's test compares whole tensors
    (tests/torch/test_multi_scale_deformable_attn.py:93-101, 256-264). The device runs the
    whole batch in one call; the oracle is run one batch entry at a time (entries are
    independent) to bound host memory. Plus two size-independent identities on the full
    result: linearity in value and <grad_out, out> == <grad_value, value>."""
    import drivingsdk_b200 as sdk
    from oracle import msda_oracle
    w = workloads.WORKLOADS[name]
    inp = workloads.make_inputs(w, dtype)
    dev = parity.to_device(inp, dtype)
    out, gv, gl, ga = parity.run_python_api(dev)
    tol = parity.TOL[dtype]
    rounded = (lambda a: a) if dtype == torch.float32 else \
        (lambda a: torch.from_numpy(a).to(dtype).double().numpy())
    masked = 0
    for b in range(w.B):
        one = {k: (inp[k][b:b + 1] if k not in ("shapes", "starts") else inp[k]) for k in inp}
        want = [rounded(x) for x in parity.oracle_all(one)]
        dist = msda_oracle.kink_distance(one["shapes"].numpy(), one["loc"].numpy())
        smooth = dist > parity.KINK_EPS[dtype]
        masked += int((~smooth).sum())
        parity.assert_close(f"output[{b}]", out[b:b + 1], want[0], tol)
        parity.assert_close(f"grad_value[{b}]", gv[b:b + 1], want[1], tol)
        parity.assert_close(f"grad_attn_weight[{b}]", ga[b:b + 1], want[3], tol)
        parity.assert_close(f"grad_sampling_loc[{b}]", gl[b:b + 1], want[2], tol,
                            mask=np.broadcast_to(smooth[..., None], want[2].shape))
    nsamples = w.B * w.Q * w.H * w.L * w.P
    assert masked <= MAX_KINK_FRACTION * nsamples, (masked, nsamples)

    out2 = sdk.multi_scale_deformable_attn(dev["value"] * 2, dev["shapes"], dev["starts"],
                                           dev["loc"], dev["attn"])
    torch.testing.assert_close(out2.double(), 2 * out.double(), rtol=tol, atol=tol)
    lhs = (dev["grad_out"].double() * out.double()).sum().item()
    rhs = (gv.double() * dev["value"].double()).sum().item()
    scale = (dev["grad_out"].double().abs() * out.double().abs()).sum().item()
    rel = 2e-3 if dtype != torch.float32 else 1e-5
    assert abs(lhs - rhs) <= rel * scale, (lhs, rhs, scale)


def test_repeat_runs_agree():
    """Atomic accumulation order varies between runs; results must agree within tolerance
    and the forward must be bit-identical."""
    w = workloads.WORKLOADS["toy"]
    inp = workloads.make_inputs(w, torch.float32)
    dev = parity.to_device(inp, torch.float32)
    a = parity.run_python_api(dev)
    b = parity.run_python_api(dev)
    assert torch.equal(a[0], b[0])
    torch.testing.assert_close(a[1], b[1], rtol=1e-4, atol=1e-5)
    assert torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])


def test_mmcv_hook_end_to_end():
    """A stand-in for mmcv's autograd function, patched by the hook, called the way mmcv
    models call it (six arguments), forward and backward, against the oracle."""
    import sys
    import types
    from drivingsdk_b200.patcher import MSDA, Patcher, PatchStatus

    class MultiScaleDeformableAttnFunction(torch.autograd.Function):
        @staticmethod
        def forward(ctx, value, shapes, starts, loc, attn, im2col_step):
            raise AssertionError("the stock implementation must have been replaced")

        @staticmethod
        def backward(ctx, grad_output):
            raise AssertionError("the stock implementation must have been replaced")

    root, ops = types.ModuleType("mmcv"), types.ModuleType("mmcv.ops")
    mod = types.ModuleType("mmcv.ops.multi_scale_deform_attn")
    mod.MultiScaleDeformableAttnFunction = MultiScaleDeformableAttnFunction
    root.ops, ops.multi_scale_deform_attn = ops, mod
    names = ("mmcv", "mmcv.ops", "mmcv.ops.multi_scale_deform_attn")
    saved = {k: sys.modules.get(k) for k in names}
    sys.modules.update(dict(zip(names, (root, ops, mod))))
    try:
        p = Patcher().add(MSDA)
        p.apply()
        assert [r.status for r in p.results] == [PatchStatus.APPLIED] * 2
        w = workloads.WORKLOADS["toy"].with_queries(128)
        inp = workloads.make_inputs(w, torch.float32)
        dev = parity.to_device(inp, torch.float32)
        value = dev["value"].clone().requires_grad_(True)
        loc = dev["loc"].clone().requires_grad_(True)
        attn = dev["attn"].clone().requires_grad_(True)
        out = mod.MultiScaleDeformableAttnFunction.apply(value, dev["shapes"], dev["starts"],
                                                         loc, attn, 64)
        out.backward(dev["grad_out"])
        parity.compare_all(inp, (out.detach(), value.grad, loc.grad, attn.grad), torch.float32)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_staging_wait_that_runs_out_falls_back_to_direct_loads(dtype):
    """The only device-side wait of the MSDA kernels is the bounded poll of a staging barrier.
    With the poll limit set to 0 every wait runs out at once (nothing faults, nothing hangs):
    the kernels must report it in the status word (bit 0), let the copies already issued land,
    and still produce results within tolerance through their direct-load path."""
    from drivingsdk_b200 import capi
    lib = capi.load()
    assert lib.msda_sm100_device_status(1) >= 0
    w = workloads.WORKLOADS["toy"]
    inp = workloads.make_inputs(w, dtype)
    dev = parity.to_device(inp, dtype)
    prev = lib.msda_sm100_tune(capi.TUNE_SPIN_LIMIT, 0)
    prev_stage = lib.msda_sm100_tune(capi.TUNE_STAGE, 1)      # staging in both directions
    try:
        B, K, H, D = dev["value"].shape
        _, Q, _, L, P, _ = dev["loc"].shape
        out = torch.empty(B, Q, H * D, device="cuda", dtype=dtype)
        shapes = dev["shapes"].to(torch.int32).contiguous()
        starts = dev["starts"].to(torch.int32).contiguous()
        rc = lib.msda_sm100_forward(dev["value"].data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                    dev["loc"].data_ptr(), dev["attn"].data_ptr(), out.data_ptr(),
                                    B, K, H, D, L, Q, P, capi.dtype_code(dtype),
                                    torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        forward_status = lib.msda_sm100_device_status(1)      # the forward kernel alone
        results = parity.run_c_abi(dev, dtype)
        status = lib.msda_sm100_device_status(1)
    finally:
        lib.msda_sm100_tune(capi.TUNE_SPIN_LIMIT, prev)
        lib.msda_sm100_tune(capi.TUNE_STAGE, prev_stage)
    assert forward_status >= 0 and (forward_status & 1) == 1, forward_status
    assert status >= 0 and (status & 1) == 1, status
    parity.compare_all(inp, results, dtype)
    # with the limit restored the same call completes without the bit
    parity.compare_all(inp, parity.run_c_abi(dev, dtype), dtype)
    assert lib.msda_sm100_device_status(1) == 0


@pytest.mark.parametrize("amp", [0, 8, 1000000])
def test_backward_precision_threshold_does_not_change_results_beyond_tolerance(amp):
    """fp32 backward: samples above the amplification threshold accumulate their dot products
    in double. Everything in double (0), the default (8) and nothing in double (a huge
    threshold) must all meet the tolerance on the toy configuration (its levels are at most
    32 pixels wide, where fp32 dot products are accurate enough)."""
    from drivingsdk_b200 import capi
    lib = capi.load()
    w = workloads.WORKLOADS["toy"]
    inp = workloads.make_inputs(w, torch.float32)
    dev = parity.to_device(inp, torch.float32)
    prev = lib.msda_sm100_tune(capi.TUNE_PRECISE_AMP, amp)
    try:
        parity.compare_all(inp, parity.run_c_abi(dev, torch.float32), torch.float32)
    finally:
        lib.msda_sm100_tune(capi.TUNE_PRECISE_AMP, prev)


def test_bad_level_table_on_the_device_is_reported_not_followed():
    """Level tables passed as device memory cannot be checked by the host without a
    synchronisation; the kernels check them themselves and, when a level would reach past
    the K rows of value, set status bit 2 (value 4) and return without reading or adding
    anything out of bounds (forward and backward)."""
    from drivingsdk_b200 import capi
    lib = capi.load()
    lib.msda_sm100_device_status(1)
    w = workloads.WORKLOADS["toy"].with_queries(64)
    inp = workloads.make_inputs(w, torch.float32)
    dev = parity.to_device(inp, torch.float32)
    dev["starts"] = dev["starts"].clone()
    dev["starts"][-1] += 100            # last level now ends 100 rows past K
    B, K, H, D = dev["value"].shape
    _, Q, _, L, P, _ = dev["loc"].shape
    gv = torch.full_like(dev["value"], 7.0)
    gl, ga = torch.empty_like(dev["loc"]), torch.empty_like(dev["attn"])
    shapes = dev["shapes"].to(torch.int32).contiguous()
    starts = dev["starts"].to(torch.int32).contiguous()
    rc = lib.msda_sm100_backward(dev["value"].data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                 dev["loc"].data_ptr(), dev["attn"].data_ptr(),
                                 dev["grad_out"].data_ptr(), gv.data_ptr(), gl.data_ptr(),
                                 ga.data_ptr(), B, K, H, D, L, Q, P, capi.F32,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    status = lib.msda_sm100_device_status(1)
    assert status >= 0 and (status & 4) == 4, status
    assert torch.count_nonzero(gv).item() == 0     # zero-filled, then left alone
    out = torch.full((B, Q, H * D), 3.0, device="cuda")
    rc = lib.msda_sm100_forward(dev["value"].data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                dev["loc"].data_ptr(), dev["attn"].data_ptr(), out.data_ptr(),
                                B, K, H, D, L, Q, P, capi.F32,
                                torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert (lib.msda_sm100_device_status(1) & 4) == 4
    assert bool((out == 3.0).all())                # nothing was written


def test_status_checks_turn_a_refused_launch_into_an_exception():
    """With set_status_checks(True) the torch operators read the device status after every
    call: a level table in device memory that reaches past value's rows then raises instead
    of returning an untouched output; with the switch off (the default, no synchronisation)
    the same call returns and the status word carries the bit."""
    import drivingsdk_b200 as sdk
    w = workloads.WORKLOADS["toy"].with_queries(64)
    inp = workloads.make_inputs(w, torch.float32)
    dev = parity.to_device(inp, torch.float32)
    bad = dev["starts"].clone()
    bad[-1] += 100
    sdk.device_status(True)
    prev = sdk.set_status_checks(True)
    try:
        with pytest.raises(RuntimeError, match="device status"):
            sdk.multi_scale_deformable_attn(dev["value"], dev["shapes"], bad, dev["loc"],
                                            dev["attn"])
        assert sdk.device_status(True) == 0          # the failed check cleared it
        good = sdk.multi_scale_deformable_attn(dev["value"], dev["shapes"], dev["starts"],
                                               dev["loc"], dev["attn"])
    finally:
        sdk.set_status_checks(prev)
    assert not prev
    sdk.multi_scale_deformable_attn(dev["value"], dev["shapes"], bad, dev["loc"], dev["attn"])
    assert sdk.device_status(True) & 4
    again = sdk.multi_scale_deformable_attn(dev["value"], dev["shapes"], dev["starts"],
                                            dev["loc"], dev["attn"])
    assert torch.equal(good, again)


@pytest.mark.parametrize("name", ["toy", "bevformer_sca", "stress_d128"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_forward_with_and_without_packed_records(name, dtype):
    """The forward kernels keep records only for the corners that exist (default) or one per
    (sample, corner) (MSDA_TUNE_PACK_ROWS = 0): both forms must agree with the oracle, with one
    task per warp pass (BEVFormer) and with several (toy, stress)."""
    from drivingsdk_b200 import capi
    lib = capi.load()
    w = workloads.WORKLOADS[name].with_batch(1)
    w = w.with_queries(min(w.Q, 700))
    inp = workloads.make_inputs(w, dtype)
    dev = parity.to_device(inp, dtype)
    prev = lib.msda_sm100_tune(capi.TUNE_PACK_ROWS, 0)
    try:
        assert prev == 1
        plain = parity.run_c_abi(dev, dtype)
        parity.compare_all(inp, plain, dtype)
    finally:
        lib.msda_sm100_tune(capi.TUNE_PACK_ROWS, prev)
    packed = parity.run_c_abi(dev, dtype)
    parity.compare_all(inp, packed, dtype)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(packed[0].float(), plain[0].float(), rtol=tol, atol=tol)

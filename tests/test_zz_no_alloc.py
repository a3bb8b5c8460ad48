"""The allocation-free backward entry point (msda_sm100_backward_static), through the C ABI.

For hosts that cannot give the operator a workspace — all device memory already handed to
their own arena, or no allocator call allowed where the operator runs — the library keeps
the fp32 accumulation scratch in a static device array. This file checks that the entry
point gives what the workspace entry point gives, twice in a row on different inputs (the
array is shared between calls and must be cleared by each), and that it refuses problems
larger than the array. It sorts last on purpose: a run that stops at the first failure has
by then run every other test.
"""
import pytest
import torch

from drivingsdk_b200 import capi, workloads
from tests import parity

pytestmark = pytest.mark.gpu


def _call_static(dev, dtype):
    lib = capi.load()
    value, loc, attn, go = dev["value"], dev["loc"], dev["attn"], dev["grad_out"]
    B, K, H, D = value.shape
    _, Q, _, L, P, _ = loc.shape
    shapes = dev["shapes"].to(torch.int32).contiguous()
    starts = dev["starts"].to(torch.int32).contiguous()
    gv, gl, ga = torch.empty_like(value), torch.empty_like(loc), torch.empty_like(attn)
    rc = lib.msda_sm100_backward_static(
        value.data_ptr(), shapes.data_ptr(), starts.data_ptr(), loc.data_ptr(), attn.data_ptr(),
        go.data_ptr(), gv.data_ptr(), gl.data_ptr(), ga.data_ptr(), B, K, H, D, L, Q, P,
        capi.dtype_code(dtype), torch.cuda.current_stream().cuda_stream)
    capi.check(rc, "backward_static")
    torch.cuda.synchronize()
    return gv, gl, ga


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_static_scratch_matches_workspace_entry_point_twice(dtype):
    tol = parity.TOL[dtype]
    # second call: other values AND a smaller problem, so stale sums from the first call
    # would show up if the used part of the array were not cleared
    for seed_offset, queries in ((0, 400), (1, 150)):
        w = workloads.WORKLOADS["toy"].with_queries(queries)
        inp = workloads.make_inputs(w, dtype, seed_offset=seed_offset)
        dev = parity.to_device(inp, dtype)
        _, want_gv, want_gl, want_ga = parity.run_c_abi(dev, dtype, workspace=True)
        gv, gl, ga = _call_static(dev, dtype)
        torch.testing.assert_close(gv.float(), want_gv.float(), rtol=tol, atol=tol)
        # these two do not depend on accumulation order: bit-identical
        assert torch.equal(gl, want_gl) and torch.equal(ga, want_ga)
        # and against the oracle, at the tolerance of the other parity tests
        want = parity.oracle_all(inp)
        if dtype != torch.float32:
            want = tuple(torch.from_numpy(x).to(dtype).double().numpy() for x in want)
        parity.assert_close("grad_value", gv, want[1], tol)


def test_static_scratch_refuses_oversized_problems():
    lib = capi.load()
    limit = lib.msda_sm100_static_scratch_bytes()
    assert limit == 32 * 1024 * 1024
    one = 256  # any non-null value: the size check comes before the pointers are touched
    B, K, H, D = 2, 30825, 8, 32            # 4 * B*K*H*D = 63 MB > 32 MiB
    assert 4 * B * K * H * D > limit
    rc = lib.msda_sm100_backward_static(one, one, one, one, one, one, one, one, one,
                                        B, K, H, D, 4, 10, 8, capi.BF16, None)
    assert rc == -6
    assert b"workspace" in lib.msda_sm100_strerror(rc)


def test_static_scratch_refuses_unknown_dtype_before_anything_else():
    """An unknown dtype code is reported as such for small and for oversized problems alike."""
    lib = capi.load()
    one = 256
    for dims in ((1, 100, 2, 32), (2, 30825, 8, 32)):
        rc = lib.msda_sm100_backward_static(one, one, one, one, one, one, one, one, one,
                                            *dims, 4, 10, 8, 7, None)
        assert rc == -5, rc
        assert b"dtype" in lib.msda_sm100_strerror(rc)

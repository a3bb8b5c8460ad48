"""Seeded random shapes against the oracle (needs a GPU): odd level/point counts, several
tasks per warp pass with a ragged last pass, unaligned head dims, single queries, levels of
one pixel, locations far outside the image."""
import random

import numpy as np
import pytest
import torch

from drivingsdk_b200 import workloads
from tests import parity

pytestmark = pytest.mark.gpu


def _random_workload(rng):
    L = rng.choice([1, 1, 2, 3, 4, 5, 8])
    P = rng.choice([1, 2, 3, 4, 5, 7, 8, 16])
    while L * P > 64:
        P = max(1, P // 2)
    levels = tuple((rng.randint(1, 12), rng.randint(1, 12)) for _ in range(L))
    D = rng.choice([4, 8, 12, 16, 24, 32, 37, 40, 64, 96, 128, 147, 256])
    H = rng.choice([1, 2, 3, 5, 8])
    B = rng.choice([1, 2, 3])
    Q = rng.choice([1, 2, 7, 31, 33, 100, 257])
    lo = rng.choice([0.0, -0.1, -1.5])
    return workloads.Workload("fuzz", B, Q, H, D, levels, P, (lo, 1.0 - lo), rng.randint(0, 10**6))


@pytest.mark.parametrize("index", range(36))
def test_random_shapes(index):
    rng = random.Random(1000 + index)
    w = _random_workload(rng)
    dtype = rng.choice([torch.float32, torch.float32, torch.float16, torch.bfloat16])
    inp = workloads.make_inputs(w, dtype)
    dev = parity.to_device(inp, dtype)
    stage = index % 2
    from drivingsdk_b200 import capi
    prev = capi.load().msda_sm100_tune(capi.TUNE_STAGE, stage)
    try:
        parity.compare_all(inp, parity.run_c_abi(dev, dtype, host_levels=bool(index % 3 == 0)), dtype)
        parity.compare_all(inp, parity.run_python_api(dev), dtype)
    finally:
        capi.load().msda_sm100_tune(capi.TUNE_STAGE, prev)
    assert capi.load().msda_sm100_device_status(1) == 0


@pytest.mark.parametrize("index", range(36))
def test_random_shapes_in_the_bounds_checking_build(index):
    """The same seeded shapes through the library compiled with -DMSDA_DEBUG_BOUNDS, where
    every row offset (and every shared-memory accumulator address) is checked before it is
    used: results must agree with the oracle and no check may have fired (status 0). This is
    what stands in for a memory checker."""
    from drivingsdk_b200 import capi
    dbg = capi.load_debug()
    assert dbg.msda_sm100_debug_bounds() == 1
    rng = random.Random(1000 + index)
    w = _random_workload(rng)
    dtype = rng.choice([torch.float32, torch.float32, torch.float16, torch.bfloat16])
    inp = workloads.make_inputs(w, dtype)
    dev = parity.to_device(inp, dtype)
    dbg.msda_sm100_device_status(1)
    parity.compare_all(inp, parity.run_c_abi(dev, dtype, host_levels=bool(index % 3 == 0), lib=dbg),
                       dtype)
    # small resident area: window edges inside the small maps
    prev = dbg.msda_sm100_tune(capi.TUNE_RESIDENT_BYTES, 4096)
    try:
        parity.compare_all(inp, parity.run_c_abi(dev, dtype, lib=dbg), dtype)
    finally:
        dbg.msda_sm100_tune(capi.TUNE_RESIDENT_BYTES, prev)
    assert dbg.msda_sm100_device_status(1) == 0


def test_bounds_checking_build_catches_a_level_that_reaches_past_value():
    """A level table in device memory whose last level ends past the K rows of value: the
    bounds-checking build's forward kernel must flag it (status bit 4, value 16) and skip the
    rows instead of reading them."""
    from drivingsdk_b200 import capi
    dbg = capi.load_debug()
    dbg.msda_sm100_device_status(1)
    w = workloads.Workload("oob", 1, 64, 2, 32, ((6, 6), (3, 3)), 4, (0.0, 1.0), 3)
    inp = workloads.make_inputs(w, torch.float32)
    dev = parity.to_device(inp, torch.float32)
    shapes = dev["shapes"].to(torch.int32).contiguous()
    starts = dev["starts"].to(torch.int32).clone()
    starts[-1] += 40                      # the 3x3 level now starts 4 rows before the end of value
    B, K, H, D = dev["value"].shape
    _, Q, _, L, P, _ = dev["loc"].shape
    out = torch.empty(B, Q, H * D, device="cuda")
    rc = dbg.msda_sm100_forward(dev["value"].data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                dev["loc"].data_ptr(), dev["attn"].data_ptr(), out.data_ptr(),
                                B, K, H, D, L, Q, P, capi.F32,
                                torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    status = dbg.msda_sm100_device_status(1)
    assert status >= 0 and (status & 16) == 16, status
    assert torch.isfinite(out).all()

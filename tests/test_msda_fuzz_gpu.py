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
    stage = index % 3      # 0 no staging, 1 both directions, 2 backward only (the default)
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
    every row offset is checked before it is used: results must agree with the oracle and no check may have fired (status 0). This is
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
    parity.compare_all(inp, parity.run_c_abi(dev, dtype, workspace=False, lib=dbg), dtype) \
        if dtype == torch.float32 else None
    assert dbg.msda_sm100_device_status(1) == 0


def test_bounds_checks_fire_when_the_tensor_is_declared_shorter_than_it_is():
    """The checks of the bounds-checking build must actually fire. Its test hook makes them
    behave as if value / grad_value ended after 100 (key, head) rows of the toy problem's
    10880: every row beyond is then "out of bounds" — flagged (status bit 4, value 16) and
    skipped, never read or added to, in forward and backward."""
    from drivingsdk_b200 import capi
    dbg = capi.load_debug()
    dbg.msda_sm100_device_status(1)
    w = workloads.WORKLOADS["toy"].with_queries(64)
    inp = workloads.make_inputs(w, torch.float32)
    dev = parity.to_device(inp, torch.float32)
    prev = dbg.msda_sm100_tune(capi.TUNE_DEBUG_ROW_LIMIT, 100)
    try:
        out, gv, gl, ga = parity.run_c_abi(dev, torch.float32, lib=dbg)
        status = dbg.msda_sm100_device_status(1)
    finally:
        dbg.msda_sm100_tune(capi.TUNE_DEBUG_ROW_LIMIT, prev)
    assert status >= 0 and (status & 16) == 16, status
    assert torch.isfinite(out).all() and torch.isfinite(gv).all()
    # nothing was added beyond the pretended end of grad_value
    assert torch.count_nonzero(gv.reshape(-1, gv.shape[-1])[100:]).item() == 0
    # and with the hook off the same call is clean
    parity.compare_all(inp, parity.run_c_abi(dev, torch.float32, lib=dbg), torch.float32)
    assert dbg.msda_sm100_device_status(1) == 0

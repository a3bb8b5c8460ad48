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

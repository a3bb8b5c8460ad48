"""Pins the geometric-kernel-attention oracle against the reference's own golden outputs (CPU)."""
import os

import numpy as np
import pytest

from oracle import msda_oracle

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gka_golden.npz")
_Z = np.load(_PATH)
NAMES = sorted({k.split("/")[0] for k in _Z.files})


def case(name):
    return {k.split("/")[1]: _Z[k] for k in _Z.files if k.startswith(name + "/")}


@pytest.mark.parametrize("name", NAMES)
def test_gka_oracle_matches_reference_golden(name):
    c = case(name)
    out = msda_oracle.gka_forward(c["value"], c["shapes"], c["starts"], c["loc"], c["attn"])
    gv, ga = msda_oracle.gka_backward(c["value"], c["shapes"], c["starts"], c["loc"], c["attn"],
                                      c["grad_out"])
    np.testing.assert_allclose(out, c["out"], rtol=1e-11, atol=1e-11)
    np.testing.assert_allclose(gv, c["grad_value"], rtol=1e-11, atol=1e-11)
    np.testing.assert_allclose(ga, c["grad_attn"], rtol=1e-11, atol=1e-11)


def test_locations_outside_the_level_are_clamped():
    """The reference draws coordinates from -3 to size+2 (tests/torch/
    test_geometric_kernel_attention.py:27-33); all of them must land on border pixels."""
    shapes = np.array([[2, 3]], dtype=np.int32)
    starts = np.array([0], dtype=np.int32)
    value = np.arange(6, dtype=np.float32).reshape(1, 6, 1, 1)
    loc = np.array([[-3, -3], [5, 7], [1, 0], [2, 1]], dtype=np.float32).reshape(1, 1, 1, 1, 4, 2)
    attn = np.ones((1, 1, 1, 1, 4), dtype=np.float32)
    out = msda_oracle.gka_forward(value, shapes, starts, loc, attn)
    assert out.item() == 0 + 5 + 1 + 5    # pixels (0,0), (y=1,x=2), (y=0,x=1), (y=1,x=2)

"""Pins the CPU oracles against the reference's own golden outputs (CPU only)."""
import numpy as np
import pytest
import torch

from oracle import golden_torch, msda_oracle
from tests.golden_cases import CASES, NAMES


@pytest.mark.parametrize("name", NAMES)
def test_c_oracle_matches_reference_golden(name):
    c = CASES[name]
    out = msda_oracle.forward(c["value"], c["shapes"], c["starts"], c["loc"], c["attn"])
    gv, gl, ga = msda_oracle.backward(c["value"], c["shapes"], c["starts"], c["loc"], c["attn"],
                                      c["grad_out"])
    # both sides are float64 evaluations of the same expression
    np.testing.assert_allclose(out, c["out"], rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(gv, c["grad_value"], rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(ga, c["grad_attn"], rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(gl, c["grad_loc"], rtol=1e-10, atol=1e-11)


@pytest.mark.parametrize("name", NAMES)
def test_torch_port_matches_reference_golden(name):
    c = CASES[name]
    t = lambda k: torch.from_numpy(c[k]).double()
    out, gv, gl, ga = golden_torch.msda_forward_backward(
        t("value"), torch.from_numpy(c["shapes"]).long(), t("loc"), t("attn"), t("grad_out"))
    np.testing.assert_allclose(out.numpy(), c["out"], rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(gv.numpy(), c["grad_value"], rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(ga.numpy(), c["grad_attn"], rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(gl.numpy(), c["grad_loc"], rtol=1e-10, atol=1e-11)


def test_oracle_threads_agree():
    c = CASES["toy_slice"]
    msda_oracle.set_threads(1)
    a = msda_oracle.backward(c["value"], c["shapes"], c["starts"], c["loc"], c["attn"], c["grad_out"])
    msda_oracle.set_threads(4)
    b = msda_oracle.backward(c["value"], c["shapes"], c["starts"], c["loc"], c["attn"], c["grad_out"])
    msda_oracle.set_threads(1)
    for x, y in zip(a, b):
        np.testing.assert_array_equal(x, y)


@pytest.mark.parametrize("fill", [float("nan"), float("inf")])
def test_oracle_nonfinite_inputs_give_zeros(fill):
    """All-NaN / all-Inf operands must produce exact zeros everywhere
    (tests/torch/test_multi_scale_deformable_attn.py:266-282)."""
    c = CASES["tiny_border"]
    full = lambda k: np.full_like(c[k], fill)
    out = msda_oracle.forward(full("value"), c["shapes"], c["starts"], full("loc"), full("attn"))
    gv, gl, ga = msda_oracle.backward(full("value"), c["shapes"], c["starts"], full("loc"),
                                      full("attn"), full("grad_out"))
    for arr in (out, gv, gl, ga):
        assert np.count_nonzero(arr) == 0 and np.isfinite(arr).all()


def test_kink_distance_flags_boundaries():
    shapes = np.array([[4, 4]], dtype=np.int32)
    loc = np.zeros((1, 1, 1, 1, 2, 2), dtype=np.float32)
    loc[0, 0, 0, 0, 0] = (0.375, 0.375)   # x = y = 1.0: exactly on a cell boundary
    loc[0, 0, 0, 0, 1] = (0.5, 0.5)       # x = y = 1.5: cell centre
    d = msda_oracle.kink_distance(shapes, loc)
    assert d[0, 0, 0, 0, 0] == 0.0 and abs(d[0, 0, 0, 0, 1] - 0.5) < 1e-12

"""The deformable-convolution oracle against the committed golden (torchvision's CPU operator
with autograd, tests/golden/make_dcn_golden.py), forward and every gradient."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import dcn_oracle  # noqa: E402

GOLDEN = np.load(os.path.join(ROOT, "tests", "golden", "dcn_golden.npz"))
CASES = sorted({k.split("/")[0] for k in GOLDEN.files})


def load_case(name):
    get = lambda key: GOLDEN[f"{name}/{key}"] if f"{name}/{key}" in GOLDEN.files else None
    N, C, Co, H, W, k, s, p, d, g, dg, modulated, with_bias = (int(v) for v in get("cfg"))
    conv = dict(stride=s, padding=p, dilation=d, groups=g, deform_groups=dg)
    return get, conv


def test_cases_cover_the_variants():
    assert len(CASES) >= 7
    cfgs = np.stack([GOLDEN[f"{n}/cfg"] for n in CASES])
    assert set(cfgs[:, 11]) == {0, 1} and set(cfgs[:, 12]) == {0, 1}   # modulated, bias
    assert cfgs[:, 9].max() > 1 and cfgs[:, 10].max() > 1               # groups, deform groups
    assert cfgs[:, 6].max() > 1 and cfgs[:, 8].max() > 1                # stride, dilation


@pytest.mark.parametrize("name", CASES)
def test_forward_matches_golden(name):
    get, conv = load_case(name)
    out = dcn_oracle.forward(get("x"), get("offset"), get("mask"), get("weight"), get("bias"), **conv)
    np.testing.assert_allclose(out, get("out"), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", CASES)
def test_backward_matches_golden(name):
    get, conv = load_case(name)
    gx, goff, gmask, gw, gb = dcn_oracle.backward(get("x"), get("offset"), get("mask"),
                                                  get("weight"), get("grad_out"), **conv)
    np.testing.assert_allclose(gx, get("grad_x"), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(goff, get("grad_offset"), rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(gw, get("grad_weight"), rtol=1e-5, atol=2e-5)
    if get("mask") is not None:
        np.testing.assert_allclose(gmask, get("grad_mask"), rtol=1e-5, atol=1e-5)
    else:
        assert gmask is None
    if get("bias") is not None:
        np.testing.assert_allclose(gb, get("grad_bias"), rtol=1e-5, atol=1e-5)


def test_samples_outside_the_image_contribute_nothing():
    x = np.ones((1, 2, 4, 4), np.float32)
    w = np.ones((1, 2, 1, 1), np.float32)
    off = np.zeros((1, 2, 4, 4), np.float32)
    off[0, 0] = 100.0    # every dy far outside
    assert np.all(dcn_oracle.forward(x, off, None, w) == 0)
    gx, goff, _, gw, _ = dcn_oracle.backward(x, off, None, w, np.ones((1, 1, 4, 4), np.float32))
    assert np.all(gx == 0) and np.all(goff == 0) and np.all(gw == 0)
    off[0, 0] = -1.0     # exactly -1 for the first row: still outside (strict inequality)
    assert np.all(dcn_oracle.forward(x, off, None, w)[0, 0, 0] == 0)

"""Pins the deformable-aggregation oracle: forward against the reference's numpy golden
(fixtures), backward against autograd of an independent PyTorch restatement (CPU)."""
import os

import numpy as np
import pytest
import torch

from oracle import golden_torch, msda_oracle

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "da_golden.npz")
_Z = np.load(_PATH)
NAMES = sorted({k.split("/")[0] for k in _Z.files})


def case(name):
    return {k.split("/")[1]: _Z[k] for k in _Z.files if k.startswith(name + "/")}


@pytest.mark.parametrize("name", NAMES)
def test_forward_matches_reference_golden(name):
    c = case(name)
    out = msda_oracle.da_forward(c["feat"], c["shapes"], c["starts"], c["loc"], c["wts"])
    # the reference golden accumulates in float32: compare at float32 resolution
    np.testing.assert_allclose(out, c["out"], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("name", NAMES)
def test_oracle_agrees_with_torch_restatement(name):
    c = case(name)
    t = lambda k: torch.from_numpy(c[k]).double()
    feat, loc, wts = t("feat").requires_grad_(), t("loc").requires_grad_(), t("wts").requires_grad_()
    out = golden_torch.da_forward(feat, torch.from_numpy(c["shapes"]), torch.from_numpy(c["starts"]),
                                  loc, wts)
    out.backward(t("grad_out"))
    want_out = msda_oracle.da_forward(c["feat"], c["shapes"], c["starts"], c["loc"], c["wts"])
    gf, gl, gw = msda_oracle.da_backward(c["feat"], c["shapes"], c["starts"], c["loc"], c["wts"],
                                         c["grad_out"])
    np.testing.assert_allclose(out.detach().numpy(), want_out, rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(feat.grad.numpy(), gf, rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(wts.grad.numpy(), gw, rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(loc.grad.numpy(), gl, rtol=1e-9, atol=1e-10)

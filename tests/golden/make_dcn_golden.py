"""Generates tests/golden/dcn_golden.npz: deformable and modulated deformable convolution,
forward and all gradients, computed by torchvision.ops.deform_conv2d on CPU with autograd.

The reference pins its operator against mmcv's CPU implementation
(tests/torch/test_deformable_conv2d.py:24-37); mmcv is not installed here, torchvision's
operator implements the same published algorithm with the same tensor conventions (NCHW,
offset channels ordered (deformable group, tap, (dy, dx)), mask channels (deformable group,
tap)) and stands in for it. Cases are seeded draws in the reference tests' value ranges
(x and offsets in [-5, 5], weights in [-0.05, 0.05], tests/torch/test_deformable_conv2d.py:60-64)
at small sizes; several have offsets that leave the image.
"""
import os

import numpy as np
import torch
from torchvision.ops import deform_conv2d

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dcn_golden.npz")

# name: (N, C, Co, H, W, k, stride, padding, dilation, groups, deform_groups, modulated, bias)
CASES = {
    "plain_3x3": (2, 8, 8, 7, 9, 3, 1, 1, 1, 1, 1, False, False),
    "modulated_3x3": (2, 8, 16, 7, 9, 3, 1, 1, 1, 1, 1, True, False),
    "groups2_dg2_bias": (1, 16, 8, 6, 5, 3, 1, 1, 1, 2, 2, True, True),
    "stride2_dil2_pad2": (2, 4, 6, 9, 10, 3, 2, 2, 2, 1, 1, False, False),
    "k1_pad0": (1, 12, 4, 5, 6, 1, 1, 0, 1, 1, 1, True, False),
    "k5_groups4": (1, 8, 8, 8, 8, 5, 1, 2, 1, 4, 1, False, True),
    "c64_dg4": (1, 64, 32, 5, 7, 3, 1, 1, 1, 1, 4, True, False),
}


def out_size(size, k, s, p, d):
    return (size + 2 * p - (d * (k - 1) + 1)) // s + 1


def main():
    blobs = {}
    for idx, (name, cfg) in enumerate(CASES.items()):
        N, C, Co, H, W, k, s, p, d, g, dg, modulated, with_bias = cfg
        gen = torch.Generator().manual_seed(1000 + idx)
        Ho, Wo = out_size(H, k, s, p, d), out_size(W, k, s, p, d)
        u = lambda *shape: torch.rand(*shape, generator=gen, dtype=torch.float64) * 10 - 5
        x = u(N, C, H, W).float()
        offset = u(N, dg * 2 * k * k, Ho, Wo).float()
        weight = (u(Co, C // g, k, k) * 0.01).float()
        mask = u(N, dg * k * k, Ho, Wo).float() if modulated else None
        bias = u(Co).float() if with_bias else None
        grad_out = u(N, Co, Ho, Wo).float()
        leaves = [t.double().requires_grad_() if t is not None else None
                  for t in (x, offset, weight, mask, bias)]
        xd, od, wd, md, bd = leaves
        out = deform_conv2d(xd, od, wd, bd, stride=s, padding=p, dilation=d, mask=md)
        out.backward(grad_out.double())
        blobs[f"{name}/cfg"] = np.array([N, C, Co, H, W, k, s, p, d, g, dg, int(modulated),
                                         int(with_bias)])
        for key, t in (("x", x), ("offset", offset), ("weight", weight), ("mask", mask),
                       ("bias", bias), ("grad_out", grad_out)):
            if t is not None:
                blobs[f"{name}/{key}"] = t.numpy()
        blobs[f"{name}/out"] = out.detach().float().numpy()
        for key, t in (("grad_x", xd), ("grad_offset", od), ("grad_weight", wd),
                       ("grad_mask", md), ("grad_bias", bd)):
            if t is not None:
                blobs[f"{name}/{key}"] = t.grad.float().numpy()
    np.savez_compressed(OUT, **blobs)
    print(OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()

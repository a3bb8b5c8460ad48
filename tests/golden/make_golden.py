"""Generates tests/golden/msda_golden.npz from the REFERENCE's own golden functions.

Run where the reference checkout is available, with MSDA_REFERENCE_ROOT set to its
directory. It imports the reference's unit-test module
tests/torch/test_multi_scale_deformable_attn.py unchanged — with `torch_npu`
and `mx_driving` stubbed, because only the two pure-PyTorch golden functions
are used — and records their float64 results on seeded inputs:

    multi_scale_deformable_attn_pytorch       (:34-64)
    multi_scale_deformable_attn_pytorch_grad  (:67-76)
    cpu_gen_inputs                            (:14-31)   (one case, its own distribution)

The cache decorator is bypassed through ``__wrapped__`` (tests/torch/data_cache.py:110).
The committed .npz is what the oracle is pinned against where no reference
checkout exists.
"""
import os
import sys
import types
import unittest

import numpy as np
import torch

REF = os.environ.get("MSDA_REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set MSDA_REFERENCE_ROOT to the directory of the reference checkout")
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "msda_golden.npz")

# name: (B, Q, H, D, levels[(h, w)], P, dtype, loc range, seed)
CASES = {
    "tiny_border": (1, 20, 2, 8, [(6, 5), (3, 2)], 3, "float32", (-0.1, 1.1), 11),
    "toy_slice": (1, 12, 8, 32, [(8, 8), (4, 4), (2, 2), (1, 1)], 4, "float32", (-0.1, 1.1), 12),
    "unaligned_d37": (2, 9, 4, 37, [(3, 4)] * 5, 3, "float32", (0.0, 1.0), 13),
    "points_lp63": (1, 6, 7, 12, [(4, 3)] * 3, 21, "float32", (0.0, 1.0), 14),
    "single_level_p8": (2, 10, 4, 32, [(7, 9)], 8, "float32", (-0.05, 1.05), 15),
    "d128_lp64": (1, 5, 2, 128, [(2, 3)] * 8, 8, "float32", (0.0, 1.0), 16),
    "fp16_inputs": (1, 12, 8, 32, [(4, 3)] * 4, 4, "float16", (0.0, 1.0), 17),
    "bf16_inputs": (1, 10, 8, 32, [(6, 7), (3, 4)], 8, "bfloat16", (-0.05, 1.05), 18),
    "one_pixel_levels": (1, 7, 3, 16, [(1, 1), (1, 3), (2, 1)], 2, "float32", (-0.3, 1.3), 19),
}


def load_reference_test_module():
    stub = types.ModuleType("torch_npu")
    testing = types.ModuleType("torch_npu.testing")
    testcase = types.ModuleType("torch_npu.testing.testcase")
    testcase.TestCase = unittest.TestCase
    testcase.run_tests = lambda: None
    stub.testing = testing
    testing.testcase = testcase
    sys.modules.setdefault("torch_npu", stub)
    sys.modules.setdefault("torch_npu.testing", testing)
    sys.modules.setdefault("torch_npu.testing.testcase", testcase)
    sys.modules.setdefault("mx_driving", types.ModuleType("mx_driving"))
    sys.path.insert(0, os.path.join(REF, "tests", "torch"))
    import test_multi_scale_deformable_attn as ref_test  # noqa: E402
    return ref_test


def make_inputs(B, Q, H, D, levels, P, dtype, loc_range, seed):
    g = torch.Generator().manual_seed(seed)
    shapes = torch.tensor(levels, dtype=torch.int64)
    sizes = shapes[:, 0] * shapes[:, 1]
    K = int(sizes.sum())
    starts = torch.cat([sizes.new_zeros(1), sizes.cumsum(0)[:-1]])
    L = len(levels)
    lo, hi = loc_range
    value = torch.randn(B, K, H, D, generator=g)
    loc = torch.rand(B, Q, H, L, P, 2, generator=g) * (hi - lo) + lo
    attn = torch.softmax(torch.randn(B, Q, H, L * P, generator=g), -1).reshape(B, Q, H, L, P)
    grad_out = torch.randn(B, Q, H * D, generator=g)
    dt = getattr(torch, dtype)
    # round to the dtype under test, keep float32 containers
    value, loc, attn, grad_out = (t.to(dt).float() for t in (value, loc, attn, grad_out))
    return shapes, starts, value, loc, attn, grad_out


def run_reference(ref_test, shapes, value, loc, attn, grad_out):
    fwd = ref_test.multi_scale_deformable_attn_pytorch.__wrapped__
    bwd = ref_test.multi_scale_deformable_attn_pytorch_grad.__wrapped__
    v = value.double().requires_grad_()
    s = loc.double().requires_grad_()
    a = attn.double().requires_grad_()
    out = fwd(v, shapes.long(), s, a)
    out64 = out.detach().numpy().copy()
    bwd(out, grad_out.double(), v, s, a)  # returns float32 copies; keep float64 grads instead
    return out64, v.grad.numpy(), s.grad.numpy(), a.grad.numpy()


def main():
    ref_test = load_reference_test_module()
    blob = {}
    for name, spec in CASES.items():
        shapes, starts, value, loc, attn, grad_out = make_inputs(*spec)
        out, gv, gl, ga = run_reference(ref_test, shapes, value, loc, attn, grad_out)
        blob.update({
            f"{name}/shapes": shapes.numpy().astype(np.int32),
            f"{name}/starts": starts.numpy().astype(np.int32),
            f"{name}/value": value.numpy(), f"{name}/loc": loc.numpy(),
            f"{name}/attn": attn.numpy(), f"{name}/grad_out": grad_out.numpy(),
            f"{name}/out": out, f"{name}/grad_value": gv,
            f"{name}/grad_loc": gl, f"{name}/grad_attn": ga,
            f"{name}/dtype": np.array(spec[6]),
        })
    # one case drawn by the reference's own generator (all levels 60x40, its distributions)
    torch.manual_seed(20)
    shapes, _, value, loc, attn, offset, grad_out = ref_test.cpu_gen_inputs.__wrapped__(
        [1, 6, 4, 1, 1, 2], torch.float32)
    out, gv, gl, ga = run_reference(ref_test, shapes, value, loc, attn, grad_out)
    name = "reference_generator"
    blob.update({
        f"{name}/shapes": shapes.numpy().astype(np.int32),
        f"{name}/starts": offset.numpy().astype(np.int32),
        f"{name}/value": value.numpy(), f"{name}/loc": loc.numpy(),
        f"{name}/attn": attn.numpy(), f"{name}/grad_out": grad_out.numpy(),
        f"{name}/out": out, f"{name}/grad_value": gv, f"{name}/grad_loc": gl,
        f"{name}/grad_attn": ga, f"{name}/dtype": np.array("float32"),
    })
    np.savez_compressed(OUT, **blob)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(CASES) + 1, "cases")


if __name__ == "__main__":
    main()

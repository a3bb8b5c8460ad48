"""Generates tests/golden/gka_golden.npz from the REFERENCE's own golden for geometric
kernel attention (tests/torch/test_geometric_kernel_attention.py): its input generator
`cpu_gen_inputs` (:20-41) and its CPU implementation `cpu_geometric_kernel_attention`
(:44-92) + autograd (:95-103), run in float64 on seeded draws. `torch_npu` and `mx_driving`
are stubbed (the module asks torch_npu for a device name at import); the cache decorator is
bypassed through ``__wrapped__``. Needs the reference checkout: set MSDA_REFERENCE_ROOT
to its directory.
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
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gka_golden.npz")

# [bs, num_queries, embed_dims, num_heads, num_levels, num_points] as in the reference test
# (:109-115), with fewer queries / batch entries so the fixture stays small (the reference's
# generator uses 6x10 levels for every batch size but 24).
SHAPES = {
    "levels_6x10_p15": [2, 20, 64, 4, 1, 15],
    "two_levels_d16": [2, 4, 16, 4, 2, 15],
    "d8_p3_l4": [2, 9, 8, 3, 4, 3],
    "d128_l2_p32": [1, 6, 128, 2, 2, 32],
}


def load_reference_test_module():
    stub = types.ModuleType("torch_npu")
    stub.npu = types.SimpleNamespace(get_device_name=lambda i: "stub-device-name")
    testing = types.ModuleType("torch_npu.testing")
    testcase = types.ModuleType("torch_npu.testing.testcase")
    testcase.TestCase = unittest.TestCase
    testcase.run_tests = lambda: None
    stub.testing, testing.testcase = testing, testcase
    sys.modules.setdefault("torch_npu", stub)
    sys.modules.setdefault("torch_npu.testing", testing)
    sys.modules.setdefault("torch_npu.testing.testcase", testcase)
    sys.modules.setdefault("mx_driving", types.ModuleType("mx_driving"))
    sys.path.insert(0, os.path.join(REF, "tests", "torch"))
    import test_geometric_kernel_attention as ref_test  # noqa: E402
    return ref_test


def main():
    ref = load_reference_test_module()
    blob = {}
    for i, (name, shape) in enumerate(SHAPES.items()):
        torch.manual_seed(100 + i)
        loc, shapes, value, attn, starts, grad_out = ref.cpu_gen_inputs.__wrapped__(shape)
        loc_int = loc.long()                       # what the reference test feeds both sides
        v = value.double().requires_grad_()
        a = attn.double().requires_grad_()
        out = ref.cpu_geometric_kernel_attention.__wrapped__(
            v, shapes.long(), starts.long(), loc_int.clone(), a)
        out.backward(grad_out.double())
        blob.update({
            f"{name}/shapes": shapes.numpy().astype(np.int32),
            f"{name}/starts": starts.numpy().astype(np.int32),
            f"{name}/value": value.numpy(), f"{name}/loc": loc_int.float().numpy(),
            f"{name}/attn": attn.numpy(), f"{name}/grad_out": grad_out.numpy(),
            f"{name}/out": out.detach().numpy(), f"{name}/grad_value": v.grad.numpy(),
            f"{name}/grad_attn": a.grad.numpy(),
        })
    np.savez_compressed(OUT, **blob)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(SHAPES), "cases")


if __name__ == "__main__":
    main()

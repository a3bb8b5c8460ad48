"""Generates tests/golden/da_golden.npz from the REFERENCE's numpy golden of deformable
aggregation (tests/torch/test_deformable_aggregation.py:33-125, a method of its TestCase; the
cache decorator is bypassed through ``__wrapped__``). Inputs are seeded draws with several
cameras and scales (the reference's own generator, :15-24, uses one camera and one 32x88
map); some locations lie outside (0, 1) to exercise the skip rule. Needs the reference
checkout: set MSDA_REFERENCE_ROOT to its directory.
"""
import os
import sys
import types
import unittest

import numpy as np

REF = os.environ.get("MSDA_REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set MSDA_REFERENCE_ROOT to the directory of the reference checkout")
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "da_golden.npz")

# name: (B, C, anchors, pts, G, maps[cam][scale] = (h, w))
CASES = {
    "one_cam_one_scale": (2, 32, 5, 7, 8, [[(8, 11)]]),
    "c32_g16_two_channels_per_group": (1, 32, 4, 3, 16, [[(6, 5)]]),
    "cams3_scales4_c64": (2, 64, 6, 5, 8, [[(8, 12), (4, 6), (2, 3), (1, 2)]] * 3),
    "cams2_scales3_c256": (1, 256, 3, 4, 8, [[(5, 7), (3, 4), (2, 2)], [(4, 4), (2, 3), (1, 1)]]),
    "scales5_c40": (1, 40, 4, 6, 8, [[(3, 3), (2, 5), (4, 2), (1, 1), (2, 2)]]),
}


def load_reference_test_class():
    stub = types.ModuleType("torch_npu")
    stub.npu = types.SimpleNamespace(get_device_name=lambda i: "stub-device-name")
    testing = types.ModuleType("torch_npu.testing")
    testcase = types.ModuleType("torch_npu.testing.testcase")
    testcase.TestCase = unittest.TestCase
    testcase.run_tests = lambda: None
    stub.testing, testing.testcase = testing, testcase
    for name, mod in (("torch_npu", stub), ("torch_npu.testing", testing),
                      ("torch_npu.testing.testcase", testcase),
                      ("mx_driving", types.ModuleType("mx_driving")),
                      ("mx_driving.fused", types.ModuleType("mx_driving.fused"))):
        sys.modules.setdefault(name, mod)
    sys.path.insert(0, os.path.join(REF, "tests", "torch"))
    import test_deformable_aggregation as ref_test  # noqa: E402
    return ref_test.TestDeformableAggregation


def main():
    cls = load_reference_test_class()
    golden = cls.golden_deformable_aggregation.__wrapped__
    rng = np.random.default_rng(7)
    blob = {}
    for name, (B, C, A, Pts, G, maps) in CASES.items():
        cams, scales = len(maps), len(maps[0])
        shapes = np.array(maps, dtype=np.int32).reshape(cams, scales, 2)
        sizes = (shapes[..., 0] * shapes[..., 1]).reshape(-1)
        starts = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int32).reshape(cams, scales)
        Fk = int(sizes.sum())
        feat = rng.random((B, Fk, C), dtype=np.float32)
        loc = (rng.random((B, A, Pts, cams, 2), dtype=np.float32) * 1.2 - 0.1).astype(np.float32)
        wts = rng.random((B, A, Pts, cams, scales, G), dtype=np.float32)
        out = golden(None, B, A, Pts, cams, scales, C, G, Fk, feat.flatten(), shapes, starts, loc,
                     wts.flatten())
        blob.update({f"{name}/feat": feat, f"{name}/shapes": shapes, f"{name}/starts": starts,
                     f"{name}/loc": loc, f"{name}/wts": wts,
                     f"{name}/grad_out": rng.standard_normal((B, A, C), dtype=np.float32),
                     f"{name}/out": out})
    np.savez_compressed(OUT, **blob)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(CASES), "cases")


if __name__ == "__main__":
    main()

"""Access to the committed golden fixtures (tests/golden/msda_golden.npz).

The fixtures hold outputs of the reference's own golden functions
(tests/torch/test_multi_scale_deformable_attn.py:34-76) on seeded inputs; see
tests/golden/make_golden.py for how they were produced.
"""
import os

import numpy as np

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "msda_golden.npz")
_FIELDS = ("shapes", "starts", "value", "loc", "attn", "grad_out",
           "out", "grad_value", "grad_loc", "grad_attn")


def load_all():
    z = np.load(_PATH)
    names = sorted({k.split("/")[0] for k in z.files})
    cases = {}
    for n in names:
        c = {f: z[f"{n}/{f}"] for f in _FIELDS}
        c["dtype"] = str(z[f"{n}/dtype"])
        cases[n] = c
    return cases


CASES = load_all()
NAMES = sorted(CASES)

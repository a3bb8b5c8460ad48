"""Deprecated import path kept by the reference (mx_driving/fused.py:7-9): re-exports the
MSDA operator names, ``npu_deformable_aggregation``, ``npu_add_relu`` and ``npu_max_pool2d``. The other operators that module
re-exports are not part of this tree."""
import warnings

from drivingsdk_b200.ops.multi_scale_deformable_attn import (  # noqa: F401
    MultiScaleDeformableAttnFunction,
    multi_scale_deformable_attn,
    npu_multi_scale_deformable_attn_function,
)

from drivingsdk_b200.ops.npu_deformable_aggregation import npu_deformable_aggregation  # noqa: F401,E402
from drivingsdk_b200.ops.npu_add_relu import npu_add_relu  # noqa: F401,E402
from drivingsdk_b200.ops.npu_max_pool2d import npu_max_pool2d  # noqa: F401,E402

warnings.warn(
    "This package is deprecated and will be removed in future. Please use `mx_driving` instead.",
    DeprecationWarning,
)

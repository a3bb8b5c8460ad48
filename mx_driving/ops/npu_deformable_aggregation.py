"""Same module path as the reference's operator wrapper
(mx_driving/ops/npu_deformable_aggregation.py)."""
from drivingsdk_b200.ops.npu_deformable_aggregation import (  # noqa: F401
    AdsDeformableAggregation,
    deformable_aggregation,
    npu_deformable_aggregation,
)

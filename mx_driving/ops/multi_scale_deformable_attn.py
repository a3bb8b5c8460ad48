"""Same module path as the reference's operator wrapper
(mx_driving/ops/multi_scale_deformable_attn.py)."""
from drivingsdk_b200.ops.multi_scale_deformable_attn import (  # noqa: F401
    MultiScaleDeformableAttnFunction,
    multi_scale_deformable_attn,
    npu_multi_scale_deformable_attn_function,
)

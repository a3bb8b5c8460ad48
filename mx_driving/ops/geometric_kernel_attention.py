"""Same module path as the reference's operator wrapper
(mx_driving/ops/geometric_kernel_attention.py)."""
from drivingsdk_b200.ops.geometric_kernel_attention import (  # noqa: F401
    GeometricKernelAttentionFunc,
    geometric_kernel_attention,
)

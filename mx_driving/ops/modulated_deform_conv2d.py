"""Same module path as the reference's operator wrapper
(mx_driving/ops/modulated_deform_conv2d.py)."""
from drivingsdk_b200.ops.modulated_deform_conv2d import (  # noqa: F401
    ModulatedDeformConv2dFunction,
    modulated_deform_conv2d,
)

"""Same module path as the reference's operator wrapper (mx_driving/ops/deform_conv2d.py)."""
from drivingsdk_b200.ops.deform_conv2d import DeformConv2dFunction, deform_conv2d  # noqa: F401

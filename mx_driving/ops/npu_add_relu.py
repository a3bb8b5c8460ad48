"""Same module path as the reference's operator wrapper (mx_driving/ops/npu_add_relu.py)."""
from drivingsdk_b200.ops.npu_add_relu import AddReluFunction, npu_add_relu  # noqa: F401

"""Same module path as the reference's operator wrapper (mx_driving/ops/npu_max_pool2d.py)."""
from drivingsdk_b200.ops.npu_max_pool2d import MaxPool2d, npu_max_pool2d  # noqa: F401

"""3x3 / stride 2 / padding 1 max pooling for inference: wrapper over the sm_100a kernel.

Mirrors the reference wrapper (mx_driving/ops/npu_max_pool2d.py:13-19): ``MaxPool2d`` (an
autograd Function without backward) and ``npu_max_pool2d = MaxPool2d.apply``; any other
kernel size, stride or padding is an error, as in the reference binding
(mx_driving/csrc/MaxPool2d.cpp:31-33). No CPU path.
"""
from torch.autograd import Function

try:
    from drivingsdk_b200 import _C
except ImportError as exc:
    raise ImportError(
        "drivingsdk_b200._C (the compiled sm_100a extension) is not built; run "
        "`python -m drivingsdk_b200.build` in the source tree. There is no CPU fallback."
    ) from exc


class MaxPool2d(Function):
    @staticmethod
    # pylint: disable=too-many-arguments
    def forward(ctx, x, kernel_size, stride, padding):
        return _C.npu_max_pool2d(x, kernel_size, stride, padding)


npu_max_pool2d = MaxPool2d.apply

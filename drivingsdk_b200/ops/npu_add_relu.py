"""Fused add + ReLU: autograd wrapper over the sm_100a kernels.

Mirrors the reference wrapper (mx_driving/ops/npu_add_relu.py:19-37): ``AddReluFunction``
and ``npu_add_relu = AddReluFunction.apply``. As in the reference, an ``x`` of at least
2,000,000 elements is overwritten with ``relu(x + y)`` and returned, a smaller one is left
untouched and the result is a new tensor (the reference computes ``F.relu(x + y)`` there);
the result is what backward keeps, and both addends receive the same gradient
``grad_output * (result > 0)``. Differences: the kernel runs at every size (on a copy of
``x`` below the threshold), the overwrite is declared to autograd (``mark_dirty``), and an
``x`` that may not be overwritten (non-contiguous, or a leaf that requires grad) is copied
first whatever its size. No CPU path.
"""
import torch
from torch.autograd import Function

try:
    from drivingsdk_b200 import _C
except ImportError as exc:
    raise ImportError(
        "drivingsdk_b200._C (the compiled sm_100a extension) is not built; run "
        "`python -m drivingsdk_b200.build` in the source tree. There is no CPU fallback."
    ) from exc


# the reference overwrites x only from this size up (mx_driving/ops/npu_add_relu.py:22)
IN_PLACE_MIN_NUMEL = 2000000


class AddReluFunction(Function):
    @staticmethod
    def forward(ctx, x, y):
        in_place = (x.numel() >= IN_PLACE_MIN_NUMEL and x.is_contiguous()
                    and not (x.is_leaf and x.requires_grad))
        if not in_place:
            x = x.clone(memory_format=torch.contiguous_format)
        x = _C.npu_add_relu(x, y)
        if in_place:
            ctx.mark_dirty(x)
        ctx.save_for_backward(x)
        return x

    @staticmethod
    def backward(ctx, grad_output):
        (x,) = ctx.saved_tensors
        result = _C.npu_add_relu_grad(x, grad_output)
        return result, result


npu_add_relu = AddReluFunction.apply

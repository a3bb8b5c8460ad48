"""Deformable convolution (DCNv1): autograd wrapper over the sm_100a kernels.

Mirrors the reference wrapper (mx_driving/ops/deform_conv2d.py:19-121), which in turn keeps
mmcv's call convention: ``DeformConv2dFunction.apply(x, offset, weight, stride, padding,
dilation, groups, deformable_groups, bias, im2col_step)`` with NCHW ``x``, ``offset``
``[n, deformable_groups * 2 * kh * kw, h_out, w_out]`` (per tap (dy, dx)) and ``weight``
``[c_out, c_in / groups, kh, kw]``; ``bias`` and ``im2col_step`` are accepted and ignored as
in the reference. The sampled input (``offset_output``) is kept for the backward. Unlike the
reference, deformable_groups > 1 is honoured. No CPU path.
"""
from typing import Tuple, Union

import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable
from torch.nn.modules.utils import _pair

try:
    from drivingsdk_b200 import _C
except ImportError as exc:
    raise ImportError(
        "drivingsdk_b200._C (the compiled sm_100a extension) is not built; run "
        "`python -m drivingsdk_b200.build` in the source tree. There is no CPU fallback."
    ) from exc


def _channels_last(t: torch.Tensor) -> torch.Tensor:
    return t.permute(0, 2, 3, 1).contiguous()


class DeformConv2dFunction(Function):
    @staticmethod
    # pylint: disable=too-many-arguments
    def forward(ctx, x: torch.Tensor, offset: torch.Tensor, weight: torch.Tensor,
                stride: Union[int, Tuple[int, ...]] = 1, padding: Union[int, Tuple[int, ...]] = 0,
                dilation: Union[int, Tuple[int, ...]] = 1, groups: int = 1,
                deformable_groups: int = 1, bias=False, im2col_step=32):
        ctx.kernel_size = [weight.size(2), weight.size(3)]
        ctx.stride = list(_pair(stride))
        ctx.padding = list(_pair(padding))
        ctx.dilation = list(_pair(dilation))
        ctx.groups = groups
        ctx.deformable_groups = deformable_groups
        nhwc_x, nhwc_offset, nhwc_weight = (_channels_last(t) for t in (x, offset, weight))
        out, offset_output = _C.deformable_conv2d(
            nhwc_x, nhwc_offset, nhwc_weight, ctx.kernel_size, ctx.stride, ctx.padding,
            ctx.dilation, ctx.groups, ctx.deformable_groups)
        ctx.save_for_backward(nhwc_x, nhwc_offset, nhwc_weight, offset_output)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        nhwc_x, nhwc_offset, nhwc_weight, offset_output = ctx.saved_tensors
        grad_x, grad_weight, grad_offset = _C.deformable_conv2d_backward(
            nhwc_x, nhwc_weight, nhwc_offset, offset_output, _channels_last(grad_out),
            ctx.kernel_size, ctx.stride, ctx.padding, ctx.dilation, ctx.groups,
            ctx.deformable_groups)
        return grad_x, grad_offset, grad_weight, None, None, None, None, None, None, None


def deform_conv2d(x: torch.Tensor, offset: torch.Tensor, weight: torch.Tensor,
                  stride: Union[int, Tuple[int, ...]] = 1,
                  padding: Union[int, Tuple[int, ...]] = 0,
                  dilation: Union[int, Tuple[int, ...]] = 1, groups: int = 1,
                  deformable_groups: int = 1, bias=False, im2col_step=32):
    return DeformConv2dFunction.apply(x, offset, weight, stride, padding, dilation, groups,
                                      deformable_groups, bias, im2col_step)

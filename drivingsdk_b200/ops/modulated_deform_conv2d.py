"""Modulated deformable convolution (DCNv2): autograd wrapper over the sm_100a kernels.

Mirrors the reference wrapper (mx_driving/ops/modulated_deform_conv2d.py:24-132) and mmcv's
call convention: ``ModulatedDeformConv2dFunction.apply(x, offset, mask, weight, bias, stride,
padding, dilation, groups, deformable_groups)`` with NCHW tensors, ``offset``
``[n, deformable_groups * 2 * kh * kw, h_out, w_out]`` and ``mask``
``[n, deformable_groups * kh * kw, h_out, w_out]``. Differences from the reference: any kernel
size and any channel count that is a multiple of 4 per group (the reference wants 3x3 and
64-aligned channels), ``bias`` is applied and differentiated (the reference drops it), and
the sampled input is always kept for the backward. Inputs are computed in fp32 under autocast,
as the reference's ``custom_fwd(cast_inputs=torch.float32)`` does. No CPU path.
"""
from typing import Optional, Tuple, Union

import torch
from torch import nn
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


class ModulatedDeformConv2dFunction(Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float32)
    # pylint: disable=too-many-arguments
    def forward(ctx, x: torch.Tensor, offset: torch.Tensor, mask: torch.Tensor,
                weight: torch.Tensor, bias: Optional[nn.Parameter] = None,
                stride: Union[int, Tuple[int, ...]] = 1, padding: Union[int, Tuple[int, ...]] = 0,
                dilation: Union[int, Tuple[int, ...]] = 1, groups: int = 1,
                deformable_groups: int = 1):
        ctx.kernel_size = [weight.size(2), weight.size(3)]
        ctx.stride = list(_pair(stride))
        ctx.padding = list(_pair(padding))
        ctx.dilation = list(_pair(dilation))
        ctx.groups = groups
        ctx.deformable_groups = deformable_groups
        ctx.with_bias = bias is not None
        nhwc_x, nhwc_offset, nhwc_mask, nhwc_weight = (
            _channels_last(t) for t in (x, offset, mask, weight))
        out, offset_output = _C.modulated_deformable_conv2d(
            nhwc_x, nhwc_offset, nhwc_mask, nhwc_weight, bias, ctx.kernel_size, ctx.stride,
            ctx.padding, ctx.dilation, ctx.groups, ctx.deformable_groups, int(ctx.with_bias))
        ctx.save_for_backward(nhwc_x, nhwc_offset, nhwc_weight, nhwc_mask, offset_output,
                              bias if ctx.with_bias else None)
        return out

    @staticmethod
    @once_differentiable
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_out):
        nhwc_x, nhwc_offset, nhwc_weight, nhwc_mask, offset_output, bias = ctx.saved_tensors
        grad_x, grad_weight, grad_bias, grad_offset, grad_mask = \
            _C.modulated_deformable_conv2d_backward(
                nhwc_x, nhwc_offset, nhwc_mask, nhwc_weight, bias, offset_output,
                _channels_last(grad_out), ctx.kernel_size, ctx.stride, ctx.padding, ctx.dilation,
                ctx.groups, ctx.deformable_groups, int(ctx.with_bias))
        return (grad_x, grad_offset, grad_mask, grad_weight, grad_bias,
                None, None, None, None, None)


def modulated_deform_conv2d(x: torch.Tensor, offset: torch.Tensor, mask: torch.Tensor,
                            weight: torch.Tensor, bias: Optional[nn.Parameter] = None,
                            stride: Union[int, Tuple[int, ...]] = 1,
                            padding: Union[int, Tuple[int, ...]] = 0,
                            dilation: Union[int, Tuple[int, ...]] = 1, groups: int = 1,
                            deformable_groups: int = 1):
    return ModulatedDeformConv2dFunction.apply(x, offset, mask, weight, bias, stride, padding,
                                               dilation, groups, deformable_groups)

"""Deformable aggregation: autograd wrapper over the sm_100a kernels.

Mirrors the reference wrapper (mx_driving/ops/npu_deformable_aggregation.py:9-88): class
``AdsDeformableAggregation``, functions ``npu_deformable_aggregation`` and
``deformable_aggregation``; empty feature maps / weights raise ``Exception``; backward
returns ``(grad_mc_ms_feat, None, None, grad_sampling_location, grad_weights)``.
No CPU path: the compiled extension is required.
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


class AdsDeformableAggregation(Function):
    @staticmethod
    # pylint: disable=too-many-arguments
    def forward(ctx, mc_ms_feat: torch.Tensor, spatial_shape: torch.Tensor,
                scale_start_index: torch.Tensor, sampling_location: torch.Tensor,
                weights: torch.Tensor):
        if torch.numel(mc_ms_feat) == 0 or torch.numel(weights) == 0:
            raise Exception("Error! Input Tensor can not be a empty Tensor.\n")
        mc_ms_feat = mc_ms_feat.contiguous()
        spatial_shape = spatial_shape.contiguous().int()
        scale_start_index = scale_start_index.contiguous().int()
        sampling_location = sampling_location.contiguous()
        weights = weights.contiguous()
        output = _C.npu_deformable_aggregation(
            mc_ms_feat, spatial_shape, scale_start_index, sampling_location, weights)
        ctx.save_for_backward(mc_ms_feat, spatial_shape, scale_start_index, sampling_location,
                              weights)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        mc_ms_feat, spatial_shape, scale_start_index, sampling_location, weights = ctx.saved_tensors
        if (torch.numel(mc_ms_feat) == 0 or torch.numel(spatial_shape) == 0
                or torch.numel(sampling_location) == 0):
            raise Exception("Error! Input Tensor can not be a empty Tensor.\n")
        grad_mc_ms_feat, grad_sampling_location, grad_weights = _C.npu_deformable_aggregation_backward(
            mc_ms_feat, spatial_shape, scale_start_index, sampling_location, weights,
            grad_output.contiguous(), mc_ms_feat.new_empty(0), sampling_location.new_empty(0),
            weights.new_empty(0))
        return grad_mc_ms_feat, None, None, grad_sampling_location, grad_weights


npu_deformable_aggregation = AdsDeformableAggregation.apply
deformable_aggregation = AdsDeformableAggregation.apply

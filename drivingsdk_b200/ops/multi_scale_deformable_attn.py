"""Multi-scale deformable attention: autograd wrapper over the sm_100a kernels.

Mirrors the reference wrapper (mx_driving/ops/multi_scale_deformable_attn.py:18-95):
same class and function names, same argument order, same behaviours —
  * under autocast all floating inputs are cast to float32 (custom_fwd, :20);
  * empty ``value`` / ``value_spatial_shapes`` / ``attention_weights`` raise
    ``Exception`` (:31-32);
  * ``value_spatial_shapes`` and ``value_level_start_index`` may be int32 or
    int64 and are cast to int32 (:33-34);
  * ``sampling_locations`` and ``attention_weights`` are cast to ``value``'s
    dtype (:35-36);
  * backward is once-differentiable and returns
    ``(grad_value, None, None, grad_sampling_loc, grad_attn_weight)`` (:46-55).
There is no CPU path: the compiled extension is required, and missing it is an
ImportError at import of this module.
"""
import warnings

import torch
from torch.amp import custom_bwd, custom_fwd
from torch.autograd.function import Function, once_differentiable

try:
    from drivingsdk_b200 import _C
except ImportError as exc:  # fail loudly: nothing else can run this operator
    raise ImportError(
        "drivingsdk_b200._C (the compiled sm_100a extension) is not built; run "
        "`python -m drivingsdk_b200.build` in the source tree. There is no CPU fallback."
    ) from exc


class MultiScaleDeformableAttnFunction(Function):
    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float32)
    # pylint: disable=too-many-arguments
    def forward(
        ctx,
        value: torch.Tensor,
        value_spatial_shapes: torch.Tensor,
        value_level_start_index: torch.Tensor,
        sampling_locations: torch.Tensor,
        attention_weights: torch.Tensor,
        **kwargs,
    ) -> torch.Tensor:
        if value.numel() == 0 or value_spatial_shapes.numel() == 0 or attention_weights.numel() == 0:
            raise Exception("Error! Input Tensor can not be a empty Tensor.\n")
        value_spatial_shapes = value_spatial_shapes.int()
        value_level_start_index = value_level_start_index.int()
        sampling_locations = sampling_locations.type_as(value)
        attention_weights = attention_weights.type_as(value)

        output = _C.multi_scale_deformable_attn(
            value, value_spatial_shapes, value_level_start_index, sampling_locations, attention_weights
        )
        ctx.save_for_backward(
            value, value_spatial_shapes, value_level_start_index, sampling_locations, attention_weights
        )
        return output

    @staticmethod
    @once_differentiable
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_output: torch.Tensor) -> tuple:
        value, value_spatial_shapes, value_level_start_index, sampling_locations, attention_weights = (
            ctx.saved_tensors
        )
        grad_value, grad_sampling_loc, grad_attn_weight = _C.multi_scale_deformable_attn_backward(
            value, value_spatial_shapes, value_level_start_index, sampling_locations, attention_weights,
            grad_output,
        )
        return grad_value, None, None, grad_sampling_loc, grad_attn_weight


multi_scale_deformable_attn = MultiScaleDeformableAttnFunction.apply


def npu_multi_scale_deformable_attn_function(value, shape, offset, locations, weight):
    warnings.warn(
        "`npu_multi_scale_deformable_attn_function` will be deprecated in future. "
        "Please use `multi_scale_deformable_attn` instead.",
        DeprecationWarning,
    )
    return MultiScaleDeformableAttnFunction.apply(value, shape, offset, locations, weight)

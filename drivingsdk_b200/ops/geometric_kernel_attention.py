"""Geometric kernel attention: autograd wrapper over the sm_100a kernels.

Mirrors the reference wrapper (mx_driving/ops/geometric_kernel_attention.py:27-54): same
class and function names, same argument order. ``sampling_locations`` holds integer pixel
coordinates (x, y) per level (any integer or floating dtype); each sample reads the one
pixel at those coordinates clamped into its level, weighted by ``attention_weights``.
Backward returns ``(grad_value, None, None, None, grad_attn_weights)``: locations have no
gradient. No CPU path: the compiled extension is required.
"""
from typing import Any

import torch
from torch.autograd import Function

try:
    from drivingsdk_b200 import _C
except ImportError as exc:
    raise ImportError(
        "drivingsdk_b200._C (the compiled sm_100a extension) is not built; run "
        "`python -m drivingsdk_b200.build` in the source tree. There is no CPU fallback."
    ) from exc


class GeometricKernelAttentionFunc(Function):
    @staticmethod
    # pylint: disable=too-many-arguments
    def forward(ctx: Any, value: torch.Tensor, spatial_shapes: torch.Tensor,
                level_start_index: torch.Tensor, sampling_locations: torch.Tensor,
                attention_weights: torch.Tensor) -> torch.Tensor:
        ctx.save_for_backward(value, spatial_shapes, level_start_index, sampling_locations,
                              attention_weights)
        ctx.value_size = value.size()
        batch_size, num_keys, num_heads, dim = value.size()
        num_queries = attention_weights.size(1)
        output = value.new_zeros(batch_size, num_queries, num_heads * dim)
        _C.geometric_kernel_attention_forward(
            value, spatial_shapes, level_start_index, sampling_locations, attention_weights, output)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        value, spatial_shapes, level_start_index, sampling_locations, attn_weights = ctx.saved_tensors
        grad_value, grad_attn_weights = _C.geometric_kernel_attention_backward(
            value, spatial_shapes, level_start_index, sampling_locations, attn_weights,
            grad_output.contiguous())
        return grad_value, None, None, None, grad_attn_weights


geometric_kernel_attention = GeometricKernelAttentionFunc.apply

"""Fused multi-scale deformable attention: the operator plus the arithmetic around it.

mmcv's ``MultiScaleDeformableAttention.forward`` (the module BEVFormer, Deformable-DETR and
the other callers of the operator use) computes, before calling the operator,

    attention_weights  = softmax(attention_logits over levels * points)
    sampling_locations = reference_points[:, :, None, :, None, :]
                         + sampling_offsets / (W_l, H_l)[None, None, None, :, None, :]

as separate kernels with two intermediate tensors. ``multi_scale_deformable_attn_fused``
takes ``reference_points [bs, nq, L, 2]``, ``sampling_offsets [bs, nq, H, L, P, 2]`` (pixels)
and ``attention_logits [bs, nq, H, L, P]`` directly; both computations, and their gradients,
run inside the sm_100a kernels. The reference library has no such operator (this is the
"caller-side fusion" step); results equal the unfused composition. Needs L * P <= 32.
"""
import torch
from torch.amp import custom_bwd, custom_fwd
from torch.autograd.function import Function, once_differentiable

try:
    from drivingsdk_b200 import _C
except ImportError as exc:
    raise ImportError(
        "drivingsdk_b200._C (the compiled sm_100a extension) is not built; run "
        "`python -m drivingsdk_b200.build` in the source tree. There is no CPU fallback."
    ) from exc


class MultiScaleDeformableAttnFusedFunction(Function):
    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float32)
    # pylint: disable=too-many-arguments
    def forward(ctx, value, value_spatial_shapes, value_level_start_index, reference_points,
                sampling_offsets, attention_logits):
        if value.numel() == 0 or value_spatial_shapes.numel() == 0 or attention_logits.numel() == 0:
            raise Exception("Error! Input Tensor can not be a empty Tensor.\n")
        value_spatial_shapes = value_spatial_shapes.int()
        value_level_start_index = value_level_start_index.int()
        reference_points = reference_points.type_as(value)
        sampling_offsets = sampling_offsets.type_as(value)
        attention_logits = attention_logits.type_as(value)
        output = _C.msda_fused_forward(value, value_spatial_shapes, value_level_start_index,
                                       reference_points, sampling_offsets, attention_logits)
        ctx.save_for_backward(value, value_spatial_shapes, value_level_start_index,
                              reference_points, sampling_offsets, attention_logits)
        return output

    @staticmethod
    @once_differentiable
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        value, shapes, starts, ref, off, logits = ctx.saved_tensors
        grad_value, grad_ref, grad_off, grad_logits = _C.msda_fused_backward(
            value, shapes, starts, ref, off, logits, grad_output)
        return grad_value, None, None, grad_ref, grad_off, grad_logits


multi_scale_deformable_attn_fused = MultiScaleDeformableAttnFusedFunction.apply


def compose_unfused(reference_points, sampling_offsets, attention_logits, value_spatial_shapes):
    """The two computations the fused operator absorbs, as the callers write them:
    returns (sampling_locations, attention_weights) for the plain operator."""
    bs, nq, H, L, P = attention_logits.shape
    normalizer = torch.stack([value_spatial_shapes[..., 1], value_spatial_shapes[..., 0]], -1)
    loc = (reference_points[:, :, None, :, None, :]
           + sampling_offsets / normalizer[None, None, None, :, None, :].to(sampling_offsets.dtype))
    attn = attention_logits.reshape(bs, nq, H, L * P).softmax(-1).reshape(bs, nq, H, L, P)
    return loc, attn

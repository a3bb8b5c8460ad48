"""The mmcv hooks: multi-scale deformable attention, and (further down) deformable and
modulated deformable convolution.

mmcv models call ``mmcv.ops.multi_scale_deform_attn.MultiScaleDeformableAttnFunction
.apply(value, spatial_shapes, level_start_index, sampling_locations, attention_weights,
im2col_step)``. This patch points that class's ``forward`` and ``backward`` at the
operator of this package, exactly as the reference does
(mx_driving/patcher/mmcv_patch.py:36-67): the forward adapter accepts and drops the
sixth positional ``im2col_step``; the backward adapter appends one ``None`` (the
gradient slot of ``im2col_step``). Replacements are given as dotted paths under
``mx_driving`` and resolved when the patch is applied, so importing this module needs
neither torch nor the compiled extension.
"""
from typing import List

from .patch import AtomicPatch, BasePatch, Patch


class MultiScaleDeformableAttention(Patch):
    """Multi-Scale Deformable Attention patch for mmcv."""

    name = "multi_scale_deformable_attention"
    legacy_name = "msda"
    target_module = "mmcv"

    @classmethod
    def patches(cls, options=None) -> List[BasePatch]:
        theirs = "mmcv.ops.multi_scale_deform_attn.MultiScaleDeformableAttnFunction"
        ours = "mx_driving.MultiScaleDeformableAttnFunction"

        def adapt_forward(our_forward):
            def forward(ctx, value, spatial_shapes, level_start_index, sampling_locations,
                        attention_weights, im2col_step=None):
                return our_forward(ctx, value, spatial_shapes, level_start_index,
                                   sampling_locations, attention_weights)
            return forward

        def adapt_backward(our_backward):
            def backward(ctx, grad_output):
                return (*our_backward(ctx, grad_output), None)
            return backward

        return [
            AtomicPatch(f"{theirs}.forward", f"{ours}.forward", replacement_wrapper=adapt_forward),
            AtomicPatch(f"{theirs}.backward", f"{ours}.backward", replacement_wrapper=adapt_backward),
        ]


class DeformConv(Patch):
    """Deformable Convolution patch for mmcv: the autograd function and the functional form
    are replaced by this package's (mx_driving/patcher/mmcv_patch.py:74-93); mmcv's
    ``DeformConv2d`` modules call the functional form, so they follow."""

    name = "deform_conv"
    legacy_name = "dc"
    target_module = "mmcv"

    @classmethod
    def patches(cls, options=None) -> List[BasePatch]:
        return [
            AtomicPatch("mmcv.ops.deform_conv.DeformConv2dFunction",
                        "mx_driving.DeformConv2dFunction"),
            AtomicPatch("mmcv.ops.deform_conv.deform_conv2d", "mx_driving.deform_conv2d"),
        ]


class ModulatedDeformConv(Patch):
    """Modulated Deformable Convolution patch for mmcv
    (mx_driving/patcher/mmcv_patch.py:100-119)."""

    name = "modulated_deform_conv"
    legacy_name = "mdc"
    target_module = "mmcv"

    @classmethod
    def patches(cls, options=None) -> List[BasePatch]:
        return [
            AtomicPatch("mmcv.ops.modulated_deform_conv.ModulatedDeformConv2dFunction",
                        "mx_driving.ModulatedDeformConv2dFunction"),
            AtomicPatch("mmcv.ops.modulated_deform_conv.modulated_deform_conv2d",
                        "mx_driving.modulated_deform_conv2d"),
        ]

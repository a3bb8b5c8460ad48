"""The mmcv hook of the MSDA path.

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

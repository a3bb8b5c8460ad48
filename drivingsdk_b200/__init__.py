"""B200-native (sm_100a) multi-scale deformable attention behind DrivingSDK's API.

Public surface, same names as the reference package exports for this path
(mx_driving/__init__.py:106-110):

    multi_scale_deformable_attn(value, value_spatial_shapes, value_level_start_index,
                                sampling_locations, attention_weights) -> Tensor
    MultiScaleDeformableAttnFunction          torch.autograd.Function
    npu_multi_scale_deformable_attn_function  deprecated alias
    patcher                                   the mmcv hook (default_patcher, MSDA, ...)
    geometric_kernel_attention(value, spatial_shapes, level_start_index, sampling_locations,
                               attention_weights) -> Tensor   (nearest-pixel sibling operator,
                               mx_driving/ops/geometric_kernel_attention.py:27-54)
    multi_scale_deformable_attn_fused(value, shapes, level_start, reference_points,
                               sampling_offsets, attention_logits) -> Tensor   (extension: the
                               operator with its callers' softmax and location arithmetic inside)
    deformable_aggregation / npu_deformable_aggregation(mc_ms_feat, spatial_shape,
                               scale_start_index, sampling_location, weights) -> Tensor
                               (mx_driving/ops/npu_deformable_aggregation.py:9-88)
    npu_add_relu(x, y) -> x = relu(x + y)      (mx_driving/ops/npu_add_relu.py:19-37)
    npu_max_pool2d(x, 3, 2, 1) -> Tensor       (mx_driving/ops/npu_max_pool2d.py:13-19)
    deform_conv2d(x, offset, weight, stride, padding, dilation, groups, deformable_groups)
                               DeformConv2dFunction   (mx_driving/ops/deform_conv2d.py:19-121)
    modulated_deform_conv2d(x, offset, mask, weight, bias, stride, padding, dilation, groups,
                               deformable_groups)   ModulatedDeformConv2dFunction
                               (mx_driving/ops/modulated_deform_conv2d.py:24-132)

    set_status_checks(on) -> previous         debugging: every operator call synchronises, reads
                               the device's status word and raises if a kernel refused or
                               abandoned work (also MSDA_CHECK_STATUS=1 in the environment)
    device_status(clear=True) -> int           the sticky status bits (synchronises)

The operator names are resolved on first use, so that the patcher (pure Python)
can be imported on a machine without the compiled extension. Using an operator
without the extension raises ImportError: there is no CPU or eager fallback.
"""
import importlib

__version__ = "0.1.0"

_OP_NAMES = (
    "multi_scale_deformable_attn",
    "MultiScaleDeformableAttnFunction",
    "npu_multi_scale_deformable_attn_function",
)
_GKA_NAMES = ("geometric_kernel_attention", "GeometricKernelAttentionFunc")
_FUSED_NAMES = ("multi_scale_deformable_attn_fused", "MultiScaleDeformableAttnFusedFunction")
_DA_NAMES = ("npu_deformable_aggregation", "deformable_aggregation", "AdsDeformableAggregation")
# operators behind the other default patches: name -> module under .ops
_CONV_SIDE = {
    "npu_add_relu": "npu_add_relu",
    "npu_max_pool2d": "npu_max_pool2d",
    "deform_conv2d": "deform_conv2d",
    "DeformConv2dFunction": "deform_conv2d",
    "modulated_deform_conv2d": "modulated_deform_conv2d",
    "ModulatedDeformConv2dFunction": "modulated_deform_conv2d",
}

__all__ = (list(_OP_NAMES) + list(_FUSED_NAMES) + list(_GKA_NAMES) + list(_DA_NAMES)
           + list(_CONV_SIDE)
           + ["patcher", "default_patcher", "dist", "set_status_checks", "device_status"])


def __getattr__(name):
    if name in _OP_NAMES:
        mod = importlib.import_module(__name__ + ".ops.multi_scale_deformable_attn")
        return getattr(mod, name)
    if name in _GKA_NAMES:
        mod = importlib.import_module(__name__ + ".ops.geometric_kernel_attention")
        return getattr(mod, name)
    if name in _FUSED_NAMES:
        mod = importlib.import_module(__name__ + ".ops.msda_fused")
        return getattr(mod, name)
    if name in _DA_NAMES:
        mod = importlib.import_module(__name__ + ".ops.npu_deformable_aggregation")
        return getattr(mod, name)
    if name in _CONV_SIDE:
        mod = importlib.import_module(__name__ + ".ops." + _CONV_SIDE[name])
        return getattr(mod, name)
    if name in ("set_status_checks", "device_status"):
        return getattr(importlib.import_module(__name__ + "._C"), name)
    if name == "_C":
        return importlib.import_module(__name__ + "._C")
    if name in ("patcher", "dist", "capi", "ops"):
        return importlib.import_module(__name__ + "." + name)
    if name == "default_patcher":
        return importlib.import_module(__name__ + ".patcher").default_patcher
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

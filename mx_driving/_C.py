"""``mx_driving._C`` for this path: the two extension entry points
(mx_driving/csrc/pybind.cpp:110-111)."""
from drivingsdk_b200._C import (  # noqa: F401
    deformable_conv2d,
    deformable_conv2d_backward,
    geometric_kernel_attention_backward,
    modulated_deformable_conv2d,
    modulated_deformable_conv2d_backward,
    geometric_kernel_attention_forward,
    multi_scale_deformable_attn,
    npu_add_relu,
    npu_add_relu_grad,
    npu_max_pool2d,
    npu_deformable_aggregation,
    npu_deformable_aggregation_backward,
    multi_scale_deformable_attn_backward,
)

/*
 * C ABI of the convolution-side operators that DrivingSDK's default patcher installs
 * next to multi-scale deformable attention (mx_driving/patcher/__init__.py:135-149):
 *   - add + ReLU and its gradient        (ResNetAddRelu;  mx_driving/csrc/AddRelu.cpp:20-32)
 *   - 3x3 / stride 2 / pad 1 max pooling (ResNetMaxPool;  mx_driving/csrc/MaxPool2d.cpp:25-100)
 *   - deformable and modulated deformable 2-D convolution, forward and backward
 *     (DeformConv, ModulatedDeformConv; mx_driving/csrc/DeformableConv2d.cpp:21-101,
 *      mx_driving/csrc/ModulatedDeformableConv2d.cpp)
 * Same library (libmsda_sm100.so), same conventions as msda_sm100.h: device pointers,
 * sizes, a dtype code and a CUDA stream in; a status code out (msda_status values,
 * text from msda_sm100_strerror). Nothing is allocated and nothing synchronises.
 */
#ifndef CONV_OPS_SM100_H_
#define CONV_OPS_SM100_H_

#include <stddef.h>
#include <stdint.h>

#include "msda_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * x[i] = max(x[i] + y[i], 0) in place, i < n. Replaces aclnnAddRelu
 * (mx_driving/csrc/AddRelu.cpp:20-24). NaN in, NaN out (as torch.relu).
 * dtype: MSDA_F32, MSDA_F16 or MSDA_BF16.
 */
int addrelu_sm100_forward(void* x, const void* y, size_t n, int dtype, void* stream);

/*
 * grad_in[i] = out[i] > 0 ? grad_out[i] : 0, where `out` is what the forward left in x.
 * Replaces the ReluGrad call of npu_add_relu_grad (mx_driving/csrc/AddRelu.cpp:26-32);
 * the same tensor is the gradient of both addends.
 */
int addrelu_sm100_backward(const void* out, const void* grad_out, void* grad_in, size_t n,
                           int dtype, void* stream);

/*
 * y[n, c, oh, ow] = max over the 3x3 window at stride 2, padding 1 of x[n, c, :, :];
 * x is [N, C, H, W] contiguous, y is [N, C, (H+1)/2, (W+1)/2]. Inference only, like the
 * reference (mx_driving/ops/npu_max_pool2d.py:13-19). Replaces aclnnMaxPool2dWithMask /
 * aclnnMaxPool2d (mx_driving/csrc/MaxPool2d.cpp:45-100) without its channel restrictions.
 * A NaN in the window gives NaN (as torch.nn.MaxPool2d).
 */
int maxpool_sm100_forward(const void* x, void* y, int N, int C, int H, int W, int dtype,
                          void* stream);

#ifdef __cplusplus
}
#endif

#endif /* CONV_OPS_SM100_H_ */

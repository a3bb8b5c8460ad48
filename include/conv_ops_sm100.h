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

/*
 * Deformable and modulated deformable 2-D convolution (DCNv1 / DCNv2), fp32, channels-last
 * tensors as the reference's extension takes them (mx_driving/ops/deform_conv2d.py:42-44):
 *   x       [N, H, W, C]
 *   offset  [N, Ho, Wo, deform_groups * 2 * kh * kw]   per tap (dy, dx)
 *   mask    [N, Ho, Wo, deform_groups * kh * kw]       or NULL (plain deformable convolution)
 *   weight  [Co, kh, kw, C / groups]
 *   bias    [Co] or NULL
 *   out     [N, Ho, Wo, Co]
 *   columns [N * Ho * Wo, groups, kh * kw, C / groups]  the sampled (and modulated) input,
 *           the reference's `offset_output`; written by the forward, read by the backward.
 * Ho, Wo follow from the offset tensor; they must equal the convolution's output size for the
 * given stride, padding and dilation. Rows move as 16-byte pieces when C / deform_groups and
 * C / groups are multiples of 4 (x and columns then have to be 16-byte aligned), else float
 * by float.
 */
typedef struct dcn_shape {
    int N, H, W, C;
    int Ho, Wo, Co;
    int kh, kw;
    int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
    int groups, deform_groups;
} dcn_shape;

/* Bytes of the `columns` tensor for this shape (0 when the shape is invalid). */
size_t dcn_sm100_columns_bytes(const dcn_shape* s);

/*
 * Bytes of scratch memory dcn_sm100_backward needs (the gradient of `columns`, plus a
 * transposed copy of the weights for the tensor-core product that forms it).
 */
size_t dcn_sm100_backward_workspace_bytes(const dcn_shape* s);

/*
 * Forward. Replaces aclnnDeformableConv2d with modulated = false / true
 * (mx_driving/csrc/DeformableConv2d.cpp:59-60, ModulatedDeformableConv2d.cpp:70-71), i.e. the
 * gather of kernels/deformable_conv2d/op_kernel/deformable_conv2d.cpp:223-420 followed by the
 * per-group matrix product (:206-221). `columns` must hold dcn_sm100_columns_bytes().
 */
int dcn_sm100_forward(const float* x, const float* offset, const float* mask, const float* weight,
                      const float* bias, float* out, float* columns, const dcn_shape* s,
                      void* stream);

/*
 * Backward. Replaces aclnnDeformableConv2dGrad (mx_driving/csrc/DeformableConv2d.cpp:92-94,
 * ModulatedDeformableConv2d.cpp:127-130). `columns` is what the forward wrote. Gradients
 * have the layouts of their tensors; grad_mask is required iff mask is given; grad_bias may
 * be NULL. grad_x, grad_weight and grad_bias are overwritten (zero-filled here first).
 */
int dcn_sm100_backward(const float* x, const float* offset, const float* mask,
                       const float* weight, const float* columns, const float* grad_out,
                       float* grad_x, float* grad_offset, float* grad_mask, float* grad_weight,
                       float* grad_bias, void* workspace, size_t workspace_bytes,
                       const dcn_shape* s, void* stream);

/*
 * Which matrix-product kernels the two calls above use: 1 (default) = the tcgen05 kernel
 * (fp32 operands split into two TF32 parts, three tensor-core products per tile, fp32
 * accumulation in tensor memory; fp32-class accuracy) where the shape allows it; 2 = the same
 * kernel with a single TF32 product per tile (three times fewer tensor-core instructions,
 * about 1e-3 relative accuracy, the trade torch.backends.cuda.matmul.allow_tf32 makes);
 * 0 = the plain fp32 FMA kernel everywhere. Returns the previous setting; any other value
 * only queries.
 */
int dcn_sm100_use_tensor_cores(int on);

/*
 * The matrix product underneath, exposed for tests and benchmarks:
 *   C[m, n] = sum_k A[m * lda + k] * B[n * ldb + k] (+ bias[n]),  C row stride ldc.
 * Uses the tcgen05 kernel when dcn_sm100_use_tensor_cores is on and A, B are 16-byte aligned
 * with lda, ldb multiples of 4, else the fp32 FMA kernel. splits > 1 cuts K across CTAs
 * (tcgen05 kernel only; C is zero-filled first). No reference counterpart.
 */
int gemm_nt_sm100_f32(const float* A, long long lda, const float* B, long long ldb, float* C,
                      long long ldc, const float* bias, int M, int N, int K, int splits,
                      void* stream);

/*
 * Same with both operands stored k-row by k-row (the grad_weight product of the convolution,
 * whose k is the pixel index):  C[m, n] = sum_k A[k * lda + m] * B[k * ldb + n].
 * tcgen05 kernel when lda, ldb are multiples of 4 and M, N multiples of 32.
 */
int gemm_tn_sm100_f32(const float* A, long long lda, const float* B, long long ldb, float* C,
                      long long ldc, int M, int N, int K, int splits, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* CONV_OPS_SM100_H_ */

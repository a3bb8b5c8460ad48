// Geometric kernel attention backward for sm_100a: for every sample s of task (b, q, h)
//     grad_value[row_s, :] += attn_s * grad_out[b, q, h, :]
//     grad_attn_s           = sum_d value[row_s, d] * grad_out[b, q, h, d]
// with row_s the clamped integer pixel of the sample; locations get no gradient. Replaces
// the reference's device kernel
// (kernels/geometric_kernel_attention/op_kernel/geometric_kernel_attn_grad.cpp).
// Same kernel template as the bilinear operator with one row per sample instead of four.
#include "msda_bwd_kernel.cuh"

namespace msda {

cudaError_t launch_gka_backward(const Params& p, int dtype, int acc_f32, const RowPlan& rp,
                                const LaunchShape& ls, cudaStream_t stream) {
    return launch_backward_cps<1>(p, dtype, acc_f32, rp, ls, stream);
}

}  // namespace msda

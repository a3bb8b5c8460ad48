// Fused MSDA backward for sm_100a: the bilinear backward kernel with the chain rule through
// location = reference point + offset / (W, H) and weight = softmax(logits) applied in phase 3:
// grad_offset = grad_location / (W, H); grad_reference_point = sum over heads and points of
// grad_location (fp32 atomics); grad_logit = p * (grad_weight - sum_j p_j * grad_weight_j).
#include "msda_bwd_kernel.cuh"

namespace msda {

cudaError_t launch_fused_backward(const Params& p, int dtype, int acc_f32, const RowPlan& rp,
                                  const LaunchShape& ls, cudaStream_t stream) {
    return launch_backward_cps<kModeFused>(p, dtype, acc_f32, rp, ls, stream);
}

}  // namespace msda

// Fused MSDA forward for sm_100a: the bilinear forward kernel whose phase 1 also does what the
// callers of the operator otherwise run as separate kernels — softmax of the attention logits
// over levels*points, and sampling location = reference point + offset / (W, H) of the level
// (the arithmetic of mmcv's MultiScaleDeformableAttention.forward around its call of the
// operator; listed as caller-side fusion in the scope of this work). L*P <= 32.
#include "msda_fwd_kernel.cuh"

namespace msda {

cudaError_t launch_fused_forward(const Params& p, int dtype, const RowPlan& rp,
                                 const LaunchShape& ls, cudaStream_t stream) {
    return launch_forward_cps<kModeFused>(p, dtype, rp, ls, stream);
}

}  // namespace msda

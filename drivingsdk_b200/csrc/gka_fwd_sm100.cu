// Geometric kernel attention forward for sm_100a: out[b,q,h,:] = sum over (level, point) of
// attention * value[b, level, clamp(y), clamp(x), h, :] — integer pixel coordinates, clamped
// into the level, no interpolation. Replaces the reference's device kernel
// (kernels/geometric_kernel_attention/op_kernel/geometric_kernel_attention.cpp:123-182).
// Same kernel template as the bilinear operator with one row per sample instead of four.
#include "msda_fwd_kernel.cuh"

namespace msda {

cudaError_t launch_gka_forward(const Params& p, int dtype, const RowPlan& rp,
                               const LaunchShape& ls, cudaStream_t stream) {
    return launch_forward_cps<1>(p, dtype, rp, ls, stream);
}

}  // namespace msda

// Host-side launch interface between the C-ABI layer and the kernel files.
#pragma once

#include <cuda_runtime.h>

#include "msda_common.cuh"

namespace msda {

// How one value row (D elements) is spread over the lanes of a warp.
//   scalar == false: the row is `lpr * nv` pieces of 16 bytes; `lpr` lanes hold
//                    one piece each, `nv` times (nv == 2 only for 1 KiB rows).
//   scalar == true : lane = channel mod 32, any D up to 256, no alignment need.
struct RowPlan {
    bool scalar;
    int lpr;
    int nv;
};

cudaError_t launch_forward(const Params& p, int dtype, const RowPlan& rp, int grid,
                           cudaStream_t stream);
size_t fwd_smem_bytes(const Params& p, size_t elem);

// acc_f32 != 0: p.grad_value points at fp32 accumulation memory even though
// the tensors are 16-bit (the caller converts afterwards).
cudaError_t launch_backward(const Params& p, int dtype, int acc_f32, const RowPlan& rp, int grid,
                            cudaStream_t stream);
size_t bwd_smem_bytes(const Params& p, size_t elem);

// out[i] = (T)acc[i] for n elements; dtype 1 = fp16, 2 = bf16.
cudaError_t launch_downcast(const float* acc, void* out, long long n, int dtype,
                            cudaStream_t stream);

}  // namespace msda

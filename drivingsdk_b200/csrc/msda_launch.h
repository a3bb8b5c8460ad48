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

// Grid of a persistent launch: `ctas_per_sm` CTAs on each of `sm_count` SMs, or — when
// ctas_per_sm <= 0 — as many as the occupancy calculator says are resident at once for this
// kernel and shared-memory size (a CTA that is not resident from the start would run its
// whole share of the work after the others have finished theirs).
struct LaunchShape {
    int sm_count;
    int ctas_per_sm;
};
inline cudaError_t persistent_grid(const void* kernel, size_t smem, const LaunchShape& ls,
                                   const Params& p, int* grid) {
    int per_sm = ls.ctas_per_sm;
    if (per_sm <= 0) {
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel,
                                                                      kThreadsPerCta, smem);
        if (e != cudaSuccess) return e;
        if (per_sm < 1) per_sm = 1;
    }
    const long long ctas_needed = (p.nitems + kWarpsPerCta - 1) / kWarpsPerCta;
    const long long cap = static_cast<long long>(ls.sm_count) * per_sm;
    *grid = static_cast<int>(ctas_needed < cap ? ctas_needed : cap);
    return cudaSuccess;
}

cudaError_t launch_forward(const Params& p, int dtype, const RowPlan& rp, const LaunchShape& ls,
                           cudaStream_t stream);
// bytes of dynamic shared memory per warp (goes into Params::warp_smem)
uint32_t fwd_warp_smem(int samples_per_item, size_t elem);

// acc_f32 != 0: p.grad_value points at fp32 accumulation memory even though
// the tensors are 16-bit (the caller converts afterwards).
cudaError_t launch_backward(const Params& p, int dtype, int acc_f32, const RowPlan& rp,
                            const LaunchShape& ls, cudaStream_t stream);
uint32_t bwd_warp_smem(int samples_per_item, size_t elem);

// Geometric kernel attention: same parameter block (grad_loc unused), one row per sample.
cudaError_t launch_gka_forward(const Params& p, int dtype, const RowPlan& rp,
                               const LaunchShape& ls, cudaStream_t stream);
cudaError_t launch_gka_backward(const Params& p, int dtype, int acc_f32, const RowPlan& rp,
                                const LaunchShape& ls, cudaStream_t stream);

// Fused variant (reference points + offsets + logits instead of locations + weights).
cudaError_t launch_fused_forward(const Params& p, int dtype, const RowPlan& rp,
                                 const LaunchShape& ls, cudaStream_t stream);
cudaError_t launch_fused_backward(const Params& p, int dtype, int acc_f32, const RowPlan& rp,
                                  const LaunchShape& ls, cudaStream_t stream);

// Adds to the library-wide kernel launch counter (msda_sm100_launch_count).
void count_launches(int n);

// Records `e` as the calling thread's last CUDA error (msda_sm100_last_cuda_error) and
// returns MSDA_ERR_CUDA.
int note_cuda_error(cudaError_t e);

// SM count of the current device and the device address of the library's sticky status word
// (msda_sm100_device_status reads and clears it); either pointer may be null. Returns an
// msda_status value.
int device_facts(int* sm_count, int** status_word);

// out[i] = (T)acc[i] for n elements; dtype 1 = fp16, 2 = bf16.
cudaError_t launch_downcast(const float* acc, void* out, long long n, int dtype,
                            cudaStream_t stream);

}  // namespace msda

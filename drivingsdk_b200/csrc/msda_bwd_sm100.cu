// MSDA backward for sm_100a. For every sample s of task (b, q, h) and corner c:
//     grad_value[row_c, :] += w_c * attn * grad_out[b, q, h, :]        (scatter)
//     S_c = sum_d value[row_c, d] * grad_out[b, q, h, d]               (gather)
// and per sample
//     grad_attn  = w1*S1 + w2*S2 + w3*S3 + w4*S4          (bilinear w, no attn)
//     grad_loc_x = W * attn * (hh*(S2 - S1) + lh*(S4 - S3))
//     grad_loc_y = H * attn * (hw*(S3 - S1) + lw*(S4 - S2))
// all three zero for a dropped sample. Replaces the reference's backward
// device kernel and tiling
// (kernels/multi_scale_deformable_attn/op_kernel/multi_scale_deformable_attn_grad.cpp:151-249,
//  op_host/multi_scale_deformable_attn_grad.cpp:35-86).
//
// Same decomposition as the forward kernel. In phase 2 each lane holds the
// piece of grad_out that matches its 16-byte piece of the row, issues one
// vector reduction into the accumulation row (red.global.add.v4.f32, or
// .v4.bf16x2 / .v4.f16x2 when accumulating straight into a 16-bit grad_value)
// and leaves its partial dot product in shared memory; when a row is spread
// over more than 8 lanes, xor shuffles first fold it to 8 partials. In phase 3
// lane = sample again: it sums the partials of its four corners, forms the
// three gradients and stores them next to its neighbours' (coalesced).
#include "msda_bwd_kernel.cuh"

namespace msda {

// fp32 accumulation buffer -> 16-bit grad_value
template <typename T>
__global__ void __launch_bounds__(256) msda_downcast_kernel(const float* __restrict__ acc,
                                                            T* __restrict__ out, long long n) {
    const long long nvec = n / 8;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
         i += stride) {
        const float4 a = reinterpret_cast<const float4*>(acc)[2 * i];
        const float4 b = reinterpret_cast<const float4*>(acc)[2 * i + 1];
        const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        reinterpret_cast<uint4*>(out)[i] = pack16<T>(f);
    }
    for (long long i = nvec * 8 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
         i < n; i += stride) {
        out[i] = Elem<T>::from_f(acc[i]);
    }
}

uint32_t bwd_warp_smem(int samples_per_item, size_t elem) {
    return warp_smem_bytes(samples_per_item, elem, kPartBytes);
}

cudaError_t launch_backward(const Params& p, int dtype, int acc_f32, const RowPlan& rp,
                            const LaunchShape& ls, cudaStream_t stream) {
    return launch_backward_cps<4>(p, dtype, acc_f32, rp, ls, stream);
}

cudaError_t launch_downcast(const float* acc, void* out, long long n, int dtype,
                            cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    long long blocks = (n / 8 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == 1) {
        msda_downcast_kernel<__half><<<(int)blocks, 256, 0, stream>>>(
            acc, static_cast<__half*>(out), n);
    } else if (dtype == 2) {
        msda_downcast_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
            acc, static_cast<__nv_bfloat16*>(out), n);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace msda

// Matrix products used by the deformable convolution: C[M, N] (+)= sum_k A(m, k) * B(n, k).
// Both operands are addressed as (row, k) with element strides, so the three products of the
// operator (columns x weights^T, grad_out x weights, grad_out^T x columns) are the same call
// with different strides.
#pragma once

#include <cuda_runtime.h>

namespace msda {

struct GemmArgs {
    const float* A;      // A(m, k) = A[m * a_row + k * a_k]
    long long a_row, a_k;
    const float* B;      // B(n, k) = B[n * b_row + k * b_k]
    long long b_row, b_k;
    float* C;            // C(m, n) = C[m * ldc + n]
    long long ldc;
    const float* bias;   // added per column n when not null
    int M, N, K;
};

// Plain fp32 FMA kernel: any strides, any sizes. Overwrites C.
cudaError_t gemm_simt(const GemmArgs& g, cudaStream_t stream);

// tcgen05 kernel: 16-byte aligned bases and either both operands with k contiguous (a_k ==
// b_k == 1, row strides multiples of 4 elements) or both with the row index contiguous
// (a_row == b_row == 1, k strides multiples of 4 elements, M and N multiples of 32; this is
// the grad_weight product, whose k is the pixel index). fp32 accuracy through a two-term TF32 split of
// both operands (passes == 3: three tensor-core products per tile), or one TF32 product per
// tile (passes == 1, about 1e-3 relative accuracy). `splits` > 1 cuts K into that many
// parts whose partial results are added into C with reductions (the first part adds the
// bias); C must be zero before. Overwrites C when splits == 1.
bool gemm_tc_supported(const GemmArgs& g);
cudaError_t gemm_tc(const GemmArgs& g, int splits, int passes, int* status_word,
                    cudaStream_t stream);

// out[c, r] = in[r, c] for an R x Cc matrix (row strides ld_in, ld_out, in elements).
cudaError_t transpose_f32(const float* in, long long ld_in, float* out, long long ld_out, int R,
                          int Cc, cudaStream_t stream);

}  // namespace msda

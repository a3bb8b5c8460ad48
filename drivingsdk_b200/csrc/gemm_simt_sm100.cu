// fp32 FMA matrix product with arbitrary operand strides, and a tiled transpose.
//
// This is the product kernel of last resort for the deformable convolution: it takes every
// shape and alignment (the tensor-core kernel has alignment rules) and is the reference the
// tensor-core kernel is checked against. 128 x 128 x 16 tiles, 256 threads, 8 x 8 results per
// thread, operands staged k-major in shared memory so that the inner loop reads two 16-byte
// vectors per operand.
#include "gemm_sm100.h"

#include <cstdint>

namespace msda {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, kThreads = 256;
constexpr int kPad = 4;

// Stages a [ROWS x BK] operand tile as s[k][row]. KMAJOR: k is the contiguous index in global
// memory, so neighbouring threads take neighbouring k; otherwise neighbouring rows.
template <bool KMAJOR>
__device__ __forceinline__ void stage_tile(const float* __restrict__ base, long long s_row,
                                           long long s_k, int row0, int rows_total, int k0,
                                           int k_total, float (*s)[BM + kPad]) {
    const int t = threadIdx.x;
    if (KMAJOR) {
        const int k = t % BK, r_first = t / BK;  // 16 k x 16 rows per pass
#pragma unroll
        for (int pass = 0; pass < BM / (kThreads / BK); ++pass) {
            const int r = r_first + pass * (kThreads / BK);
            const int gr = row0 + r, gk = k0 + k;
            s[k][r] = (gr < rows_total && gk < k_total) ? base[gr * s_row + gk * s_k] : 0.f;
        }
    } else {
        const int r = t % BM, k_first = t / BM;  // 128 rows x 2 k per pass
#pragma unroll
        for (int pass = 0; pass < BK / (kThreads / BM); ++pass) {
            const int k = k_first + pass * (kThreads / BM);
            const int gr = row0 + r, gk = k0 + k;
            s[k][r] = (gr < rows_total && gk < k_total) ? base[gr * s_row + gk * s_k] : 0.f;
        }
    }
}

template <bool A_KMAJOR, bool B_KMAJOR>
__global__ void __launch_bounds__(kThreads)
gemm_simt_kernel(GemmArgs g) {
    __shared__ __align__(16) float sA[BK][BM + kPad];
    __shared__ __align__(16) float sB[BK][BN + kPad];
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int tm = (threadIdx.x / 16) * 8, tn = (threadIdx.x % 16) * 8;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < g.K; k0 += BK) {
        stage_tile<A_KMAJOR>(g.A, g.a_row, g.a_k, m0, g.M, k0, g.K, sA);
        stage_tile<B_KMAJOR>(g.B, g.b_row, g.b_k, n0, g.N, k0, g.K, sB);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&sA[k][tm]);
            const float4 a1 = *reinterpret_cast<const float4*>(&sA[k][tm + 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&sB[k][tn]);
            const float4 b1 = *reinterpret_cast<const float4*>(&sB[k][tn + 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + tm + i;
        if (m >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + tn + j;
            if (n < g.N) g.C[m * g.ldc + n] = acc[i][j] + (g.bias ? g.bias[n] : 0.f);
        }
    }
}

constexpr int kTile = 32;
__global__ void __launch_bounds__(kTile * 8)
transpose_kernel(const float* __restrict__ in, long long ld_in, float* __restrict__ out,
                 long long ld_out, int R, int Cc) {
    __shared__ float tile[kTile][kTile + 1];
    const int r0 = blockIdx.x * kTile, c0 = blockIdx.y * kTile;
    for (int i = threadIdx.y; i < kTile; i += 8) {
        const int r = r0 + i, c = c0 + threadIdx.x;
        tile[i][threadIdx.x] = (r < R && c < Cc) ? in[r * ld_in + c] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < kTile; i += 8) {
        const int c = c0 + i, r = r0 + threadIdx.x;
        if (c < Cc && r < R) out[c * ld_out + r] = tile[threadIdx.x][i];
    }
}

}  // namespace

cudaError_t gemm_simt(const GemmArgs& g, cudaStream_t stream) {
    if (g.M <= 0 || g.N <= 0) return cudaSuccess;
    const dim3 grid((g.M + BM - 1) / BM, (g.N + BN - 1) / BN);
    const bool ak = g.a_k == 1, bk = g.b_k == 1;
    if (ak && bk) gemm_simt_kernel<true, true><<<grid, kThreads, 0, stream>>>(g);
    else if (ak) gemm_simt_kernel<true, false><<<grid, kThreads, 0, stream>>>(g);
    else if (bk) gemm_simt_kernel<false, true><<<grid, kThreads, 0, stream>>>(g);
    else gemm_simt_kernel<false, false><<<grid, kThreads, 0, stream>>>(g);
    return cudaGetLastError();
}

cudaError_t transpose_f32(const float* in, long long ld_in, float* out, long long ld_out, int R,
                          int Cc, cudaStream_t stream) {
    if (R <= 0 || Cc <= 0) return cudaSuccess;
    const dim3 grid((R + kTile - 1) / kTile, (Cc + kTile - 1) / kTile);
    transpose_kernel<<<grid, dim3(kTile, 8), 0, stream>>>(in, ld_in, out, ld_out, R, Cc);
    return cudaGetLastError();
}

}  // namespace msda

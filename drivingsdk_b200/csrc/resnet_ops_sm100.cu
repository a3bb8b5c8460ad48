// Element-wise add + ReLU (with its gradient) and the 3x3 / stride-2 / pad-1 max pooling of a
// ResNet stem, for sm_100a. Both are pure streaming work: the only figure of merit is the share
// of HBM bandwidth they reach, so every thread moves 16 bytes per access and keeps four
// independent accesses in flight.
//
// Replaces aclnnAddRelu + ReluGrad (mx_driving/csrc/AddRelu.cpp:20-32) and
// aclnnMaxPool2dWithMask / aclnnMaxPool2d (mx_driving/csrc/MaxPool2d.cpp:45-100).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/conv_ops_sm100.h"
#include "msda_launch.h"

namespace {

constexpr int kThreads = 256;
constexpr int kVecPerThread = 4;  // 16-byte accesses in flight per thread and operand

template <typename T> struct Cvt;
template <> struct Cvt<float> {
    static __device__ __forceinline__ float up(float v) { return v; }
    static __device__ __forceinline__ float down(float v) { return v; }
};
template <> struct Cvt<__half> {
    static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
};

// relu that keeps NaN: (v > 0) is false for NaN, so select on !(v <= 0)
__device__ __forceinline__ float relu_keep_nan(float v) { return (v <= 0.f) ? 0.f : v; }

template <typename T> struct alignas(16) Vec16 {
    static constexpr int kN = 16 / sizeof(T);
    T v[kN];
};

// BACKWARD == false: a = relu(a + b) written to `dst` (== a)
// BACKWARD == true : dst = a > 0 ? b : 0          (a = forward result, b = grad_out)
template <typename T, bool BACKWARD>
__device__ __forceinline__ T combine(T a, T b) {
    if (BACKWARD) return (Cvt<T>::up(a) > 0.f) ? b : Cvt<T>::down(0.f);
    return Cvt<T>::down(relu_keep_nan(Cvt<T>::up(a) + Cvt<T>::up(b)));
}

template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(kThreads)
pointwise_vec_kernel(const T* a, const T* __restrict__ b, T* dst,  // a may alias dst
                     size_t nvec) {
    using V = Vec16<T>;
    const V* av = reinterpret_cast<const V*>(a);
    const V* bv = reinterpret_cast<const V*>(b);
    V* dv = reinterpret_cast<V*>(dst);
    const size_t tile = static_cast<size_t>(kThreads) * kVecPerThread;
    for (size_t base = static_cast<size_t>(blockIdx.x) * tile; base < nvec;
         base += static_cast<size_t>(gridDim.x) * tile) {
        V ra[kVecPerThread], rb[kVecPerThread];
#pragma unroll
        for (int u = 0; u < kVecPerThread; ++u) {
            const size_t i = base + static_cast<size_t>(u) * kThreads + threadIdx.x;
            if (i < nvec) {
                ra[u] = av[i];
                rb[u] = bv[i];
            }
        }
#pragma unroll
        for (int u = 0; u < kVecPerThread; ++u) {
            const size_t i = base + static_cast<size_t>(u) * kThreads + threadIdx.x;
            if (i < nvec) {
                V r;
#pragma unroll
                for (int k = 0; k < V::kN; ++k) r.v[k] = combine<T, BACKWARD>(ra[u].v[k], rb[u].v[k]);
                dv[i] = r;
            }
        }
    }
}

// elements [first, n): the tail after the last whole 16 bytes, or everything when a pointer
// is not 16-byte aligned
template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(kThreads)
pointwise_scalar_kernel(const T* a, const T* __restrict__ b, T* dst,
                        size_t first, size_t n) {
    for (size_t i = first + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * kThreads)
        dst[i] = combine<T, BACKWARD>(a[i], b[i]);
}

int sm_count_of_current_device(int* sms) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return msda::note_cuda_error(e);
    e = cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return msda::note_cuda_error(e);
    return MSDA_OK;
}

template <typename T, bool BACKWARD>
int launch_pointwise(const void* a, const void* b, void* dst, size_t n, cudaStream_t stream) {
    int sms = 0;
    const int rc = sm_count_of_current_device(&sms);
    if (rc != MSDA_OK) return rc;
    const T* ap = static_cast<const T*>(a);
    const T* bp = static_cast<const T*>(b);
    T* dp = static_cast<T*>(dst);
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                           reinterpret_cast<uintptr_t>(dst)) % 16) == 0;
    const size_t per_vec = 16 / sizeof(T);
    const size_t nvec = aligned ? n / per_vec : 0;
    int launches = 0;
    if (nvec > 0) {
        const size_t tile = static_cast<size_t>(kThreads) * kVecPerThread;
        const size_t want = (nvec + tile - 1) / tile;
        const size_t cap = static_cast<size_t>(sms) * 8;  // 8 resident CTAs of 256 threads per SM
        const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
        pointwise_vec_kernel<T, BACKWARD><<<grid, kThreads, 0, stream>>>(ap, bp, dp, nvec);
        ++launches;
    }
    const size_t first = nvec * per_vec;
    if (first < n) {
        const size_t want = (n - first + kThreads - 1) / kThreads;
        const size_t cap = static_cast<size_t>(sms) * 8;
        const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
        pointwise_scalar_kernel<T, BACKWARD><<<grid, kThreads, 0, stream>>>(ap, bp, dp, first, n);
        ++launches;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return msda::note_cuda_error(e);
    msda::count_launches(launches);
    return MSDA_OK;
}

template <bool BACKWARD>
int dispatch_pointwise(const void* a, const void* b, void* dst, size_t n, int dtype,
                       void* stream) {
    if (a == nullptr || b == nullptr || dst == nullptr) return MSDA_ERR_NULL;
    if (n == 0) return MSDA_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MSDA_F32: return launch_pointwise<float, BACKWARD>(a, b, dst, n, s);
        case MSDA_F16: return launch_pointwise<__half, BACKWARD>(a, b, dst, n, s);
        case MSDA_BF16: return launch_pointwise<__nv_bfloat16, BACKWARD>(a, b, dst, n, s);
        default: return MSDA_ERR_DTYPE;
    }
}

// ---------------------------------------------------------------------------------------------
// 3x3 / stride 2 / pad 1 max pooling, NCHW. One thread produces four neighbouring outputs of
// one output row: they need nine input columns (2*ow0 - 1 .. 2*ow0 + 7) of three input rows,
// read as eight contiguous elements (16-byte loads where the row allows it) plus the one column
// to their left. Neighbouring threads take neighbouring groups, so a warp reads contiguous
// stretches of each input row; the overlap between output rows is served by L1 / L2.
// ---------------------------------------------------------------------------------------------
struct NanMax {
    float best = -INFINITY;
    bool seen_nan = false;
    __device__ __forceinline__ void take(float v) {
        seen_nan |= (v != v);
        best = fmaxf(best, v);
    }
    __device__ __forceinline__ float result() const {
        return seen_nan ? __int_as_float(0x7fc00000) : best;
    }
};

template <typename T>
__global__ void __launch_bounds__(kThreads)
maxpool3s2_kernel(const T* __restrict__ x, T* __restrict__ y, int H, int W, int OH, int OW,
                  int groups_per_row, size_t total_groups, int vec_in, int vec_out) {
    constexpr int kPerVec = 16 / sizeof(T);   // elements per 16-byte load
    for (size_t idx = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; idx < total_groups;
         idx += static_cast<size_t>(gridDim.x) * kThreads) {
        const int gq = static_cast<int>(idx % groups_per_row);
        const size_t t = idx / groups_per_row;
        const int oh = static_cast<int>(t % OH);
        const size_t plane = t / OH;  // n * C + c
        const T* src = x + plane * static_cast<size_t>(H) * W;
        const int ow0 = 4 * gq, c0 = 2 * ow0;
        NanMax acc[4];
        const bool whole = vec_in && (c0 + 7 < W);
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int h = 2 * oh - 1 + i;
            if (h < 0 || h >= H) continue;
            const T* row = src + static_cast<size_t>(h) * W;
            float v[9];   // columns c0 - 1 .. c0 + 7; -inf where outside the image
            v[0] = (c0 >= 1) ? Cvt<T>::up(row[c0 - 1]) : -INFINITY;
            if (whole) {
                alignas(16) T tmp[8];
#pragma unroll
                for (int q = 0; q < 8 / kPerVec; ++q)
                    *reinterpret_cast<uint4*>(&tmp[q * kPerVec]) =
                        *reinterpret_cast<const uint4*>(row + c0 + q * kPerVec);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[1 + j] = Cvt<T>::up(tmp[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[1 + j] = (c0 + j < W) ? Cvt<T>::up(row[c0 + j]) : -INFINITY;
            }
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                // a column outside the image was read as -inf, which never wins and is not NaN
                acc[o].take(v[2 * o]);
                acc[o].take(v[2 * o + 1]);
                acc[o].take(v[2 * o + 2]);
            }
        }
        T* dst = y + (plane * OH + oh) * static_cast<size_t>(OW) + ow0;
        if (vec_out && ow0 + 3 < OW) {
            alignas(16) T out4[4];
#pragma unroll
            for (int o = 0; o < 4; ++o) out4[o] = Cvt<T>::down(acc[o].result());
            if (sizeof(T) == 4) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(out4);
            else *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<uint2*>(out4);
        } else {
#pragma unroll
            for (int o = 0; o < 4; ++o)
                if (ow0 + o < OW) dst[o] = Cvt<T>::down(acc[o].result());
        }
    }
}

template <typename T>
int launch_maxpool(const void* x, void* y, int N, int C, int H, int W, cudaStream_t stream) {
    int sms = 0;
    const int rc = sm_count_of_current_device(&sms);
    if (rc != MSDA_OK) return rc;
    const int OH = (H + 1) / 2, OW = (W + 1) / 2;
    const int groups_per_row = (OW + 3) / 4;
    const size_t total = static_cast<size_t>(N) * C * OH * groups_per_row;
    // 16-byte loads need every row to start on a 16-byte boundary; vector stores likewise
    const int per_vec = 16 / static_cast<int>(sizeof(T));
    const int vec_in = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (W % per_vec == 0);
    const int vec_out = (reinterpret_cast<uintptr_t>(y) % 16 == 0) && (OW % 4 == 0);
    const size_t want = (total + kThreads - 1) / kThreads;
    const size_t cap = static_cast<size_t>(sms) * 8 * 4;  // four waves of resident CTAs at most
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    maxpool3s2_kernel<T><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(x), static_cast<T*>(y),
                                                        H, W, OH, OW, groups_per_row, total, vec_in,
                                                        vec_out);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return msda::note_cuda_error(e);
    msda::count_launches(1);
    return MSDA_OK;
}

}  // namespace

extern "C" {

int addrelu_sm100_forward(void* x, const void* y, size_t n, int dtype, void* stream) {
    return dispatch_pointwise<false>(x, y, x, n, dtype, stream);
}

int addrelu_sm100_backward(const void* out, const void* grad_out, void* grad_in, size_t n,
                           int dtype, void* stream) {
    return dispatch_pointwise<true>(out, grad_out, grad_in, n, dtype, stream);
}

int maxpool_sm100_forward(const void* x, void* y, int N, int C, int H, int W, int dtype,
                          void* stream) {
    if (x == nullptr || y == nullptr) return MSDA_ERR_NULL;
    if (N < 0 || C < 0 || H < 0 || W < 0) return MSDA_ERR_DIMS;
    if (static_cast<size_t>(N) * C * H * W == 0) return MSDA_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MSDA_F32: return launch_maxpool<float>(x, y, N, C, H, W, s);
        case MSDA_F16: return launch_maxpool<__half>(x, y, N, C, H, W, s);
        case MSDA_BF16: return launch_maxpool<__nv_bfloat16>(x, y, N, C, H, W, s);
        default: return MSDA_ERR_DTYPE;
    }
}

}  // extern "C"

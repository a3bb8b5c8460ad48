// Measured ceilings for the two operations that bound the MSDA kernels on B200: gathering
// random rows out of an L2-resident buffer with 16-byte vector loads (what the forward does
// with value rows) and adding random rows into such a buffer with red.global.add.v4.f32 (what
// the backward does with grad_value rows). The HBM roofline counts every operand once; these
// kernels move every value row ~10 times between L2 and the SMs, so the rates measured here —
// on the same device, in the same run — are the ceilings their row traffic can be held to.
// The reference has no counterpart (its device code reports no such ceilings).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/msda_sm100.h"
#include "msda_launch.h"

namespace {

// LPR lanes cover one row with 16 bytes each; U independent accesses in flight per lane;
// row numbers from a per-warp linear congruential generator, masked to the buffer.
template <int LPR, int OP /*0 gather, 1 red.add.v4.f32*/>
__global__ void __launch_bounds__(1024, 1)
row_rate_kernel(unsigned char* buf, uint32_t row_mask, int iters, float* sink) {
    constexpr int U = 8;
    constexpr uint32_t kRowBytes = LPR * 16;
    const int lane = threadIdx.x & 31;
    const int g = lane / LPR, j = lane % LPR;
    uint32_t s = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * 2654435761u + 12345u;
    float acc = 0.f;
    for (int it = 0; it < iters; ++it) {
        uint32_t rows[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            s = s * 1664525u + 1013904223u;
            rows[u] = ((s >> 7) + g * 0x9E3779B1u) & row_mask;
        }
        if (OP == 0) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                v[u] = msda::ldg16(buf + static_cast<size_t>(rows[u]) * kRowBytes + j * 16);
#pragma unroll
            for (int u = 0; u < U; ++u) acc += __uint_as_float(v[u].x) + __uint_as_float(v[u].w);
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u)
                msda::red_add_f32x4(reinterpret_cast<float*>(
                                        buf + static_cast<size_t>(rows[u]) * kRowBytes + j * 16),
                                    0.f, 0.f, 0.f, 0.f);
        }
    }
    if (acc == 12345.678f) sink[0] = acc;   // keeps the loads alive; never true for zeros
}

template <int LPR, int OP>
cudaError_t time_rate(unsigned char* buf, uint32_t rows, int sms, cudaStream_t stream,
                      double* rows_per_s) {
    const int iters = 256, threads = 1024;
    float* sink = reinterpret_cast<float*>(buf);   // never written (see kernel)
    cudaEvent_t a, b;
    cudaError_t e = cudaEventCreate(&a);
    if (e != cudaSuccess) return e;
    e = cudaEventCreate(&b);
    if (e != cudaSuccess) { cudaEventDestroy(a); return e; }
    for (int w = 0; w < 2; ++w)
        row_rate_kernel<LPR, OP><<<sms, threads, 0, stream>>>(buf, rows - 1, iters, sink);
    cudaEventRecord(a, stream);
    const int reps = 3;
    for (int r = 0; r < reps; ++r)
        row_rate_kernel<LPR, OP><<<sms, threads, 0, stream>>>(buf, rows - 1, iters, sink);
    cudaEventRecord(b, stream);
    e = cudaEventSynchronize(b);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (e != cudaSuccess) return e;
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const double total = static_cast<double>(sms) * (threads / 32) * iters * 8 * (32 / LPR) * reps;
    *rows_per_s = total / (ms * 1e-3);
    msda::count_launches(2 + reps);
    return cudaSuccess;
}

template <int OP>
cudaError_t time_rate_rows(int row_bytes, unsigned char* buf, uint32_t rows, int sms,
                           cudaStream_t stream, double* out) {
    switch (row_bytes) {
        case 64: return time_rate<4, OP>(buf, rows, sms, stream, out);
        case 128: return time_rate<8, OP>(buf, rows, sms, stream, out);
        case 256: return time_rate<16, OP>(buf, rows, sms, stream, out);
        case 512: return time_rate<32, OP>(buf, rows, sms, stream, out);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

extern "C" int msda_sm100_probe_row_rates(void* buffer, size_t buffer_bytes, int gather_row_bytes,
                                          int red_row_bytes, double* gather_rows_per_s,
                                          double* red_rows_per_s, void* stream_v) {
    if (!buffer || !gather_rows_per_s || !red_rows_per_s) return MSDA_ERR_NULL;
    auto ok_row = [](int b) { return b == 64 || b == 128 || b == 256 || b == 512; };
    if (!ok_row(gather_row_bytes) || !ok_row(red_row_bytes)) return MSDA_ERR_DIMS;
    if ((reinterpret_cast<uintptr_t>(buffer) & 15u) != 0) return MSDA_ERR_ALIGN;
    // largest power-of-two number of rows that fits (at least 1 MiB of either row size)
    auto pow2_rows = [&](int row_bytes) {
        uint32_t r = 1;
        while (static_cast<size_t>(r) * 2 * row_bytes <= buffer_bytes && r < (1u << 30)) r *= 2;
        return r;
    };
    if (buffer_bytes < (1u << 20)) return MSDA_ERR_WORKSPACE;
    int sms = 0;
    int rc = msda::device_facts(&sms, nullptr);
    if (rc != MSDA_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    unsigned char* buf = static_cast<unsigned char*>(buffer);
    cudaError_t e = cudaMemsetAsync(buf, 0, buffer_bytes, stream);
    if (e == cudaSuccess)
        e = time_rate_rows<0>(gather_row_bytes, buf, pow2_rows(gather_row_bytes), sms, stream,
                              gather_rows_per_s);
    if (e == cudaSuccess)
        e = time_rate_rows<1>(red_row_bytes, buf, pow2_rows(red_row_bytes), sms, stream,
                              red_rows_per_s);
    if (e != cudaSuccess) return msda::note_cuda_error(e);
    return MSDA_OK;
}

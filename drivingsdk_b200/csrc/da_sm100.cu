// Deformable aggregation (Sparse4D-style multi-camera, multi-scale feature sampling) for
// sm_100a, forward and backward, fp32. Replaces the reference's device kernels
// (kernels/deformable_aggregation/op_kernel/deformable_aggregation.cpp and
// deformable_aggregation_grad.cpp) and their host tiling.
//
//   feat [B, F, C]                      all cameras' and scales' feature maps, concatenated
//   spatial_shape [cams, scales, 2]     (h, w) of each map;  scale_start [cams, scales]
//   loc  [B, A, Pts, cams, 2]           (w, h) in (0, 1), shared by all scales of a camera
//   wts  [B, A, Pts, cams, scales, G]   one weight per group of C/G channels
//   out  [B, A, C] = sum over (pts, cam, scale) of bilinear(feat map, loc) * wts[group]
// A sample takes part only if 0 < loc_w < 1 and 0 < loc_h < 1; pixel coordinates are
// loc * size - 0.5, corners outside the map read as zero (same rules as the bilinear MSDA
// kernels, whose per-sample set-up and slot records are reused here).
//
// One warp per task = (batch, camera, block of points, anchor): the points are cut into blocks
// of floor(32 / scales), so a task's samples (point, scale) fill one warp pass and the scales
// of one point never straddle tasks. Tasks are ordered batch-major, then camera: the warps in
// flight at any time sample the maps of one or two cameras of one batch entry (15 MB each at
// the Sparse4D shape), which stay in L2; walking all cameras of an anchor in one task instead
// spread the working set over the whole batch entry (92 MB) and 4x the compulsory bytes came
// from DRAM. The price: a task's output row is a partial sum, added into `out` with vector
// reductions (out is zero-filled first; the order of those additions is not fixed).
//   phase 1  lane = sample: slot records {row offset | no row, bilinear weight}; the pass's
//            group weights are copied to shared memory.
//   phase 2  lane = (row slot, 16-byte piece of the C-channel row): gather, multiply by
//            bilinear weight * group weight, accumulate (forward); backward also issues the
//            vector reduction into grad_feat and leaves, per (slot, group), the dot product
//            of the row piece with grad_out in shared memory.
//   phase 3  (backward) lane = sample: grad_wts for its G groups, and its share of grad_loc,
//            which is summed over the scales of the (pts, cam) with shuffles.
#include <cstring>

#include "../../include/msda_sm100.h"
#include "msda_common.cuh"
#include "msda_launch.h"

namespace msda {

constexpr int kDaMaxMaps = 64;   // cams * scales
constexpr int kDaMaxGroups = 32;

struct DaParams {
    const float* feat;
    const float* loc;
    const float* wts;
    float* out;
    const float* grad_out;
    float* grad_feat;
    float* grad_loc;
    float* grad_wts;
    const int* shapes_dev;   // [cams*scales*2] (h, w), used when use_table == 0
    const int* starts_dev;   // [cams*scales]
    int use_table;
    int B, F, C, A, Pts, cams, scales, G;
    int S;         // samples per (batch, anchor): Pts * cams * scales
    int ppt;       // points per task: floor(32 / scales)
    int nparts;    // blocks of points: ceil(Pts / ppt)
    int cpg;       // channels per group
    uint32_t row_units;
    uint32_t warp_smem;
    long long ntasks;   // B * cams * nparts * A
    int lv_h[kDaMaxMaps], lv_w[kDaMaxMaps], lv_start[kDaMaxMaps];
};

// shared memory of one warp: slot records | group weights [32][G] | (bwd) A [32][4G+1]
__host__ __device__ inline uint32_t da_warp_smem(int G, bool backward) {
    uint32_t bytes = (kSlots + kSlotPad) * 8 + kChunk * G * 4;
    if (backward) bytes += kChunk * (4 * G + 1) * 4;
    return (bytes + 15u) & ~15u;
}

// Two CTAs per SM: with the camera-major task order fewer warps in flight mean fewer maps
// in flight, and the backward is faster with 106 registers at two CTAs than squeezed into 80
// for three (1.60 vs 1.80 ms at the Sparse4D shape); the forward needs 80 and gets three.
template <int LPR, int NV, bool SCALAR, bool BACKWARD>
__global__ void __launch_bounds__(kThreadsPerCta, 2) da_kernel(const __grid_constant__ DaParams p) {
    constexpr int VEC = SCALAR ? 1 : 4;
    constexpr int RPI = 32 / LPR;
    constexpr int UNROLL = (RPI >= 16) ? 2 : 4;
    constexpr int STEP = RPI * UNROLL;
    static_assert(kSlots % STEP == 0 && STEP <= kSlotPad, "slot loop must tile the slots");

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_lv[3][kDaMaxMaps];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane / LPR;
    const int j = lane % LPR;
    const int nmaps = p.cams * p.scales;
    for (int i = threadIdx.x; i < nmaps; i += blockDim.x) {
        s_lv[0][i] = p.use_table ? p.lv_h[i] : p.shapes_dev[2 * i];
        s_lv[1][i] = p.use_table ? p.lv_w[i] : p.shapes_dev[2 * i + 1];
        s_lv[2][i] = p.use_table ? p.lv_start[i] : p.starts_dev[i];
    }
    __syncthreads();

    unsigned char* wb = smem + static_cast<size_t>(warp) * p.warp_smem;
    uint2* s_slot = reinterpret_cast<uint2*>(wb);
    float* s_wt = reinterpret_cast<float*>(wb + (kSlots + kSlotPad) * 8);
    float* s_A = s_wt + kChunk * p.G;   // backward only
    const int G = p.G;
    const int astride = 4 * G + 1;

    const unsigned char* vlane = reinterpret_cast<const unsigned char*>(p.feat) + j * 16;
    unsigned char* glane = reinterpret_cast<unsigned char*>(p.grad_feat) + j * 16;
    // group of each of this lane's pieces (vector path) or channels (scalar path)
    int grp[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int ch = SCALAR ? (j + 32 * k) : (j + k * LPR) * 4;
        grp[k] = min(ch / p.cpg, G - 1);
    }
    const int lpg = SCALAR ? 1 : max(1, p.cpg / 4);   // lanes that share one group of a row (2^k)
    const bool group_writer = (j & (lpg - 1)) == 0;   // the lane that stores a group's dot product

    const long long stride = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    for (long long task = static_cast<long long>(blockIdx.x) * kWarpsPerCta + warp;
         task < p.ntasks; task += stride) {
        // task -> (b, cam, part, anchor); `row` = b * A + anchor indexes out / grad_out / loc / wts
        const long long per_b = static_cast<long long>(p.cams) * p.nparts * p.A;
        const uint32_t b = static_cast<uint32_t>(task / per_b);
        const int rem = static_cast<int>(task - static_cast<long long>(b) * per_b);
        const int anchor = rem % p.A;
        const int part = (rem / p.A) % p.nparts;
        const int cam = rem / (p.A * p.nparts);
        const long long row = static_cast<long long>(b) * p.A + anchor;
        const int pt0 = part * p.ppt;
        const int ns = min(p.ppt, p.Pts - pt0) * p.scales;   // samples of this task
        float acc[NV][VEC];
        float go[NV][VEC];
#pragma unroll
        for (int k = 0; k < NV; ++k)
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[k][e] = 0.f;
        if constexpr (BACKWARD) {
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                if constexpr (!SCALAR) {
                    const float4 t = *reinterpret_cast<const float4*>(
                        p.grad_out + row * p.C + (j + k * LPR) * 4);
                    go[k][0] = t.x; go[k][1] = t.y; go[k][2] = t.z; go[k][3] = t.w;
                } else {
                    const int c = j + 32 * k;
                    go[k][0] = (c < p.C) ? p.grad_out[row * p.C + c] : 0.f;
                }
            }
        }

        {
            // ---- phase 1: lane = sample ---------------------------------------------
            const bool active = lane < ns;
            uint4 rec01 = make_uint4(kNoRow, 0u, kNoRow, 0u);
            uint4 rec23 = rec01;
            SampleGeom geom;
            geom.lw = geom.lh = geom.a = geom.wf = geom.hf = geom.prob = 0.f;
            geom.valid = false;
            int pc = 0, scale = 0;
            if (active) {
                scale = lane % p.scales;
                pc = (pt0 + lane / p.scales) * p.cams + cam;   // pts * cams + cam
                const int map = cam * p.scales + scale;
                const long long li = (row * p.Pts * p.cams + pc) * 2;
                const float lw_n = p.loc[li];
                const float lh_n = p.loc[li + 1];
                const bool inside = (lw_n > 0.f) && (lw_n < 1.f) && (lh_n > 0.f) && (lh_n < 1.f);
                if (inside) {
                    const uint32_t row_base = b * static_cast<uint32_t>(p.F) +
                                              static_cast<uint32_t>(s_lv[2][map]);
                    sample_setup(lw_n, lh_n, 1.f, s_lv[1][map], s_lv[0][map], row_base, 1u,
                                 p.row_units, rec01, rec23, geom);
                }
            }
            uint4* dst = reinterpret_cast<uint4*>(s_slot) + 2 * lane;
            dst[0] = rec01;
            dst[1] = rec23;
            // the weights of one (point, camera) are scales * G contiguous floats
            const int per_pt = p.scales * G;
            for (int i = lane; i < ns * G; i += 32) {
                const int ptl = i / per_pt;
                s_wt[i] = p.wts[((row * p.Pts + pt0 + ptl) * p.cams + cam) * per_pt + (i - ptl * per_pt)];
            }
            if constexpr (BACKWARD && SCALAR) {
                for (int i = lane; i < kChunk * astride; i += 32) s_A[i] = 0.f;
            }
            __syncwarp();

            // ---- phase 2: lane = (row slot, piece of row) -----------------------------
            const int slot_end = 4 * ns;
#pragma unroll 1
            for (int base = 0; base < slot_end; base += STEP) {
                const uint2* sp = s_slot + base + g;
                uint2 rec[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) rec[u] = sp[u * RPI];
                if constexpr (!SCALAR) {
                    uint4 raw[UNROLL][NV];
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
                        for (int k = 0; k < NV; ++k) {
                            raw[u][k] = make_uint4(0u, 0u, 0u, 0u);
                            if (rec[u].x != kNoRow)
                                raw[u][k] = ldg16(vlane + static_cast<size_t>(rec[u].x) * 16 +
                                                  k * (LPR * 16));
                        }
                    }
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) {
                        const int slot = base + u * RPI + g;
                        const int sl = min(slot >> 2, kChunk - 1);
                        const float bw = __uint_as_float(rec[u].y);
#pragma unroll
                        for (int k = 0; k < NV; ++k) {
                            float f[4];
                            unpack16<float>(raw[u][k], f);
                            // a slot without a row may sit past the staged weights: never
                            // let whatever is there (possibly NaN bits) into the product
                            const float w =
                                (rec[u].x != kNoRow) ? bw * s_wt[sl * G + grp[k]] : 0.f;
                            if constexpr (!BACKWARD) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) acc[k][e] = fmaf(w, f[e], acc[k][e]);
                            } else {
                                float part = 0.f;
#pragma unroll
                                for (int e = 0; e < 4; ++e) part = fmaf(f[e], go[k][e], part);
                                if (rec[u].x != kNoRow) {
                                    red_add_f32x4(reinterpret_cast<float*>(
                                                      glane + static_cast<size_t>(rec[u].x) * 16 +
                                                      k * (LPR * 16)),
                                                  w * go[k][0], w * go[k][1], w * go[k][2],
                                                  w * go[k][3]);
                                }
                                // sum over the lanes that hold this group's pieces of the row
#pragma unroll
                                for (int off = 16; off >= 1; off >>= 1)
                                    if (off < lpg) part += __shfl_xor_sync(0xffffffffu, part, off);
                                if (slot < slot_end && group_writer)
                                    s_A[sl * astride + (slot & 3) * G + grp[k]] = part;
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) {
                        const int slot = base + u * RPI + g;
                        const int sl = min(slot >> 2, kChunk - 1);
                        const float bw = __uint_as_float(rec[u].y);
#pragma unroll
                        for (int k = 0; k < NV; ++k) {
                            const int c = j + 32 * k;
                            if (rec[u].x != kNoRow && c < p.C) {
                                const size_t idx = static_cast<size_t>(rec[u].x) + c;
                                const float v = __ldg(p.feat + idx);
                                const float w = bw * s_wt[sl * G + grp[k]];
                                if constexpr (!BACKWARD) {
                                    acc[k][0] = fmaf(w, v, acc[k][0]);
                                } else {
                                    atomicAdd(p.grad_feat + idx, w * go[k][0]);
                                    atomicAdd(&s_A[sl * astride + (slot & 3) * G + grp[k]],
                                              v * go[k][0]);
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();

            // ---- phase 3 (backward): lane = sample ------------------------------------
            if constexpr (BACKWARD) {
                float g_w = 0.f, g_h = 0.f;
                if (active) {
                    const float lw = geom.lw, lh = geom.lh;
                    const float hw = 1.f - lw, hh = 1.f - lh;
                    const float b1 = hh * hw, b2 = hh * lw, b3 = lh * hw, b4 = lh * lw;
                    float T1 = 0.f, T2 = 0.f, T3 = 0.f, T4 = 0.f;
                    float* gw = p.grad_wts + ((row * p.Pts * p.cams + pc) * p.scales + scale) * G;
                    const float* A = s_A + lane * astride;
                    for (int q = 0; q < G; ++q) {
                        float a1 = 0.f, a2 = 0.f, a3 = 0.f, a4 = 0.f;
                        if (geom.valid) {
                            // corners that do not exist were never visited: read as zero
                            const uint2* r = s_slot + 4 * lane;
                            a1 = (r[0].x != kNoRow) ? A[q] : 0.f;
                            a2 = (r[1].x != kNoRow) ? A[G + q] : 0.f;
                            a3 = (r[2].x != kNoRow) ? A[2 * G + q] : 0.f;
                            a4 = (r[3].x != kNoRow) ? A[3 * G + q] : 0.f;
                        }
                        gw[q] = b1 * a1 + b2 * a2 + b3 * a3 + b4 * a4;
                        const float wt = s_wt[lane * G + q];
                        T1 = fmaf(wt, a1, T1);
                        T2 = fmaf(wt, a2, T2);
                        T3 = fmaf(wt, a3, T3);
                        T4 = fmaf(wt, a4, T4);
                    }
                    if (geom.valid) {
                        g_w = geom.wf * (hh * (T2 - T1) + lh * (T4 - T3));
                        g_h = geom.hf * (hw * (T3 - T1) + lw * (T4 - T2));
                    }
                }
                // sum over the scales of one (pts, cam): `scales` consecutive lanes
                float sum_w = g_w, sum_h = g_h;
                for (int d = 1; d < p.scales; ++d) {
                    const float ow = __shfl_down_sync(0xffffffffu, g_w, d);
                    const float oh = __shfl_down_sync(0xffffffffu, g_h, d);
                    if (lane + d < 32) {
                        sum_w += ow;
                        sum_h += oh;
                    }
                }
                if (active && scale == 0) {
                    const long long li = (row * p.Pts * p.cams + pc) * 2;
                    p.grad_loc[li] = sum_w;
                    p.grad_loc[li + 1] = sum_h;
                }
                __syncwarp();
            }
        }

        if constexpr (!BACKWARD) {
#pragma unroll
            for (int k = 0; k < NV; ++k) {
#pragma unroll
                for (int off = LPR; off < 32; off <<= 1) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e)
                        acc[k][e] += __shfl_xor_sync(0xffffffffu, acc[k][e], off);
                }
                if (g == 0) {
                    if constexpr (!SCALAR) {
                        red_add_f32x4(p.out + row * p.C + (j + k * LPR) * 4, acc[k][0], acc[k][1],
                                      acc[k][2], acc[k][3]);
                    } else {
                        const int c = j + 32 * k;
                        if (c < p.C) atomicAdd(p.out + row * p.C + c, acc[k][0]);
                    }
                }
            }
        }
    }
}

template <bool BACKWARD>
static cudaError_t da_launch(const DaParams& p, bool scalar, int lpr, int nv, int sm_count,
                             cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(p.warp_smem) * kWarpsPerCta;
    auto go = [&](auto kern) -> cudaError_t {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(smem));
            if (e != cudaSuccess) return e;
        }
        int per_sm = 1;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern,
                                                                      kThreadsPerCta, smem);
        if (e != cudaSuccess) return e;
        if (per_sm < 1) per_sm = 1;
        const long long need = (p.ntasks + kWarpsPerCta - 1) / kWarpsPerCta;
        const long long cap = static_cast<long long>(sm_count) * per_sm;
        const int grid = static_cast<int>(need < cap ? need : cap);
        kern<<<grid, kThreadsPerCta, smem, stream>>>(p);
        return cudaGetLastError();
    };
    if (scalar) return go(da_kernel<32, 8, true, BACKWARD>);
    switch (lpr * 100 + nv) {
        case 101: return go(da_kernel<1, 1, false, BACKWARD>);
        case 201: return go(da_kernel<2, 1, false, BACKWARD>);
        case 401: return go(da_kernel<4, 1, false, BACKWARD>);
        case 801: return go(da_kernel<8, 1, false, BACKWARD>);
        case 1601: return go(da_kernel<16, 1, false, BACKWARD>);
        case 3201: return go(da_kernel<32, 1, false, BACKWARD>);
        case 3202: return go(da_kernel<32, 2, false, BACKWARD>);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace msda

namespace {

using msda::DaParams;
thread_local int t_da_cuda_error = 0;

bool is_pow2(long long v) { return v > 0 && (v & (v - 1)) == 0; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int da_common(DaParams& p, const void* feat, const int32_t* shapes, const int32_t* starts,
              const void* loc, const void* wts, int B, int F, int C, int A, int Pts, int cams,
              int scales, int G, bool* scalar, int* lpr, int* nv, int* sm_count, bool vec_ptrs) {
    if (!feat || !shapes || !starts || !loc || !wts) return MSDA_ERR_NULL;
    if (B <= 0 || F <= 0 || C <= 0 || A <= 0 || Pts <= 0 || cams <= 0 || scales <= 0 || G <= 0)
        return MSDA_ERR_DIMS;
    if (C > 256 || G > msda::kDaMaxGroups || C % G != 0 || scales > 32 ||
        cams * scales > msda::kDaMaxMaps)
        return MSDA_ERR_LIMIT;
    const long long rows = static_cast<long long>(B) * F;
    if (rows >= (1LL << 31) || static_cast<long long>(B) * A >= (1LL << 31)) return MSDA_ERR_LIMIT;
    std::memset(&p, 0, sizeof(p));
    p.feat = static_cast<const float*>(feat);
    p.loc = static_cast<const float*>(loc);
    p.wts = static_cast<const float*>(wts);
    p.B = B; p.F = F; p.C = C; p.A = A; p.Pts = Pts; p.cams = cams; p.scales = scales; p.G = G;
    p.S = Pts * cams * scales;
    p.ppt = msda::kChunk / scales;
    p.nparts = (Pts + p.ppt - 1) / p.ppt;
    p.cpg = C / G;
    p.ntasks = static_cast<long long>(B) * cams * p.nparts * A;

    // both level arrays on the host or both on the device
    auto on_device = [](const void* ptr) {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
    };
    const bool on_dev = on_device(shapes);
    if (on_dev != on_device(starts)) return MSDA_ERR_ALIGN;
    if (on_dev) {
        p.use_table = 0;
        p.shapes_dev = shapes;
        p.starts_dev = starts;
    } else {
        p.use_table = 1;
        for (int i = 0; i < cams * scales; ++i) {
            p.lv_h[i] = shapes[2 * i];
            p.lv_w[i] = shapes[2 * i + 1];
            p.lv_start[i] = starts[i];
            if (p.lv_h[i] <= 0 || p.lv_w[i] <= 0 || p.lv_start[i] < 0 ||
                static_cast<long long>(p.lv_start[i]) +
                        static_cast<long long>(p.lv_h[i]) * p.lv_w[i] > F)
                return MSDA_ERR_DIMS;
        }
    }
    // vector path: the row is 2^k pieces of 16 bytes, a piece never straddles two groups, and
    // a group's pieces sit in one pass over the lanes (at most 32 pieces = 128 channels per
    // group: the backward keeps one dot product per (slot, group) and pass)
    const long long pieces = C / 4;
    *scalar = !(vec_ptrs && C % 4 == 0 && is_pow2(pieces) && pieces <= 64 && p.cpg % 4 == 0 &&
                is_pow2(p.cpg / 4) && p.cpg <= 128);
    *lpr = 32;
    *nv = 8;
    if (!*scalar) {
        *lpr = pieces < 32 ? static_cast<int>(pieces) : 32;
        *nv = static_cast<int>(pieces) / *lpr;
    }
    const unsigned long long units = *scalar ? static_cast<unsigned long long>(C)
                                             : static_cast<unsigned long long>(pieces);
    if (static_cast<unsigned long long>(rows) * units >= 0xffffffffull) return MSDA_ERR_LIMIT;
    p.row_units = static_cast<uint32_t>(units);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
        t_da_cuda_error = static_cast<int>(e);
        return MSDA_ERR_CUDA;
    }
    return MSDA_OK;
}

}  // namespace

extern "C" {

int da_sm100_forward(const void* feat, const int32_t* spatial_shape, const int32_t* scale_start,
                     const void* sampling_location, const void* weights, void* out, int B, int F,
                     int C, int A, int Pts, int cams, int scales, int G, void* stream) {
    if (!out) return MSDA_ERR_NULL;
    DaParams p;
    bool scalar;
    int lpr, nv, sms = 0;
    const int rc = da_common(p, feat, spatial_shape, scale_start, sampling_location, weights, B, F,
                             C, A, Pts, cams, scales, G, &scalar, &lpr, &nv, &sms,
                             aligned16(feat) && aligned16(out));
    if (rc != MSDA_OK) return rc;
    p.out = static_cast<float*>(out);
    p.warp_smem = msda::da_warp_smem(G, false);
    cudaError_t e = cudaMemsetAsync(out, 0, static_cast<size_t>(B) * A * C * sizeof(float),
                                    static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess)
        e = msda::da_launch<false>(p, scalar, lpr, nv, sms, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        t_da_cuda_error = static_cast<int>(e);
        return MSDA_ERR_CUDA;
    }
    msda::count_launches(1);
    return MSDA_OK;
}

int da_sm100_backward(const void* feat, const int32_t* spatial_shape, const int32_t* scale_start,
                      const void* sampling_location, const void* weights, const void* grad_out,
                      void* grad_feat, void* grad_sampling_location, void* grad_weights, int B,
                      int F, int C, int A, int Pts, int cams, int scales, int G, void* stream_v) {
    if (!grad_out || !grad_feat || !grad_sampling_location || !grad_weights) return MSDA_ERR_NULL;
    DaParams p;
    bool scalar;
    int lpr, nv, sms = 0;
    const int rc = da_common(p, feat, spatial_shape, scale_start, sampling_location, weights, B, F,
                             C, A, Pts, cams, scales, G, &scalar, &lpr, &nv, &sms,
                             aligned16(feat) && aligned16(grad_out) && aligned16(grad_feat));
    if (rc != MSDA_OK) return rc;
    p.grad_out = static_cast<const float*>(grad_out);
    p.grad_feat = static_cast<float*>(grad_feat);
    p.grad_loc = static_cast<float*>(grad_sampling_location);
    p.grad_wts = static_cast<float*>(grad_weights);
    p.warp_smem = msda::da_warp_smem(G, true);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    cudaError_t e = cudaMemsetAsync(grad_feat, 0, static_cast<size_t>(B) * F * C * sizeof(float),
                                    stream);
    if (e == cudaSuccess) e = msda::da_launch<true>(p, scalar, lpr, nv, sms, stream);
    if (e != cudaSuccess) {
        t_da_cuda_error = static_cast<int>(e);
        return MSDA_ERR_CUDA;
    }
    msda::count_launches(1);
    return MSDA_OK;
}

int da_sm100_last_cuda_error(void) { return t_da_cuda_error; }

}  // extern "C"

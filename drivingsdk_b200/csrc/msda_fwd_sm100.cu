// MSDA forward for sm_100a: out[b,q,h,:] = sum over (level, point) of
// attention * bilinear(value[b, level], location), zero outside the level.
// Replaces the reference's forward device kernel and its host tiling
// (kernels/multi_scale_deformable_attn/op_kernel/multi_scale_deformable_attn.cpp:116-250,
//  op_host/multi_scale_deformable_attn.cpp:32-114).
//
// One warp per (batch, query, head) task (several tasks per warp when L*P < 32).
//   phase 1  lane = sample: read (x, y, weight) — from the bulk-copied shared
//            tile or straight from global memory — and leave, per corner, the
//            value row index (or -1) and the combined weight in shared memory.
//   phase 2  lane = (row slot, 16-byte piece of the row): the warp reads
//            32/LPR whole rows per instruction (LPR lanes x 16 bytes = one
//            contiguous row), several instructions in flight, and accumulates
//            in fp32 registers.
//   epilogue the row-slot groups are summed with xor shuffles and one group
//            writes the D outputs as 16-byte stores.
// Rows whose byte length is not 16 * 2^k take the SCALAR instantiation: lane =
// channel (mod 32), one row per instruction.
#include "msda_launch.h"
#include "msda_tile.cuh"

namespace msda {

template <typename T, int LPR, int NV, bool SCALAR>
__global__ void __launch_bounds__(kThreadsPerCta)
msda_fwd_kernel(const __grid_constant__ Params p) {
    constexpr int VEC = SCALAR ? 1 : Elem<T>::kVec;
    constexpr int RPI = 32 / LPR;                  // rows per warp instruction
    constexpr int UNROLL = (RPI >= 16) ? 2 : ((NV > 2) ? 4 : 8);

    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane / LPR;   // row slot within one instruction
    const int j = lane % LPR;   // 16-byte piece (or channel mod 32) within the row

    Stage<T> st = stage_init<T>(p, smem);
    unsigned char* warp_base =
        smem + (p.stage ? stage_smem_bytes(p.tasks_per_item, p.LP, sizeof(T)) : 0);
    warp_base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(warp_base) + 15) & ~uintptr_t(15));
    int* s_rows = reinterpret_cast<int*>(warp_base) + warp * 2 * kSlots;
    float* s_wts = reinterpret_cast<float*>(s_rows + kSlots);

    const LaneLevels lv = load_lane_levels(p, lane);
    const T* __restrict__ value = static_cast<const T*>(p.value);
    const T* __restrict__ gloc = static_cast<const T*>(p.loc);
    const T* __restrict__ gattn = static_cast<const T*>(p.attn);
    T* __restrict__ out = static_cast<T*>(p.out);

    const int TPC = p.tasks_per_item;
    const int LP = p.LP;
    const int D = p.D;
    const int nchunks = (TPC == 1) ? (LP + kChunk - 1) / kChunk : 1;
    const int QH = p.Q * p.H;
    const long long ntiles = (p.nitems + kWarpsPerCta - 1) / kWarpsPerCta;

    bool stage_ok = st.enabled;
    if (stage_ok && threadIdx.x == 0 && blockIdx.x < ntiles && st.full(blockIdx.x)) {
        st.issue(p, blockIdx.x, 0);
    }

    int iter = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++iter) {
        const int buf = iter & 1;
        bool from_smem = false;
        if (stage_ok) {
            const long long next = tile + gridDim.x;
            if (threadIdx.x == 0 && next < ntiles && st.full(next)) st.issue(p, next, buf ^ 1);
            if (st.full(tile)) {
                from_smem = mbar_wait(st.bar + buf, (iter >> 1) & 1);
                if (!from_smem) {
                    stage_ok = false;
                    atomicOr(p.status, kStatusStageTimeout);
                }
            }
        }

        const T* sloc = st.loc(buf);
        const T* sattn = st.attn(buf);
        const long long item = tile * kWarpsPerCta + warp;
        if (item < p.nitems) {
            const int t0 = static_cast<int>(item) * TPC;
            const int ntask_here = min(TPC, static_cast<int>(p.ntasks - t0));
            float acc[NV][VEC];

            for (int chunk = 0; chunk < nchunks; ++chunk) {
                // ---- phase 1: lane = sample -------------------------------------
                int tl, s;
                lane_sample_index(p, chunk, lane, tl, s);
                const bool active = (tl < ntask_here) && (s < LP);
                int4 rows = make_int4(-1, -1, -1, -1);
                float4 wts = make_float4(0.f, 0.f, 0.f, 0.f);
                if (active) {
                    const int t = t0 + tl;
                    float lx, ly, a;
                    if (from_smem) {
                        const int li = (warp * TPC + tl) * LP + s;
                        lx = Elem<T>::to_f(sloc[2 * li]);
                        ly = Elem<T>::to_f(sloc[2 * li + 1]);
                        a = Elem<T>::to_f(sattn[li]);
                    } else {
                        const long long gi = static_cast<long long>(t) * LP + s;
                        lx = Elem<T>::to_f(gloc[2 * gi]);
                        ly = Elem<T>::to_f(gloc[2 * gi + 1]);
                        a = Elem<T>::to_f(gattn[gi]);
                    }
                    const int b = t / QH;
                    const int h = t % p.H;
                    const int c = (TPC == 1) ? chunk : 0;
                    const int row_base = (b * p.K + lv.start(c)) * p.H + h;
                    SampleGeom geom;
                    sample_setup(lx, ly, a, lv.w(c), lv.h(c), row_base, p.H, rows, wts, geom);
                }
                reinterpret_cast<int4*>(s_rows)[lane] = rows;
                reinterpret_cast<float4*>(s_wts)[lane] = wts;
                __syncwarp();

                // ---- phase 2: lane = (row slot, piece of row) -------------------
                for (int tl2 = 0; tl2 < ntask_here; ++tl2) {
                    int slot_begin, slot_end;
                    if (TPC == 1) {
                        slot_begin = 0;
                        slot_end = 4 * min(kChunk, LP - chunk * kChunk);
                    } else {
                        slot_begin = tl2 * 4 * LP;
                        slot_end = slot_begin + 4 * LP;
                    }
                    if (chunk == 0) {
#pragma unroll
                        for (int k = 0; k < NV; ++k)
#pragma unroll
                            for (int e = 0; e < VEC; ++e) acc[k][e] = 0.f;
                    }
#pragma unroll 1
                    for (int base = slot_begin; base < slot_end; base += RPI * UNROLL) {
                        int r[UNROLL];
                        float w[UNROLL];
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u) {
                            const int slot = base + u * RPI + g;
                            const bool in = slot < slot_end;
                            r[u] = in ? s_rows[slot] : -1;
                            w[u] = in ? s_wts[slot] : 0.f;
                        }
                        if constexpr (!SCALAR) {
                            uint4 raw[UNROLL][NV];
#pragma unroll
                            for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
                                for (int k = 0; k < NV; ++k) {
                                    raw[u][k] = make_uint4(0u, 0u, 0u, 0u);
                                    if (r[u] >= 0) {
                                        raw[u][k] = ldg16(value + static_cast<size_t>(r[u]) * D +
                                                          (j + k * LPR) * VEC);
                                    }
                                }
                            }
#pragma unroll
                            for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
                                for (int k = 0; k < NV; ++k) {
                                    float f[Elem<T>::kVec];
                                    unpack16<T>(raw[u][k], f);
#pragma unroll
                                    for (int e = 0; e < VEC; ++e)
                                        acc[k][e] = fmaf(w[u], f[e], acc[k][e]);
                                }
                            }
                        } else {
                            float f[UNROLL][NV];
#pragma unroll
                            for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
                                for (int k = 0; k < NV; ++k) {
                                    const int c = j + k * 32;
                                    f[u][k] = 0.f;
                                    if (r[u] >= 0 && c < D) {
                                        f[u][k] = Elem<T>::to_f(
                                            __ldg(value + static_cast<size_t>(r[u]) * D + c));
                                    }
                                }
                            }
#pragma unroll
                            for (int u = 0; u < UNROLL; ++u)
#pragma unroll
                                for (int k = 0; k < NV; ++k)
                                    acc[k][0] = fmaf(w[u], f[u][k], acc[k][0]);
                        }
                    }

                    // ---- epilogue ----------------------------------------------
                    if (chunk == nchunks - 1) {
                        const size_t obase = static_cast<size_t>(t0 + tl2) * D;
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
                                    float f[VEC];
#pragma unroll
                                    for (int e = 0; e < VEC; ++e) f[e] = acc[k][e];
                                    *reinterpret_cast<uint4*>(out + obase + (j + k * LPR) * VEC) =
                                        pack16<T>(f);
                                } else {
                                    const int c = j + k * 32;
                                    if (c < D) out[obase + c] = Elem<T>::from_f(acc[k][0]);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
            }
        }
        if (st.enabled) __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// host side: instantiation table and launch
// ---------------------------------------------------------------------------
template <typename T, int LPR, int NV, bool SCALAR>
static cudaError_t launch_fwd_inst(const Params& p, int grid, size_t smem, cudaStream_t stream) {
    auto kern = msda_fwd_kernel<T, LPR, NV, SCALAR>;
    if (smem > 48 * 1024) {
        cudaError_t e =
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    kern<<<grid, kThreadsPerCta, smem, stream>>>(p);
    return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_fwd_typed(const Params& p, const RowPlan& rp, int grid, size_t smem,
                                    cudaStream_t stream) {
    if (rp.scalar) return launch_fwd_inst<T, 32, 8, true>(p, grid, smem, stream);
    switch (rp.lpr * 100 + rp.nv) {
        case 101: return launch_fwd_inst<T, 1, 1, false>(p, grid, smem, stream);
        case 201: return launch_fwd_inst<T, 2, 1, false>(p, grid, smem, stream);
        case 401: return launch_fwd_inst<T, 4, 1, false>(p, grid, smem, stream);
        case 801: return launch_fwd_inst<T, 8, 1, false>(p, grid, smem, stream);
        case 1601: return launch_fwd_inst<T, 16, 1, false>(p, grid, smem, stream);
        case 3201: return launch_fwd_inst<T, 32, 1, false>(p, grid, smem, stream);
        case 3202: return launch_fwd_inst<T, 32, 2, false>(p, grid, smem, stream);
        default: return cudaErrorInvalidValue;
    }
}

size_t fwd_smem_bytes(const Params& p, size_t elem) {
    size_t s = p.stage ? stage_smem_bytes(p.tasks_per_item, p.LP, elem) : 0;
    s = (s + 15) & ~size_t(15);
    return s + static_cast<size_t>(kWarpsPerCta) * 2 * kSlots * 4 + 16;
}

cudaError_t launch_forward(const Params& p, int dtype, const RowPlan& rp, int grid,
                           cudaStream_t stream) {
    switch (dtype) {
        case 0: return launch_fwd_typed<float>(p, rp, grid, fwd_smem_bytes(p, 4), stream);
        case 1: return launch_fwd_typed<__half>(p, rp, grid, fwd_smem_bytes(p, 2), stream);
        case 2: return launch_fwd_typed<__nv_bfloat16>(p, rp, grid, fwd_smem_bytes(p, 2), stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace msda

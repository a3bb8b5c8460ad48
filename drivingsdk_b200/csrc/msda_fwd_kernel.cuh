// Forward kernel template and its launch table, shared by the bilinear operator (MSDA,
// CPS = 4 corners per sample) and the nearest-pixel operator (geometric kernel attention,
// CPS = 1). Included by one .cu file per operator so that the two sets of instantiations
// compile side by side.
#pragma once

#include <type_traits>

#include "msda_launch.h"
#include "msda_tile.cuh"

// Compile-time tuning, chosen by measurement on B200 (BEVFormer / Deformable-DETR shapes):
// four resident CTAs per SM (64 registers per thread, no spills) with four row loads in
// flight per lane beat both deeper unrolling (spills) and more CTAs (fewer registers).
#ifndef MSDA_FWD_MIN_CTAS
#define MSDA_FWD_MIN_CTAS 4
#endif
#ifndef MSDA_FWD_UNROLL
#define MSDA_FWD_UNROLL 4
#endif

namespace msda {

// PACK (bilinear sampling, vector rows): phase 1 leaves records only for the corners that
// exist, so the gather loop neither issues nor predicates anything for the others
// (BEVFormer shape, 18 % of the corners outside the image: 146 -> 132 us).
template <typename T, int LPR, int NV, bool SCALAR, int MODE, bool PACK>
__global__ void __launch_bounds__(kThreadsPerCta, (SCALAR || NV > 1) ? 2 : MSDA_FWD_MIN_CTAS)
msda_fwd_kernel(const __grid_constant__ Params p) {
    static_assert(!PACK || (MODE != kModeNearest && !SCALAR),
                  "packing is for the bilinear vector kernels");
    constexpr int CPS = (MODE == kModeFused) ? 4 : MODE;   // rows (corners) per sample
    constexpr bool FUSED = MODE == kModeFused;
    constexpr int VEC = SCALAR ? 1 : Elem<T>::kVec;
    constexpr int RPI = 32 / LPR;                  // rows per warp instruction
    constexpr int UNROLL =
        (RPI >= 16) ? 2 : ((NV > 2) ? 4 : MSDA_FWD_UNROLL);
    constexpr int STEP = RPI * UNROLL;             // slots per trip of the gather loop
    static_assert(kSlots % STEP == 0 && STEP <= kSlotPad, "slot loop must tile the slots");

    if (!device_level_table_ok(p)) return;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane / LPR;   // row slot within one instruction
    const int j = lane % LPR;   // 16-byte piece (or channel mod 32) within the row

    unsigned char* wb = smem + static_cast<size_t>(warp) * p.warp_smem;
    uint2* s_slot = reinterpret_cast<uint2*>(wb);
    init_unused_slots<CPS>(s_slot, lane);
    WarpStage<T> st = warp_stage_init<T>(p, wb + kSlotBytes, lane);

    const LaneLevels lv = load_lane_levels(p, lane);
    const T* __restrict__ value = static_cast<const T*>(p.value);
    const unsigned char* vlane = static_cast<const unsigned char*>(p.value) + j * 16;
    T* __restrict__ out = static_cast<T*>(p.out);

    const int TPC = p.tasks_per_item;
    const int LP = p.LP;
    const int D = p.D;
    const int nchunks = (TPC == 1) ? (LP + kChunk - 1) / kChunk : 1;
    ItemWalk walk = make_walk(p, warp);
    auto full = [&](long long it) { return (it + 1) * TPC <= p.ntasks; };

    if (st.ok && lane == 0 && walk.idx < walk.end && full(walk.item(p))) {
        st.issue(p, walk.item(p), 0);
    }

    for (int n = 0; walk.idx < walk.end; walk.idx += walk.stride, ++n) {
        const int buf = n & 1;
        const long long item = walk.item(p);
        const T* sloc = nullptr;
        const T* sattn = nullptr;
        if (st.ok) {
            const long long next = walk.item_at(p, walk.idx + walk.stride);
            const bool next_issued = walk.idx + walk.stride < walk.end && full(next);
            if (lane == 0 && next_issued) st.issue(p, next, buf ^ 1);
            if (full(item)) {
                const bool arrived =
                    __all_sync(0xffffffffu,
                               mbar_wait(st.bar + buf, (n >> 1) & 1, p.spin_limit) ? 1 : 0) != 0;
                if (arrived) {
                    sloc = st.loc(p, buf);
                    sattn = st.attn(p, buf);
                } else {
                    // give up staging for good, report it, let the copies in flight land,
                    // and carry on with direct loads
                    st.ok = false;
                    if (lane == 0) atomicOr(p.status, kStatusStageTimeout);
                    st.drain(buf, n, next_issued);
                }
            }
        }

        const int t0 = static_cast<int>(item) * TPC;
        const int ntask_here = min(TPC, static_cast<int>(p.ntasks - t0));
        float acc[NV][VEC];

        for (int chunk = 0; chunk < nchunks; ++chunk) {
            // ---- phase 1: lane = sample -----------------------------------------
            SampleGeom geom;
            long long gi;
            Compaction packed;
            packed.rows = 0;
            phase1<T, CPS, FUSED>(p, lv, chunk, lane, item, ntask_here, sloc, sattn, s_slot, geom,
                                  gi, PACK ? &packed : nullptr);
            __syncwarp();

            // ---- phase 2: lane = (row slot, piece of row) -----------------------
            for (int tl2 = 0; tl2 < ntask_here; ++tl2) {
                int slot_begin, slot_end, unguarded_end;
                if constexpr (PACK) {
                    // only existing rows have records: a task's begin where its first
                    // sample's would, and end where the next task's begin; what follows them
                    // is another task's or stale, so the last trip is guarded
                    if (TPC == 1) {
                        slot_begin = 0;
                        slot_end = packed.rows;
                    } else {
                        const int next = (tl2 + 1) * LP;   // first lane of the next task
                        slot_begin = __shfl_sync(0xffffffffu, packed.first, tl2 * LP);
                        const int e = __shfl_sync(0xffffffffu, packed.first, min(next, 31));
                        slot_end = next < 32 ? e : packed.rows;
                    }
                    unguarded_end = slot_end - STEP + 1;
                } else if (TPC == 1) {
                    // slots past the last sample hold "no row" records: no guard needed
                    slot_begin = 0;
                    slot_end = CPS * min(kChunk, LP - chunk * kChunk);
                    unguarded_end = slot_end;
                } else {
                    // slots past slot_end belong to the next task: the last trip is guarded
                    slot_begin = tl2 * CPS * LP;
                    slot_end = slot_begin + CPS * LP;
                    unguarded_end = slot_end - STEP + 1;
                }
                if (chunk == 0) {
#pragma unroll
                    for (int k = 0; k < NV; ++k)
#pragma unroll
                        for (int e = 0; e < VEC; ++e) acc[k][e] = 0.f;
                }

                auto gather = [&](int base, auto unroll_tag, auto guarded_tag, auto present_tag) {
                    constexpr int U = decltype(unroll_tag)::value;   // rows in flight per lane
                    constexpr bool GUARDED = decltype(guarded_tag)::value;
                    constexpr bool PRESENT = decltype(present_tag)::value;   // every record has a row
                    const uint2* sp = s_slot + base + g;
                    uint2 rec[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        rec[u] = sp[u * RPI];
                        // (with packed records what lies behind the last one is stale, weight
                        // included)
                        if (GUARDED && base + u * RPI + g >= slot_end)
                            rec[u] = make_uint2(kNoRow, 0u);
                    }
                    if constexpr (!SCALAR) {
                        // A missing corner loads nothing and reads as zeros (its weight is
                        // zero as well, so it adds nothing — and no 0 * NaN can arise).
                        uint4 raw[U][NV];
#pragma unroll
                        for (int u = 0; u < U; ++u) {
#pragma unroll
                            for (int k = 0; k < NV; ++k) {
                                if constexpr (PRESENT) {
                                    raw[u][k] = ldg16(vlane + static_cast<size_t>(rec[u].x) * 16 +
                                                      k * (LPR * 16));
                                } else {
                                    raw[u][k] = make_uint4(0u, 0u, 0u, 0u);
                                    if (rec[u].x != kNoRow)
                                        raw[u][k] = ldg16(vlane +
                                                          static_cast<size_t>(rec[u].x) * 16 +
                                                          k * (LPR * 16));
                                }
                            }
                        }
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const float w = __uint_as_float(rec[u].y);
#pragma unroll
                            for (int k = 0; k < NV; ++k) {
                                float f[VEC];
                                unpack16<T>(raw[u][k], f);
#pragma unroll
                                for (int e = 0; e < VEC; e += 2) {
                                    const float2 r =
                                        ffma2(make_float2(w, w), make_float2(f[e], f[e + 1]),
                                              make_float2(acc[k][e], acc[k][e + 1]));
                                    acc[k][e] = r.x;
                                    acc[k][e + 1] = r.y;
                                }
                            }
                        }
                    } else {
                        float f[U][NV];
#pragma unroll
                        for (int u = 0; u < U; ++u) {
#pragma unroll
                            for (int k = 0; k < NV; ++k) {
                                const int c = j + k * 32;
                                f[u][k] = 0.f;
                                if (rec[u].x != kNoRow && c < D) {
                                    f[u][k] = Elem<T>::to_f(
                                        __ldg(value + static_cast<size_t>(rec[u].x) + c));
                                }
                            }
                        }
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const float w = __uint_as_float(rec[u].y);
#pragma unroll
                            for (int k = 0; k < NV; ++k) acc[k][0] = fmaf(w, f[u][k], acc[k][0]);
                        }
                    }
                };

                // full trips, then the rest: a task with few slots left (small L*P) does not
                // pay for instructions that carry no row
                int base = slot_begin;
#pragma unroll 1
                for (; base < unguarded_end; base += STEP)
                    gather(base, std::integral_constant<int, UNROLL>{}, std::false_type{},
                           std::integral_constant<bool, PACK>{});
                if (slot_end - base > 2 * RPI) {
                    // more than two instructions' worth left: one guarded trip at full width
                    // keeps them all in flight (a chain of short trips is latency-bound)
                    gather(base, std::integral_constant<int, UNROLL>{}, std::true_type{},
                           std::false_type{});
                } else {
                    if constexpr (UNROLL > 2) {
                        if (base + 2 * RPI <= slot_end) {
                            gather(base, std::integral_constant<int, 2>{}, std::false_type{},
                                   std::integral_constant<bool, PACK>{});
                            base += 2 * RPI;
                        }
                    }
#pragma unroll 1
                    for (; base < slot_end; base += RPI)
                        gather(base, std::integral_constant<int, 1>{}, std::true_type{},
                               std::false_type{});
                }

                // ---- epilogue ---------------------------------------------------
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
}

// ---------------------------------------------------------------------------
// launch table
// ---------------------------------------------------------------------------
template <typename T, int LPR, int NV, bool SCALAR, int MODE, bool PACK>
static cudaError_t launch_fwd_pack(const Params& p, const LaunchShape& ls, size_t smem,
                                   cudaStream_t stream) {
    auto kern = msda_fwd_kernel<T, LPR, NV, SCALAR, MODE, PACK>;
    if (smem > 48 * 1024) {
        cudaError_t e =
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    int grid = 0;
    cudaError_t e = persistent_grid(reinterpret_cast<const void*>(kern), smem, ls, p, &grid);
    if (e != cudaSuccess) return e;
    kern<<<grid, kThreadsPerCta, smem, stream>>>(p);
    return cudaGetLastError();
}

template <typename T, int LPR, int NV, bool SCALAR, int MODE>
static cudaError_t launch_fwd_inst(const Params& p, const LaunchShape& ls, size_t smem,
                                   cudaStream_t stream) {
    if constexpr (MODE != kModeNearest && !SCALAR) {
        if (p.pack_rows) return launch_fwd_pack<T, LPR, NV, SCALAR, MODE, true>(p, ls, smem, stream);
    }
    return launch_fwd_pack<T, LPR, NV, SCALAR, MODE, false>(p, ls, smem, stream);
}

template <typename T, int MODE>
static cudaError_t launch_fwd_typed(const Params& p, const RowPlan& rp, const LaunchShape& ls, size_t smem,
                                    cudaStream_t stream) {
    if (rp.scalar) return launch_fwd_inst<T, 32, 8, true, MODE>(p, ls, smem, stream);
    switch (rp.lpr * 100 + rp.nv) {
        case 101: return launch_fwd_inst<T, 1, 1, false, MODE>(p, ls, smem, stream);
        case 201: return launch_fwd_inst<T, 2, 1, false, MODE>(p, ls, smem, stream);
        case 401: return launch_fwd_inst<T, 4, 1, false, MODE>(p, ls, smem, stream);
        case 801: return launch_fwd_inst<T, 8, 1, false, MODE>(p, ls, smem, stream);
        case 1601: return launch_fwd_inst<T, 16, 1, false, MODE>(p, ls, smem, stream);
        case 3201: return launch_fwd_inst<T, 32, 1, false, MODE>(p, ls, smem, stream);
        case 3202:
            if constexpr (sizeof(T) == 4) {
                return launch_fwd_inst<T, 32, 2, false, MODE>(p, ls, smem, stream);
            }
            return cudaErrorInvalidValue;
        default: return cudaErrorInvalidValue;
    }
}

template <int MODE>
static cudaError_t launch_forward_cps(const Params& p, int dtype, const RowPlan& rp,
                                      const LaunchShape& ls, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(p.warp_smem) * kWarpsPerCta;
    switch (dtype) {
        case 0: return launch_fwd_typed<float, MODE>(p, rp, ls, smem, stream);
        case 1: return launch_fwd_typed<__half, MODE>(p, rp, ls, smem, stream);
        case 2: return launch_fwd_typed<__nv_bfloat16, MODE>(p, rp, ls, smem, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace msda

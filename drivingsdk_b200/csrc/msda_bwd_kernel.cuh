// Backward kernel template and its launch table, shared by the bilinear operator (MSDA,
// CPS = 4 corners per sample) and the nearest-pixel operator (geometric kernel attention,
// CPS = 1). Included by one .cu file per operator.
#pragma once

#include <type_traits>

#include "msda_launch.h"
#include "msda_tile.cuh"

namespace msda {

// Partial dot products <value row, grad_out> kept per (sample, corner): room for 8 floats; a
// trip that runs in double (see sample_grad) leaves 4 doubles in the same 32 bytes.
constexpr int kPartMax = 8;
constexpr int kPartMaxF64 = 4;
constexpr int kPartBytes = ((kChunk * (4 * kPartMax + 2) * 4 + 15) / 16) * 16;

// Compile-time tuning, chosen by measurement on B200: three resident CTAs per SM (80
// registers per thread) and four rows in flight per lane; the kernel is bound by the rate
// at which L2 retires vector reductions, and more warps in flight made that worse.
#ifndef MSDA_BWD_MIN_CTAS
#define MSDA_BWD_MIN_CTAS 3
#endif
#ifndef MSDA_BWD_UNROLL
#define MSDA_BWD_UNROLL 4
#endif

// Per-sample gradients from the partial dot products S_c = <value row of corner c, grad_out>
// that phase 2 parked in shared memory (`part`: CPS * PART floats of this sample):
//   grad_attn  = w1*S1 + w2*S2 + w3*S3 + w4*S4                (bilinear w, no attention)
//   grad_loc_x = W * attn * (hh*(S2 - S1) + lh*(S4 - S3))
//   grad_loc_y = H * attn * (hw*(S3 - S1) + lw*(S4 - S2))
// (op_kernel/multi_scale_deformable_attn_grad.cpp:215-242), all zero for a dropped sample; a
// corner that does not exist left zero partials behind. For fp32 tensors the sums, the
// differences and the products run in double precision: the differences of the S_c cancel
// and are then multiplied by W * attn (up to ~200), which turns the fp32 rounding of the
// S_c themselves into errors beyond 1e-4 on wide levels (measured on 200-pixel-wide levels
// with N(0,1) values: fp32 dot products miss rtol = atol = 1e-4 on a few samples per million,
// fp32 partial sums added in double still on one). So for fp32 tensors the partial sums are
// doubles from phase 2 on: samples whose amplification max(W, H) * |attention| reaches
// Params::precise_amp accumulate in double from the first product on (phase 2 takes that
// form for the trips they are in; fp32 -> fp64 conversions run at 16 per clock per SM, so
// doing it for every sample costs a quarter more time), the others sum a lane's four to
// eight products in fp32 and widen the result. 16-bit tensors (tolerance 1e-2) keep fp32
// arithmetic throughout.
__device__ __forceinline__ float dot_fma(float v, float g, float acc) { return fmaf(v, g, acc); }
__device__ __forceinline__ double dot_fma(float v, double g, double acc) {
    return fma(static_cast<double>(v), g, acc);
}

struct SampleGrad {
    float attn, x, y;
};
// `part`: this sample's partials, CSTR floats per corner: PART_F fp32 partials, or — when the
// sample's trip ran in double (`wide`) — PART_D doubles in the same place. Acc: the type the
// gradients are formed in (double for the fp32 bilinear operator, else float).
template <typename Acc, int CPS, int PART_F, int PART_D, int CSTR>
__device__ __forceinline__ SampleGrad sample_grad(const float* part, const SampleGeom& geom,
                                                  bool wide) {
    Acc S[CPS];
    if (sizeof(Acc) == 8 && wide) {
#pragma unroll
        for (int c = 0; c < CPS; ++c) {
            double acc = 0.0;
#pragma unroll
            for (int q = 0; q < PART_D; ++q)
                acc += *reinterpret_cast<const double*>(part + c * CSTR + 2 * q);
            S[c] = static_cast<Acc>(acc);
        }
    } else {
        // fp32 partials: summed in fp32 (as accurate as the partials themselves) and widened
        // once per corner — conversions to double are a scarce resource (16 per clock per SM)
#pragma unroll
        for (int c = 0; c < CPS; ++c) {
            float acc = 0.f;
#pragma unroll
            for (int q = 0; q < PART_F; ++q) acc += part[c * CSTR + q];
            S[c] = static_cast<Acc>(acc);
        }
    }
    SampleGrad r{0.f, 0.f, 0.f};
    if constexpr (CPS == 4) {
        if (geom.valid) {
            const Acc lw = geom.lw, lh = geom.lh;
            const Acc hw = Acc(1) - lw, hh = Acc(1) - lh;
            r.attn = static_cast<float>(hh * hw * S[0] + hh * lw * S[1] + lh * hw * S[2] +
                                        lh * lw * S[3]);
            r.x = static_cast<float>(static_cast<Acc>(geom.wf) * static_cast<Acc>(geom.a) *
                                     (hh * (S[1] - S[0]) + lh * (S[3] - S[2])));
            r.y = static_cast<float>(static_cast<Acc>(geom.hf) * static_cast<Acc>(geom.a) *
                                     (hw * (S[2] - S[0]) + lw * (S[3] - S[1])));
        }
    } else {
        r.attn = static_cast<float>(S[0]);
    }
    return r;
}

template <typename T, typename TG, int LPR, int NV, bool SCALAR, int MODE>
__global__ void __launch_bounds__(kThreadsPerCta, (SCALAR || NV > 1) ? 2 : MSDA_BWD_MIN_CTAS)
msda_bwd_kernel(const __grid_constant__ Params p) {
    constexpr int CPS = (MODE == kModeFused) ? 4 : MODE;   // rows (corners) per sample
    constexpr bool FUSED = MODE == kModeFused;
    constexpr int VEC = SCALAR ? 1 : Elem<T>::kVec;
    constexpr int RPI = 32 / LPR;
    // fp32 bilinear operator: dot products may need double precision (see sample_grad)
    constexpr bool WIDE = sizeof(T) == 4 && CPS == 4;
    using Acc = typename std::conditional<WIDE, double, float>::type;
    constexpr int PART_F = (LPR < kPartMax) ? LPR : kPartMax;        // fp32 partials per slot
    constexpr int PART_D = (LPR < kPartMaxF64) ? LPR : kPartMaxF64;  // double partials per slot
    constexpr int CSTR = WIDE ? ((PART_F > 2 * PART_D) ? PART_F : 2 * PART_D) : PART_F;
    // per-sample stride in floats: odd spreads the banks; even where doubles are stored
    constexpr int SSTRIDE = CPS * CSTR + (WIDE ? 2 : 1);
    // 16-bit rows of <= 128 bytes: an instruction already covers >= 4 rows, and the fp32
    // accumulation path carries a second copy of grad_out; two instructions in flight keep
    // the kernel free of register spills (four in flight measured 5 % slower at the
    // BEVFormer shape in bf16 and 12 % slower at the temporal self-attention shape).
    constexpr int UNROLL = (RPI >= 16 || (sizeof(T) == 2 && RPI >= 4)) ? 2 : MSDA_BWD_UNROLL;
    constexpr int STEP = RPI * UNROLL;
    static_assert(kSlots % STEP == 0 && STEP <= kSlotPad, "slot loop must tile the slots");
    // 16-bit operands accumulated in fp32: a lane's 16-byte piece of the value row is 8
    // channels, i.e. 32 bytes of the fp32 accumulation row. Two reductions at +0 and +16
    // bytes of that span would touch every 32-byte sector of the row with half a sector each
    // time; instead lane j adds the float4 pieces j and LPR + j, so each instruction covers
    // whole sectors. The scatter does not depend on the value data, so any lane may add any
    // channels — it only needs grad_out for those channels (gred below).
    constexpr bool SPLIT_RED = !SCALAR && sizeof(T) == 2 && sizeof(TG) == 4;

    if (!device_level_table_ok(p)) return;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane / LPR;
    const int j = lane % LPR;

    unsigned char* wb = smem + static_cast<size_t>(warp) * p.warp_smem;
    uint2* s_slot = reinterpret_cast<uint2*>(wb);
    float* s_part = reinterpret_cast<float*>(wb + kSlotBytes);
    // where this lane's row slot sits inside the partials of its sample (used when an
    // instruction covers whole samples)
    const int part_lane = (g / CPS) * SSTRIDE + (g % CPS) * CSTR;
    init_unused_slots<CPS>(s_slot, lane);
    WarpStage<T> st = warp_stage_init<T>(p, wb + kSlotBytes + kPartBytes, lane);

    const LaneLevels lv = load_lane_levels(p, lane);
    const T* __restrict__ value = static_cast<const T*>(p.value);
    const unsigned char* vlane = static_cast<const unsigned char*>(p.value) + j * 16;
    const T* __restrict__ gout = static_cast<const T*>(p.grad_out);
    TG* __restrict__ gval = static_cast<TG*>(p.grad_value);
    unsigned char* glane = static_cast<unsigned char*>(p.grad_value) + j * 16;

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

        for (int chunk = 0; chunk < nchunks; ++chunk) {
            // ---- phase 1: lane = sample -----------------------------------------
            SampleGeom geom;
            long long gi;
            const bool active =
                phase1<T, CPS, FUSED>(p, lv, chunk, lane, item, ntask_here, sloc, sattn, s_slot,
                                      geom, gi);
            // which samples (bit = lane) want their dot products in double: the location
            // gradient multiplies them by W * attention (H * attention)
            uint32_t m_precise = 0u;
            if constexpr (WIDE) {
                m_precise = __ballot_sync(
                    0xffffffffu, active && geom.valid &&
                                     fmaxf(geom.wf, geom.hf) * fabsf(geom.a) >= p.precise_amp);
            }
            // did the trip that holds this lane's sample run in double? (same rule as `trip`
            // below: trips start at the task's first slot and cover STEP slots)
            auto lane_trip_wide = [&]() -> bool {
                if constexpr (!WIDE) return false;   // fp32 partials
                const int slot = lane * CPS;
                const int begin = (TPC == 1) ? 0 : (slot / (CPS * LP)) * (CPS * LP);
                const int base = begin + ((slot - begin) / STEP) * STEP;
                const int s0 = base / CPS;
                const int s1 = min(32, (base + STEP + CPS - 1) / CPS);
                const uint32_t bits =
                    (s1 - s0 >= 32 ? 0xffffffffu : ((1u << (s1 - s0)) - 1u)) << s0;
                return (m_precise & bits) != 0u;
            };
            __syncwarp();

            // ---- phase 2: lane = (row slot, piece of row) -----------------------
            for (int tl2 = 0; tl2 < ntask_here; ++tl2) {
                int slot_begin, slot_end, unguarded_end;
                if (TPC == 1) {
                    slot_begin = 0;
                    slot_end = CPS * min(kChunk, LP - chunk * kChunk);
                    unguarded_end = slot_end;
                } else {
                    slot_begin = tl2 * CPS * LP;
                    slot_end = slot_begin + CPS * LP;
                    unguarded_end = slot_end - STEP + 1;
                }
                // this lane's piece of grad_out[b, q, h, :]
                float go[NV][VEC];
                const size_t obase = static_cast<size_t>(t0 + tl2) * D;
#pragma unroll
                for (int k = 0; k < NV; ++k) {
                    if constexpr (!SCALAR) {
                        const uint4 raw =
                            *reinterpret_cast<const uint4*>(gout + obase + (j + k * LPR) * VEC);
                        unpack16<T>(raw, go[k]);
                    } else {
                        const int c = j + k * 32;
                        go[k][0] = (c < D) ? Elem<T>::to_f(gout[obase + c]) : 0.f;
                    }
                }
                float gred[2][4];
                if constexpr (SPLIT_RED) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const T* src = gout + obase + (half * LPR + j) * 4;
                        const uint2 raw = *reinterpret_cast<const uint2*>(src);
                        const uint32_t wds[2] = {raw.x, raw.y};
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const uint16_t l16 = static_cast<uint16_t>(wds[i] & 0xffffu);
                            const uint16_t h16 = static_cast<uint16_t>(wds[i] >> 16);
                            gred[half][2 * i] = Elem<T>::to_f(*reinterpret_cast<const T*>(&l16));
                            gred[half][2 * i + 1] =
                                Elem<T>::to_f(*reinterpret_cast<const T*>(&h16));
                        }
                    }
                }

                auto scatter_gather = [&](int base, auto unroll_tag, auto guarded_tag,
                                          auto precise_tag) {
                    constexpr int U = decltype(unroll_tag)::value;   // rows in flight per lane
                    constexpr bool GUARDED = decltype(guarded_tag)::value;
                    // PRECISE: the trip's dot products are accumulated in double from the first
                    // product on; otherwise in the lane's fp32 registers, widened afterwards
                    constexpr bool PRECISE = decltype(precise_tag)::value;
                    using Part = typename std::conditional<PRECISE, double, float>::type;
                    // grad_out in the type of the products (converted once per trip)
                    Part gop[NV][VEC];
#pragma unroll
                    for (int k = 0; k < NV; ++k)
#pragma unroll
                        for (int e = 0; e < VEC; ++e) gop[k][e] = static_cast<Part>(go[k][e]);
                    const uint2* sp = s_slot + base + g;
                    uint2 rec[U];
                    Part part[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        rec[u] = sp[u * RPI];
                        if (GUARDED && base + u * RPI + g >= slot_end) rec[u].x = kNoRow;
                        part[u] = 0;
                    }
                    if constexpr (!SCALAR) {
                        // A missing corner loads row 0 instead of branching around the load;
                        // it is skipped below, so it neither scatters nor contributes.
                        uint4 raw[U][NV];
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const uint32_t off = (rec[u].x != kNoRow) ? rec[u].x : 0u;
#pragma unroll
                            for (int k = 0; k < NV; ++k)
                                raw[u][k] =
                                    ldg16(vlane + static_cast<size_t>(off) * 16 + k * (LPR * 16));
                        }
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            // Straight-line code: the products are formed for every slot and
                            // only the reduction itself is predicated on the row existing
                            // (a branch per row costs more than the wasted multiplies).
                            const bool has_row = rec[u].x != kNoRow;
                            const float w = __uint_as_float(rec[u].y);
                            if constexpr (SPLIT_RED) {
                                float* row = reinterpret_cast<float*>(
                                    glane + static_cast<size_t>(rec[u].x) * 32);
                                if (has_row) {
                                    red_add_f32x4(row, w * gred[0][0], w * gred[0][1],
                                                  w * gred[0][2], w * gred[0][3]);
                                    red_add_f32x4(row + LPR * 4, w * gred[1][0], w * gred[1][1],
                                                  w * gred[1][2], w * gred[1][3]);
                                }
                            } else {
#pragma unroll
                                for (int k = 0; k < NV; ++k) {
                                    float contrib[VEC];
#pragma unroll
                                    for (int e = 0; e < VEC; e += 2) {
                                        const float2 c2 = fmul2(make_float2(w, w),
                                                                make_float2(go[k][e], go[k][e + 1]));
                                        contrib[e] = c2.x;
                                        contrib[e + 1] = c2.y;
                                    }
                                    if (has_row)
                                        red_add_vec<TG, VEC>(
                                            reinterpret_cast<TG*>(
                                                glane + static_cast<size_t>(rec[u].x) * 16 +
                                                k * (LPR * 16)),
                                            contrib);
                                }
                            }
                            Part acc = 0;
                            if constexpr (PRECISE) {
#pragma unroll
                                for (int k = 0; k < NV; ++k) {
                                    float f[VEC];
                                    unpack16<T>(raw[u][k], f);
#pragma unroll
                                    for (int e = 0; e < VEC; ++e)
                                        acc = dot_fma(f[e], gop[k][e], acc);
                                }
                            } else {
                                // even and odd channels in the two halves of packed fp32x2
                                // multiply-adds, added at the end
                                float2 a2 = make_float2(0.f, 0.f);
#pragma unroll
                                for (int k = 0; k < NV; ++k) {
                                    float f[VEC];
                                    unpack16<T>(raw[u][k], f);
#pragma unroll
                                    for (int e = 0; e < VEC; e += 2)
                                        a2 = ffma2(make_float2(f[e], f[e + 1]),
                                                   make_float2(go[k][e], go[k][e + 1]), a2);
                                }
                                acc = a2.x + a2.y;
                            }
                            // a select, not a multiplication by zero: row 0 (loaded in place of
                            // a missing row) may hold anything
                            part[u] = has_row ? acc : Part(0);
                        }
                    } else {
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const float w = __uint_as_float(rec[u].y);
#pragma unroll
                            for (int k = 0; k < NV; ++k) {
                                const int c = j + k * 32;
                                if (rec[u].x != kNoRow && c < D) {
                                    const size_t idx = static_cast<size_t>(rec[u].x) + c;
                                    const float v = Elem<T>::to_f(__ldg(value + idx));
                                    red_add_scalar(gval + idx, w * go[k][0]);
                                    part[u] = dot_fma(v, gop[k][0], part[u]);
                                }
                            }
                        }
                    }
                    // fold to PART partials per slot, then park them in shared memory
                    constexpr int PART = PRECISE ? PART_D : PART_F;
#pragma unroll
                    for (int u = 0; u < U; ++u) {
#pragma unroll
                        for (int off = LPR / 2; off >= PART; off >>= 1)
                            part[u] += __shfl_xor_sync(0xffffffffu, part[u], off);
                        const int slot = base + u * RPI + g;
                        if ((!GUARDED || slot < slot_end) && j < PART) {
                            float* dst;
                            if constexpr (RPI % CPS == 0) {
                                // whole samples per instruction: the lane's place inside a
                                // sample's partials never changes (part_lane), the sample
                                // advances by RPI / CPS per instruction
                                dst = s_part + (base / CPS + u * (RPI / CPS)) * SSTRIDE + part_lane;
                            } else {
                                dst = s_part + (slot / CPS) * SSTRIDE + (slot % CPS) * CSTR;
                            }
                            if constexpr (PRECISE) {
                                reinterpret_cast<double*>(dst)[j] = part[u];
                            } else {
                                dst[j] = part[u];
                            }
                        }
                    }
                };

                // a trip takes the double-precision form when one of its samples asked for it
                auto trip = [&](int base, auto guarded_tag) {
                    bool precise = false;
                    if constexpr (WIDE) {
                        // samples base/CPS .. of this trip (STEP / CPS of them)
                        constexpr int NS = (STEP / CPS > 0) ? STEP / CPS : 1;
                        constexpr uint32_t kBits = NS >= 32 ? 0xffffffffu : ((1u << NS) - 1u);
                        precise = ((m_precise >> (base / CPS)) & kBits) != 0u;
                    }
                    if (precise) {
                        if constexpr (WIDE)
                            scatter_gather(base, std::integral_constant<int, UNROLL>{}, guarded_tag,
                                           std::true_type{});
                    } else {
                        scatter_gather(base, std::integral_constant<int, UNROLL>{}, guarded_tag,
                                       std::false_type{});
                    }
                };
                int base = slot_begin;
#pragma unroll 1
                for (; base < unguarded_end; base += STEP) trip(base, std::false_type{});
#pragma unroll 1
                for (; base < slot_end; base += STEP) trip(base, std::true_type{});
            }
            __syncwarp();

            // ---- phase 3: lane = sample -----------------------------------------
            if constexpr (!FUSED) {
                if (active) {
                    const SampleGrad sg = sample_grad<Acc, CPS, PART_F, PART_D, CSTR>(
                        s_part + lane * SSTRIDE, geom, lane_trip_wide());
                    if constexpr (CPS == 4) {
                        store_pair(static_cast<T*>(p.grad_loc) + 2 * gi, sg.x, sg.y);
                        static_cast<T*>(p.grad_attn)[gi] = Elem<T>::from_f(sg.attn);
                    } else {
                        // nearest-pixel operator: d out / d attention = <value row, grad_out>;
                        // the integer locations have no gradient
                        static_cast<T*>(p.grad_attn)[gi] = Elem<T>::from_f(sg.attn);
                    }
                }
            } else {
                // Fused variant: chain the sample gradients through
                //   location = reference point + offset / (W, H)   and   weight = softmax(logits).
                float g_attn = 0.f, g_x = 0.f, g_y = 0.f;
                if (active && geom.valid) {
                    const SampleGrad sg = sample_grad<Acc, 4, PART_F, PART_D, CSTR>(
                        s_part + lane * SSTRIDE, geom, lane_trip_wide());
                    g_attn = sg.attn;
                    g_x = sg.x;
                    g_y = sg.y;
                }
                int tl, s;
                lane_sample_index(p, chunk, lane, tl, s);
                float* scratch = fused_scratch(s_slot);
                const float prob = active ? geom.prob : 0.f;
                // softmax backward: d logit_s = p_s * (d a_s - sum_j p_j * d a_j)
                const float dot = task_sum(p, prob * g_attn, lane, tl, scratch);
                __syncwarp();
                scratch[32 + lane] = g_x;
                scratch[64 + lane] = g_y;
                __syncwarp();
                if (active) {
                    store_pair(static_cast<T*>(p.grad_loc) + 2 * gi, g_x / geom.wf,
                               g_y / geom.hf);
                    static_cast<T*>(p.grad_attn)[gi] = Elem<T>::from_f(prob * (g_attn - dot));
                    if (s % p.P == 0) {
                        // first point of a level: the reference point of (b, q, level) gets
                        // the sum over this head's points (heads meet in the atomic)
                        float sx = 0.f, sy = 0.f;
                        for (int i = 0; i < p.P; ++i) {
                            sx += scratch[32 + lane + i];
                            sy += scratch[64 + lane + i];
                        }
                        const uint32_t t = static_cast<uint32_t>(item) * TPC + tl;
                        const uint32_t bq = fd_div(t, p.fd_h);
                        float* gr = p.grad_ref + (static_cast<size_t>(bq) * p.L + lv.level0) * 2;
                        atomicAdd(gr, sx);
                        atomicAdd(gr + 1, sy);
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
template <typename T, typename TG, int LPR, int NV, bool SCALAR, int MODE>
static cudaError_t launch_bwd_inst(const Params& p, const LaunchShape& ls, size_t smem,
                                   cudaStream_t stream) {
    auto kern = msda_bwd_kernel<T, TG, LPR, NV, SCALAR, MODE>;
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

template <typename T, typename TG, int MODE>
static cudaError_t launch_bwd_typed(const Params& p, const RowPlan& rp, const LaunchShape& ls, size_t smem,
                                    cudaStream_t stream) {
    if (rp.scalar) return launch_bwd_inst<T, TG, 32, 8, true, MODE>(p, ls, smem, stream);
    switch (rp.lpr * 100 + rp.nv) {
        case 101: return launch_bwd_inst<T, TG, 1, 1, false, MODE>(p, ls, smem, stream);
        case 201: return launch_bwd_inst<T, TG, 2, 1, false, MODE>(p, ls, smem, stream);
        case 401: return launch_bwd_inst<T, TG, 4, 1, false, MODE>(p, ls, smem, stream);
        case 801: return launch_bwd_inst<T, TG, 8, 1, false, MODE>(p, ls, smem, stream);
        case 1601: return launch_bwd_inst<T, TG, 16, 1, false, MODE>(p, ls, smem, stream);
        case 3201: return launch_bwd_inst<T, TG, 32, 1, false, MODE>(p, ls, smem, stream);
        case 3202:
            if constexpr (sizeof(T) == 4) {
                return launch_bwd_inst<T, TG, 32, 2, false, MODE>(p, ls, smem, stream);
            }
            return cudaErrorInvalidValue;
        default: return cudaErrorInvalidValue;
    }
}

template <int MODE>
static cudaError_t launch_backward_cps(const Params& p, int dtype, int acc_f32, const RowPlan& rp,
                                       const LaunchShape& ls, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(p.warp_smem) * kWarpsPerCta;
    switch (dtype) {
        case 0: return launch_bwd_typed<float, float, MODE>(p, rp, ls, smem, stream);
        case 1:
            return acc_f32 ? launch_bwd_typed<__half, float, MODE>(p, rp, ls, smem, stream)
                           : launch_bwd_typed<__half, __half, MODE>(p, rp, ls, smem, stream);
        case 2:
            return acc_f32
                       ? launch_bwd_typed<__nv_bfloat16, float, MODE>(p, rp, ls, smem, stream)
                       : launch_bwd_typed<__nv_bfloat16, __nv_bfloat16, MODE>(p, rp, ls, smem,
                                                                             stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace msda

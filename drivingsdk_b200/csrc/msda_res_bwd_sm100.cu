// MSDA backward for sm_100a with resident levels: the grad_value accumulators of a head's
// small pyramid levels live in the CTA's shared memory (see msda_res.cuh). Replaces, like
// msda_bwd_sm100.cu, the reference's backward device kernel and tiling
// (kernels/multi_scale_deformable_attn/op_kernel/multi_scale_deformable_attn_grad.cpp:151-249,
//  op_host/multi_scale_deformable_attn_grad.cpp:35-86); same arithmetic, different routing of
// the scatter.
//
// Per task (one warp, lane roles as in the other kernels):
//   phase 1  lane = sample: locations/weights (bulk-copied ahead into shared memory), the
//            four slot records {value row offset | none, bilinear * attention} and, per
//            slot, the shared-memory address of the accumulator row if the corner is resident.
//   phase 2  lane = (row slot, 16-byte piece): gathers the value row (through L2), adds
//            weight * grad_out into the accumulator row — a 16-byte compare-and-swap loop in
//            shared memory for resident rows, red.global.add.v4.f32 (or .v4.bf16x2/.f16x2)
//            otherwise — and leaves its partial dot product <value row, grad_out> in shared
//            memory. For fp32 tensors the dot products are doubles; samples whose location
//            gradient amplifies them little (max(W, H) * |attention| below a threshold) form
//            the product sums in fp32 and widen only the per-lane result.
//   phase 3  lane = sample: grad_attn, grad_loc from the partials (sample_grad).
// Per unit: the CTA adds its resident accumulators to global memory (vector reductions,
// rows that stayed zero are skipped) and clears them.
#include "msda_bwd_kernel.cuh"
#include "msda_res.cuh"

namespace msda {

#ifndef MSDA_RES_BWD_WARPS
#define MSDA_RES_BWD_WARPS 12
#endif
constexpr int kResBwdWarps = MSDA_RES_BWD_WARPS;

// shared memory of one warp: records (8 B per slot), accumulator addresses (4 B per slot),
// partial dot products, staging barriers, two staging buffers
constexpr uint32_t kResRecBytes = kSlots * 8;
constexpr uint32_t kResSaBytes = kSlots * 4;
__host__ __device__ inline uint32_t res_bwd_warp_bytes(int samples_per_item, size_t e) {
    return kResRecBytes + kResSaBytes + kPartBytes + 16 +
           2 * stage_bytes_per_buffer(samples_per_item, e);
}

template <typename T, typename TG, int LPR>
__global__ void __launch_bounds__(kResBwdWarps * 32, 1)
msda_bwd_res_kernel(const __grid_constant__ ResParams rp) {
    const Params& p = rp.p;
    constexpr int VEC = Elem<T>::kVec;
    constexpr int RPI = 32 / LPR;
    using Dot = DotT<T>;
    constexpr bool F32 = sizeof(T) == 4;
    constexpr int PART_MAX = F32 ? kPartMaxF64 : kPartMax;
    constexpr int PART = (LPR < PART_MAX) ? LPR : PART_MAX;
    constexpr int SSTRIDE = 4 * PART + 1;
    constexpr int UNROLL = (RPI >= 16) ? 2 : 4;
    constexpr int STEP = RPI * UNROLL;
    constexpr bool SPLIT_RED = sizeof(T) == 2 && sizeof(TG) == 4;
    constexpr int NW = kResBwdWarps;

    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane / LPR;
    const int j = lane % LPR;

    int* s_ctl = reinterpret_cast<int*>(smem);           // [0] bad level table
    ResLevel* s_lv = reinterpret_cast<ResLevel*>(smem + rp.lv_off);
    unsigned char* wb = smem + rp.warp_off + static_cast<size_t>(warp) * rp.warp_bytes;
    uint2* s_rec = reinterpret_cast<uint2*>(wb);
    uint32_t* s_sa = reinterpret_cast<uint32_t*>(wb + kResRecBytes);
    Dot* s_part = reinterpret_cast<Dot*>(wb + kResRecBytes + kResSaBytes);
    const uint32_t map_saddr = smem_u32(smem + rp.map_off);

    if (!res_plan_levels(rp, s_lv, s_ctl)) return;
    ResLane lv0, lv1;
    res_lane_levels(p, s_lv, lane, lv0, lv1);

    // clear the accumulators once; every unit leaves them cleared behind
    for (uint32_t i = threadIdx.x * 16u; i < rp.map_bytes; i += NW * 32 * 16u)
        sts128(map_saddr + i, make_uint4(0u, 0u, 0u, 0u));

    WarpStage<T> st =
        warp_stage_init<T>(p, wb + kResRecBytes + kResSaBytes + kPartBytes, lane);
    int stage_uses = 0;   // how many staged items this warp has consumed (barrier parity)

    const unsigned char* vlane = static_cast<const unsigned char*>(p.value) + j * 16;
    const T* __restrict__ gout = static_cast<const T*>(p.grad_out);
    unsigned char* glane = static_cast<unsigned char*>(p.grad_value) + j * 16;

    const int TPC = p.tasks_per_item;
    const int LP = p.LP;
    const int D = p.D;
    const int nchunks = (TPC == 1) ? (LP + kChunk - 1) / kChunk : 1;
    const uint32_t units_per_b = rp.chunks * static_cast<uint32_t>(p.H);

    __syncthreads();

    for (uint32_t unit = blockIdx.x; unit < rp.nunits; unit += gridDim.x) {
        const uint32_t b = unit / units_per_b;
        const uint32_t r = unit - b * units_per_b;
        const uint32_t chunk_q = r / static_cast<uint32_t>(p.H);
        const uint32_t h = r - chunk_q * static_cast<uint32_t>(p.H);
        const int q0 = static_cast<int>(chunk_q * rp.unit_q);
        const int q1 = min(p.Q, q0 + static_cast<int>(rp.unit_q));
        const int nitems = (q1 - q0 + TPC - 1) / TPC;
        // task number of query q of this unit: (b * Q + q) * H + h
        const long long task0 = (static_cast<long long>(b) * p.Q) * p.H + h;

        // issues the bulk copies of one item's locations and weights (lane 0)
        auto issue = [&](int item, int buf) {
            const int qa = q0 + item * TPC;
            const int nt = min(TPC, q1 - qa);
            const uint32_t ab = static_cast<uint32_t>(LP * sizeof(T));   // weights of one task
            unsigned char* dst = st.buffer(p, buf);
            mbar_expect_tx(st.bar + buf, 3u * ab * nt);
            for (int tl = 0; tl < nt; ++tl) {
                const long long t = task0 + static_cast<long long>(qa + tl) * p.H;
                bulk_g2s(dst + 2u * ab * tl, static_cast<const T*>(p.loc) + t * LP * 2, 2u * ab,
                         st.bar + buf);
                bulk_g2s(dst + 2u * ab * TPC + ab * tl, static_cast<const T*>(p.attn) + t * LP,
                         ab, st.bar + buf);
            }
        };

        int item = warp;
        if (st.ok && lane == 0 && item < nitems) issue(item, stage_uses & 1);

        for (; item < nitems; item += NW) {
            const int buf = stage_uses & 1;
            const T* sloc = nullptr;
            const T* sattn = nullptr;
            if (st.ok) {
                const bool next_issued = item + NW < nitems;
                if (lane == 0 && next_issued) issue(item + NW, buf ^ 1);
                const bool arrived =
                    __all_sync(0xffffffffu, mbar_wait(st.bar + buf, (stage_uses >> 1) & 1,
                                                      p.spin_limit) ? 1 : 0) != 0;
                if (arrived) {
                    sloc = reinterpret_cast<const T*>(st.buffer(p, buf));
                    sattn = reinterpret_cast<const T*>(st.buffer(p, buf) +
                                                       2u * TPC * LP * sizeof(T));
                } else {
                    st.ok = false;
                    if (lane == 0) atomicOr(p.status, kStatusStageTimeout);
                    st.drain(buf, stage_uses, next_issued);
                }
                ++stage_uses;
            }

            const int qa = q0 + item * TPC;
            const int ntask_here = min(TPC, q1 - qa);

            for (int chunk = 0; chunk < nchunks; ++chunk) {
                // ---- phase 1: lane = sample -------------------------------------
                int tl, s;
                lane_sample_index(p, chunk, lane, tl, s);
                const bool active = (tl < ntask_here) && (s < LP);
                uint4 rec01 = make_uint4(kNoRow, 0u, kNoRow, 0u);
                uint4 rec23 = rec01;
                ResCorners rc;
                rc.sa[0] = rc.sa[1] = rc.sa[2] = rc.sa[3] = 0u;
                SampleGeom geom;
                geom.lw = geom.lh = geom.a = geom.wf = geom.hf = geom.prob = 0.f;
                geom.x0 = geom.y0 = 0;
                geom.valid = false;
                long long gi = 0;
                if (active) {
                    const long long t = task0 + static_cast<long long>(qa + tl) * p.H;
                    gi = t * LP + s;
                    float lx, ly, a;
                    if (sloc != nullptr) {
                        const int li = tl * LP + s;
                        lx = Elem<T>::to_f(sloc[2 * li]);
                        ly = Elem<T>::to_f(sloc[2 * li + 1]);
                        a = Elem<T>::to_f(sattn[li]);
                    } else {
                        const T* gl = static_cast<const T*>(p.loc);
                        lx = Elem<T>::to_f(gl[2 * gi]);
                        ly = Elem<T>::to_f(gl[2 * gi + 1]);
                        a = Elem<T>::to_f(static_cast<const T*>(p.attn)[gi]);
                    }
                    const ResLane& lv = (TPC == 1 && chunk == 1) ? lv1 : lv0;
                    const uint32_t row_base =
                        (b * static_cast<uint32_t>(p.K) + static_cast<uint32_t>(lv.start)) *
                            static_cast<uint32_t>(p.H) + h;
                    sample_setup_res(lx, ly, a, lv, row_base, static_cast<uint32_t>(p.H),
                                     p.row_units, map_saddr, rp.map_row_bytes, rec01, rec23, geom,
                                     rc);
                    if (F32 && fmaxf(geom.wf, geom.hf) * fabsf(geom.a) >= rp.precise_amp) {
                        // accumulator addresses are multiples of 16: bit 0 carries the flag
                        rc.sa[0] |= 1u; rc.sa[1] |= 1u; rc.sa[2] |= 1u; rc.sa[3] |= 1u;
                    }
                }
                {
                    uint4* dst = reinterpret_cast<uint4*>(s_rec) + 2 * lane;
                    dst[0] = rec01;
                    dst[1] = rec23;
                    reinterpret_cast<uint4*>(s_sa)[lane] =
                        make_uint4(rc.sa[0], rc.sa[1], rc.sa[2], rc.sa[3]);
                }
                __syncwarp();

                // ---- phase 2: lane = (row slot, piece of row) --------------------
                for (int tl2 = 0; tl2 < ntask_here; ++tl2) {
                    int slot_begin, slot_end;
                    if (TPC == 1) {
                        slot_begin = 0;
                        slot_end = 4 * min(kChunk, LP - chunk * kChunk);
                    } else {
                        slot_begin = tl2 * 4 * LP;
                        slot_end = slot_begin + 4 * LP;
                    }
                    float go[VEC];
                    const size_t obase =
                        static_cast<size_t>(task0 + static_cast<long long>(qa + tl2) * p.H) * D;
                    unpack16<T>(*reinterpret_cast<const uint4*>(gout + obase + j * VEC), go);
                    Dot god[VEC];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) god[e] = static_cast<Dot>(go[e]);
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
                                gred[half][2 * i] =
                                    Elem<T>::to_f(*reinterpret_cast<const T*>(&l16));
                                gred[half][2 * i + 1] =
                                    Elem<T>::to_f(*reinterpret_cast<const T*>(&h16));
                            }
                        }
                    }

#pragma unroll 1
                    for (int base = slot_begin; base < slot_end; base += STEP) {
                        uint2 rec[UNROLL];
                        uint32_t sa[UNROLL];
                        uint4 raw[UNROLL];
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u) {
                            const int slot = base + u * RPI + g;
                            rec[u] = s_rec[slot];
                            sa[u] = s_sa[slot];
                            if (slot >= slot_end) rec[u].x = kNoRow;
                        }
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u) {
                            // a missing corner loads row 0 instead of branching around the load
                            const uint32_t off = (rec[u].x != kNoRow) ? rec[u].x : 0u;
                            raw[u] = ldg16(vlane + static_cast<size_t>(off) * 16);
                        }
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u) {
                            const int slot = base + u * RPI + g;
                            Dot part = 0;
                            if (rec[u].x != kNoRow) {
                                const float w = __uint_as_float(rec[u].y);
                                const uint32_t acc_row = sa[u] & ~15u;
                                if (acc_row != 0u) {
                                    // resident: fp32 accumulators in shared memory
#pragma unroll
                                    for (int v4 = 0; v4 < VEC / 4; ++v4)
                                        smem_add_f32x4(acc_row + (j * VEC + v4 * 4) * 4,
                                                       w * go[v4 * 4], w * go[v4 * 4 + 1],
                                                       w * go[v4 * 4 + 2], w * go[v4 * 4 + 3],
                                                       p.status);
                                } else if constexpr (SPLIT_RED) {
                                    float* row = reinterpret_cast<float*>(
                                        glane + static_cast<size_t>(rec[u].x) * 32);
                                    red_add_f32x4(row, w * gred[0][0], w * gred[0][1],
                                                  w * gred[0][2], w * gred[0][3]);
                                    red_add_f32x4(row + LPR * 4, w * gred[1][0], w * gred[1][1],
                                                  w * gred[1][2], w * gred[1][3]);
                                } else {
                                    float contrib[VEC];
#pragma unroll
                                    for (int e = 0; e < VEC; ++e) contrib[e] = w * go[e];
                                    red_add_vec<TG, VEC>(
                                        reinterpret_cast<TG*>(
                                            glane + static_cast<size_t>(rec[u].x) * 16),
                                        contrib);
                                }
                                float f[VEC];
                                unpack16<T>(raw[u], f);
                                if (!F32 || (sa[u] & 1u)) {
#pragma unroll
                                    for (int e = 0; e < VEC; ++e) part = dot_fma(f[e], god[e], part);
                                } else {
                                    float pf = 0.f;
#pragma unroll
                                    for (int e = 0; e < VEC; ++e) pf = fmaf(f[e], go[e], pf);
                                    part = static_cast<Dot>(pf);
                                }
                            }
#pragma unroll
                            for (int off = LPR / 2; off >= PART; off >>= 1)
                                part += __shfl_xor_sync(0xffffffffu, part, off);
                            if (slot < slot_end && j < PART)
                                s_part[(slot >> 2) * SSTRIDE + (slot & 3) * PART + j] = part;
                        }
                    }
                }
                __syncwarp();

                // ---- phase 3: lane = sample --------------------------------------
                if (active) {
                    const SampleGrad sg = sample_grad<T, 4, PART>(s_part + lane * SSTRIDE, geom);
                    store_pair(static_cast<T*>(p.grad_loc) + 2 * gi, sg.x, sg.y);
                    static_cast<T*>(p.grad_attn)[gi] = Elem<T>::from_f(sg.attn);
                }
                __syncwarp();
            }
        }

        // ---- end of unit: add the resident accumulators to global memory, clear them -----
        __syncthreads();
        {
            const uint32_t ppr = rp.map_row_bytes / 16;   // 16-byte pieces per accumulator row
            for (int l = 0; l < p.L; ++l) {
                const ResLevel L = s_lv[l];
                if (L.ry1 <= L.ry0) continue;
                const uint32_t npieces = static_cast<uint32_t>(L.ry1 - L.ry0) * L.w * ppr;
                const uint32_t row0 =
                    (b * static_cast<uint32_t>(p.K) + static_cast<uint32_t>(L.start + L.ry0 * L.w)) *
                        static_cast<uint32_t>(p.H) + h;
                if constexpr (sizeof(TG) == 4) {
                    for (uint32_t i = threadIdx.x; i < npieces; i += NW * 32) {
                        const uint32_t a = map_saddr + L.roff + i * 16;
                        const uint4 v = lds128(a);
                        if ((v.x | v.y | v.z | v.w) != 0u) {
                            const uint32_t pix = i / ppr, piece = i - pix * ppr;
                            float* dst = static_cast<float*>(p.grad_value) +
                                         (static_cast<size_t>(row0) + static_cast<size_t>(pix) * p.H) * D +
                                         piece * 4;
                            red_add_f32x4(dst, __uint_as_float(v.x), __uint_as_float(v.y),
                                          __uint_as_float(v.z), __uint_as_float(v.w));
                            sts128(a, make_uint4(0u, 0u, 0u, 0u));
                        }
                    }
                } else {
                    // 16-bit grad_value accumulated directly: eight channels per reduction
                    for (uint32_t i = threadIdx.x; i < npieces / 2; i += NW * 32) {
                        const uint32_t a = map_saddr + L.roff + i * 32;
                        const uint4 v0 = lds128(a), v1 = lds128(a + 16);
                        if ((v0.x | v0.y | v0.z | v0.w | v1.x | v1.y | v1.z | v1.w) != 0u) {
                            const uint32_t pix = (2 * i) / ppr, piece = 2 * i - pix * ppr;
                            TG* dst = static_cast<TG*>(p.grad_value) +
                                      (static_cast<size_t>(row0) + static_cast<size_t>(pix) * p.H) * D +
                                      piece * 4;
                            const float c[8] = {__uint_as_float(v0.x), __uint_as_float(v0.y),
                                                __uint_as_float(v0.z), __uint_as_float(v0.w),
                                                __uint_as_float(v1.x), __uint_as_float(v1.y),
                                                __uint_as_float(v1.z), __uint_as_float(v1.w)};
                            red_add_vec<TG, 8>(dst, c);
                            sts128(a, make_uint4(0u, 0u, 0u, 0u));
                            sts128(a + 16, make_uint4(0u, 0u, 0u, 0u));
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// launch
// ---------------------------------------------------------------------------
template <typename T, typename TG, int LPR>
static cudaError_t launch_res_bwd_inst(const ResParams& rp, int grid, cudaStream_t stream) {
    auto kern = msda_bwd_res_kernel<T, TG, LPR>;
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kResMaxSmem);
    if (e != cudaSuccess) return e;
    kern<<<grid, kResBwdWarps * 32, kResMaxSmem, stream>>>(rp);
    return cudaGetLastError();
}

template <typename T, typename TG>
static cudaError_t launch_res_bwd_typed(const ResParams& rp, int lpr, int grid,
                                        cudaStream_t stream) {
    switch (lpr) {
        case 1: return launch_res_bwd_inst<T, TG, 1>(rp, grid, stream);
        case 2: return launch_res_bwd_inst<T, TG, 2>(rp, grid, stream);
        case 4: return launch_res_bwd_inst<T, TG, 4>(rp, grid, stream);
        case 8: return launch_res_bwd_inst<T, TG, 8>(rp, grid, stream);
        case 16: return launch_res_bwd_inst<T, TG, 16>(rp, grid, stream);
        case 32: return launch_res_bwd_inst<T, TG, 32>(rp, grid, stream);
        default: return cudaErrorInvalidValue;
    }
}

bool resident_backward_applies(const Params& p, const RowPlan& rp) {
    // 16-byte vector path with one piece per lane; offsets of value rows below 2^31 units
    return !rp.scalar && rp.nv == 1;
}

cudaError_t launch_backward_resident(const Params& p_in, int dtype, int acc_f32,
                                     const RowPlan& rowplan, const LaunchShape& ls,
                                     const ResTune& tune, cudaStream_t stream) {
    ResParams rp;
    rp.p = p_in;
    Params& p = rp.p;
    const size_t e = dtype == 0 ? 4 : 2;
    const int spi = p.tasks_per_item * p.LP;
    // staging: one bulk copy per task and array, so a task's weights must be whole 16-byte
    // pieces; with many tiny tasks per item direct loads are cheaper than tiny copies
    if (!(p.stage && (static_cast<size_t>(p.LP) * e) % 16 == 0 && p.tasks_per_item <= 2))
        p.stage = 0;
    const UnitPlan up =
        plan_units(p.B, p.H, p.Q, p.tasks_per_item, ls.sm_count, kResBwdWarps);
    rp.chunks = up.chunks;
    rp.unit_q = up.unit_q;
    rp.nunits = up.nunits;
    rp.lv_off = 128;
    rp.warp_off = rp.lv_off + ((static_cast<uint32_t>(p.L) * sizeof(ResLevel) + 127u) & ~127u);
    rp.warp_bytes = (res_bwd_warp_bytes(spi, e) + 127u) & ~127u;
    rp.map_off = rp.warp_off + kResBwdWarps * rp.warp_bytes;
    rp.map_row_bytes = static_cast<uint32_t>(p.D) * 4u;
    if (rp.map_off + rp.map_row_bytes > static_cast<uint32_t>(kResMaxSmem))
        return cudaErrorInvalidConfiguration;
    uint32_t cap = (static_cast<uint32_t>(kResMaxSmem) - rp.map_off) & ~15u;
    if (tune.max_resident_bytes >= 0 && static_cast<uint32_t>(tune.max_resident_bytes) < cap)
        cap = static_cast<uint32_t>(tune.max_resident_bytes) & ~15u;
    rp.map_bytes = cap;
    rp.precise_amp = tune.precise_amp;
    switch (dtype) {
        case 0: return launch_res_bwd_typed<float, float>(rp, rowplan.lpr, up.grid, stream);
        case 1:
            return acc_f32 ? launch_res_bwd_typed<__half, float>(rp, rowplan.lpr, up.grid, stream)
                           : launch_res_bwd_typed<__half, __half>(rp, rowplan.lpr, up.grid, stream);
        case 2:
            return acc_f32 ? launch_res_bwd_typed<__nv_bfloat16, float>(rp, rowplan.lpr, up.grid,
                                                                        stream)
                           : launch_res_bwd_typed<__nv_bfloat16, __nv_bfloat16>(
                                 rp, rowplan.lpr, up.grid, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace msda

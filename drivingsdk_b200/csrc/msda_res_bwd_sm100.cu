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
#define MSDA_RES_BWD_WARPS 16
#endif
constexpr int kResBwdWarps = MSDA_RES_BWD_WARPS;

// shared memory of one warp: records (8 B per slot), accumulator addresses (4 B per slot),
// dot products (one per slot, 8 B), staging barriers, two staging buffers; the arrays have
// room for the slots a last trip may touch beyond the 128 of a pass
constexpr uint32_t kResSlotRoom = kSlots + kSlotPad;
constexpr uint32_t kResRecBytes = kResSlotRoom * 8;
constexpr uint32_t kResSaBytes = kResSlotRoom * 4;
constexpr uint32_t kResDotBytes = kSlots * 8;
// One staging buffer: locations and weights of the item's tasks (when they are staged), then
// the tasks' grad_output rows.
__host__ __device__ inline uint32_t res_bwd_la_bytes(int stage_la, int samples_per_item, size_t e) {
    return stage_la ? stage_bytes_per_buffer(samples_per_item, e) : 0u;
}
__host__ __device__ inline uint32_t res_bwd_stage_bytes(int stage_la, int samples_per_item,
                                                        int tasks_per_item, int D, size_t e) {
    return res_bwd_la_bytes(stage_la, samples_per_item, e) +
           static_cast<uint32_t>(tasks_per_item * D * e);
}
__host__ __device__ inline uint32_t res_bwd_warp_bytes(int stage_la, int samples_per_item,
                                                       int tasks_per_item, int D, size_t e) {
    return kResRecBytes + kResSaBytes + kResDotBytes + 16 +
           2 * res_bwd_stage_bytes(stage_la, samples_per_item, tasks_per_item, D, e);
}

// Sums GS partial dot products (one per row instruction of a group, this lane's piece of each
// row) over the LPR lanes of a row and parks the result of slot s in dot[s]. With four values
// and rows of at least four lanes the sums are formed by a transposing reduction: every
// exchange halves the number of values a lane carries, so four sums cost four exchanges
// instead of 4 * log2(LPR).
template <int LPR, int RPI, int GS, typename V, typename DotType>
__device__ __forceinline__ void park_dots(V (&v)[GS], DotType* dot, int slot0, int g, int j,
                                          int slot_end) {
    if constexpr (GS == 4) {
        static_assert(LPR >= 4, "transposing reduction needs four lanes per row");
        const bool hi_a = (j & (LPR / 2)) != 0;
        const bool hi_b = (j & (LPR / 4)) != 0;
        V k0 = hi_a ? v[2] : v[0], k1 = hi_a ? v[3] : v[1];
        const V s0 = hi_a ? v[0] : v[2], s1 = hi_a ? v[1] : v[3];
        k0 += __shfl_xor_sync(0xffffffffu, s0, LPR / 2);
        k1 += __shfl_xor_sync(0xffffffffu, s1, LPR / 2);
        V k = hi_b ? k1 : k0;
        const V s = hi_b ? k0 : k1;
        k += __shfl_xor_sync(0xffffffffu, s, LPR / 4);
#pragma unroll
        for (int off = LPR / 8; off >= 1; off >>= 1) k += __shfl_xor_sync(0xffffffffu, k, off);
        const int u = (hi_a ? 2 : 0) + (hi_b ? 1 : 0);
        const int slot = slot0 + u * RPI + g;
        if ((j & (LPR / 4 - 1)) == 0 && slot < slot_end) dot[slot] = static_cast<DotType>(k);
    } else {
#pragma unroll
        for (int u = 0; u < GS; ++u) {
            V k = v[u];
#pragma unroll
            for (int off = LPR / 2; off >= 1; off >>= 1) k += __shfl_xor_sync(0xffffffffu, k, off);
            const int slot = slot0 + u * RPI + g;
            if (j == 0 && slot < slot_end) dot[slot] = static_cast<DotType>(k);
        }
    }
}

template <typename T, typename TG, int LPR>
__global__ void __launch_bounds__(kResBwdWarps * 32, 1)
msda_bwd_res_kernel(const __grid_constant__ ResParams rp) {
    const Params& p = rp.p;
    constexpr int VEC = Elem<T>::kVec;
    constexpr int RPI = 32 / LPR;
    using Dot = DotT<T>;
    constexpr bool F32 = sizeof(T) == 4;
    constexpr int UBIG = (RPI >= 16) ? 2 : 8;     // row instructions per trip
    constexpr int USMALL = (RPI >= 16) ? 2 : 4;   //   ... for what is left of a task
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
    Dot* s_dot = reinterpret_cast<Dot*>(wb + kResRecBytes + kResSaBytes);   // one per slot
    const uint32_t map_saddr = smem_u32(smem + rp.map_off);
    const uint32_t trash_saddr = smem_u32(smem + rp.trash_off);   // one accumulator row of zeros

    if (!res_plan_levels(rp, s_lv, s_ctl)) return;
    ResLane lv0, lv1;
    res_lane_levels(p, s_lv, lane, lv0, lv1);

    // clear the scratch row and the accumulators once; every unit leaves them cleared behind
    for (uint32_t i = threadIdx.x * 16u; i < rp.map_off - rp.trash_off + rp.map_bytes;
         i += NW * 32 * 16u)
        sts128(trash_saddr + i, make_uint4(0u, 0u, 0u, 0u));

    // Staging (bulk copies into one of two per-warp buffers, one item ahead): the item's
    // locations and weights when p.stage is set, and always its grad_output rows.
    WarpStage<T> st;
    st.bar = reinterpret_cast<uint64_t*>(wb + kResRecBytes + kResSaBytes + kResDotBytes);
    st.ok = true;
    if (lane == 0) {
        mbar_init(st.bar, 1);
        mbar_init(st.bar + 1, 1);
        mbar_fence_init();
    }
    __syncwarp();
    int stage_uses = 0;   // how many staged items this warp has consumed (barrier parity)
    const uint32_t la_bytes = res_bwd_la_bytes(p.stage, p.tasks_per_item * p.LP, sizeof(T));
    const uint32_t buf_bytes =
        res_bwd_stage_bytes(p.stage, p.tasks_per_item * p.LP, p.tasks_per_item, p.D, sizeof(T));
    auto stage_buffer = [&](int bi) {
        return reinterpret_cast<unsigned char*>(st.bar) + 16 + bi * buf_bytes;
    };

    const unsigned char* vlane = static_cast<const unsigned char*>(p.value) + j * 16;
    const T* __restrict__ gout = static_cast<const T*>(p.grad_out);
    unsigned char* glane = static_cast<unsigned char*>(p.grad_value) + j * 16;

    const int TPC = p.tasks_per_item;
    const int LP = p.LP;
    const int D = p.D;
    const int nchunks = (TPC == 1) ? (LP + kChunk - 1) / kChunk : 1;
    // Units: per batch entry, the H * ceil(Q / TPC) items in (head, query) order are cut into
    // gridDim.x equal ranges, one per CTA; a range that crosses a head boundary is worked as
    // two units. All CTAs are on the same batch entry at (about) the same time, so that
    // entry's value rows and grad_value rows - twice the pyramid - are what L2 has to hold.
    const long long items_per_head = (p.Q + TPC - 1) / TPC;
    const long long items_per_b = items_per_head * p.H;

    __syncthreads();

    for (uint32_t b = 0; b < static_cast<uint32_t>(p.B); ++b)
    for (long long lo = items_per_b * blockIdx.x / gridDim.x,
                   hi = items_per_b * (blockIdx.x + 1) / gridDim.x; lo < hi;) {
        const uint32_t h = static_cast<uint32_t>(lo / items_per_head);
        const long long ia = lo - static_cast<long long>(h) * items_per_head;
        const long long ib = min(items_per_head, ia + (hi - lo));
        lo += ib - ia;
        const int q0 = static_cast<int>(ia) * TPC;
        const int q1 = min(p.Q, static_cast<int>(ib) * TPC);
        const int nitems = static_cast<int>(ib - ia);
        // task number of query q of this unit: (b * Q + q) * H + h
        const long long task0 = (static_cast<long long>(b) * p.Q) * p.H + h;

        // issues the bulk copies of one item (lane 0)
        auto issue = [&](int item, int buf) {
            const int qa = q0 + item * TPC;
            const int nt = min(TPC, q1 - qa);
            const uint32_t ab = static_cast<uint32_t>(LP * sizeof(T));   // weights of one task
            const uint32_t gb = static_cast<uint32_t>(D * sizeof(T));    // one grad_output row
            unsigned char* dst = stage_buffer(buf);
            mbar_expect_tx(st.bar + buf, (p.stage ? 3u * ab : 0u) * nt + gb * nt);
            for (int tl = 0; tl < nt; ++tl) {
                const long long t = task0 + static_cast<long long>(qa + tl) * p.H;
                if (p.stage) {
                    bulk_g2s(dst + 2u * ab * tl, static_cast<const T*>(p.loc) + t * LP * 2,
                             2u * ab, st.bar + buf);
                    bulk_g2s(dst + 2u * ab * TPC + ab * tl,
                             static_cast<const T*>(p.attn) + t * LP, ab, st.bar + buf);
                }
                bulk_g2s(dst + la_bytes + gb * tl, gout + t * D, gb, st.bar + buf);
            }
        };

        int item = warp;
        if (st.ok && lane == 0 && item < nitems) issue(item, stage_uses & 1);

        for (; item < nitems; item += NW) {
            const int buf = stage_uses & 1;
            const T* sloc = nullptr;
            const T* sattn = nullptr;
            const T* sgo = nullptr;
            if (st.ok) {
                const bool next_issued = item + NW < nitems;
                if (lane == 0 && next_issued) issue(item + NW, buf ^ 1);
                const bool arrived =
                    __all_sync(0xffffffffu, mbar_wait(st.bar + buf, (stage_uses >> 1) & 1,
                                                      p.spin_limit) ? 1 : 0) != 0;
                if (arrived) {
                    if (p.stage) {
                        sloc = reinterpret_cast<const T*>(stage_buffer(buf));
                        sattn = reinterpret_cast<const T*>(stage_buffer(buf) +
                                                           2u * TPC * LP * sizeof(T));
                    }
                    sgo = reinterpret_cast<const T*>(stage_buffer(buf) + la_bytes);
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
#ifdef MSDA_DEBUG_BOUNDS
                    {
                        // resident accumulator rows must lie inside the resident area
                        bool bad = false;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint32_t a16 = rc.sa[c];
                            if (a16 != 0u && (a16 < map_saddr ||
                                              a16 + rp.map_row_bytes > map_saddr + rp.map_bytes)) {
                                bad = true;
                                rc.sa[c] = 0u;
                            }
                        }
                        if (bad) atomicOr(p.status, kStatusOutOfBounds);
                    }
                    debug_check_rows(p, rec01, rec23);
#endif
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
                    // this lane's piece of grad_out[b, q, h, :] (from the staged row)
                    float go[VEC];
                    const T* grow =
                        sgo != nullptr
                            ? sgo + tl2 * D
                            : gout + static_cast<size_t>(task0 +
                                                         static_cast<long long>(qa + tl2) * p.H) * D;
                    unpack16<T>(*reinterpret_cast<const uint4*>(grow + j * VEC), go);
                    double god[F32 ? VEC : 1];
                    if constexpr (F32) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) god[e] = static_cast<double>(go[e]);
                    }
                    float gred[2][4];
                    if constexpr (SPLIT_RED) {
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const T* src = grow + (half * LPR + j) * 4;
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

                    // One trip: U row instructions (U * RPI slots): loads first, then the dot
                    // products (reduced over a row's lanes and parked per slot), then the
                    // scatter. A trip is compiled in several forms and the form is picked per
                    // trip by warp votes, so that the common cases run without per-row
                    // branches: KIND 0 = no resident row (reductions in L2 only), 1 = every row
                    // that exists is resident (compare-and-swap in shared memory only; rows
                    // that do not exist add zero to a scratch row), 2 = both kinds.
                    // PRECISE = dot products in double. GUARDED = slots past the task's last
                    // one are skipped.
                    auto trip = [&](int base, auto unroll_tag, auto kind_tag, auto precise_tag,
                                    auto guarded_tag) {
                        constexpr int U = decltype(unroll_tag)::value;
                        constexpr int KIND = decltype(kind_tag)::value;
                        constexpr bool PRECISE = decltype(precise_tag)::value;
                        constexpr bool GUARDED = decltype(guarded_tag)::value;
                        uint2 rec[U];
                        uint32_t sa[U];
                        uint4 raw[U];
                        bool exists[U];
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const int slot = base + u * RPI + g;
                            rec[u] = s_rec[slot];
                            sa[u] = (KIND != 0) ? (s_sa[slot] & ~15u) : 0u;
                            exists[u] = rec[u].x != kNoRow && (!GUARDED || slot < slot_end);
                            if (GUARDED && slot >= slot_end) sa[u] = 0u;
                            // KIND 1: a corner that does not exist adds zero to the scratch row
                            if (KIND == 1 && !exists[u]) sa[u] = trash_saddr;
                        }
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            // a missing corner loads row 0 instead of branching around the load
                            const uint32_t off = exists[u] ? rec[u].x : 0u;
                            raw[u] = ldg16(vlane + static_cast<size_t>(off) * 16);
                        }
                        // ---- dot products, GS row instructions at a time ----
                        constexpr int GS = (U >= 4 && LPR >= 4) ? 4 : 1;
#pragma unroll
                        for (int ub = 0; ub < U; ub += GS) {
                            if constexpr (PRECISE) {
                                double pd[GS];
#pragma unroll
                                for (int u = 0; u < GS; ++u) {
                                    float f[VEC];
                                    unpack16<T>(raw[ub + u], f);
                                    double acc = 0.0;
#pragma unroll
                                    for (int e = 0; e < VEC; ++e)
                                        acc = fma(static_cast<double>(f[e]), god[e], acc);
                                    pd[u] = exists[ub + u] ? acc : 0.0;
                                }
                                park_dots<LPR, RPI, GS>(pd, s_dot, base + ub * RPI, g, j, slot_end);
                            } else {
                                float pf[GS];
#pragma unroll
                                for (int u = 0; u < GS; ++u) {
                                    float f[VEC];
                                    unpack16<T>(raw[ub + u], f);
                                    float acc = 0.f;
#pragma unroll
                                    for (int e = 0; e < VEC; ++e) acc = fmaf(f[e], go[e], acc);
                                    pf[u] = exists[ub + u] ? acc : 0.f;
                                }
                                park_dots<LPR, RPI, GS>(pf, s_dot, base + ub * RPI, g, j, slot_end);
                            }
                        }
                        // ---- scatter ----
                        constexpr int NP = VEC / 4;   // 16-byte pieces of accumulator per lane
                        auto global_red = [&](int u, float w) {
                            if constexpr (SPLIT_RED) {
                                float* row = reinterpret_cast<float*>(
                                    glane + static_cast<size_t>(rec[u].x) * 32);
                                red_add_f32x4(row, w * gred[0][0], w * gred[0][1], w * gred[0][2],
                                              w * gred[0][3]);
                                red_add_f32x4(row + LPR * 4, w * gred[1][0], w * gred[1][1],
                                              w * gred[1][2], w * gred[1][3]);
                            } else {
                                float contrib[VEC];
#pragma unroll
                                for (int e = 0; e < VEC; ++e) contrib[e] = w * go[e];
                                red_add_vec<TG, VEC>(
                                    reinterpret_cast<TG*>(glane +
                                                          static_cast<size_t>(rec[u].x) * 16),
                                    contrib);
                            }
                        };
                        if constexpr (KIND == 0) {
#pragma unroll
                            for (int u = 0; u < U; ++u)
                                if (exists[u]) global_red(u, __uint_as_float(rec[u].y));
                        } else if constexpr (KIND == 1) {
                            // every slot has an accumulator row (the scratch row for corners
                            // that do not exist, which get weight 0): no branches until a
                            // compare-and-swap is lost
                            constexpr int SB = (U >= 4) ? (NP == 1 ? 4 : 2) : 1;
#pragma unroll
                            for (int ub = 0; ub < U; ub += SB) {
                                uint4 old[SB][NP];
#pragma unroll
                                for (int v = 0; v < SB; ++v)
#pragma unroll
                                    for (int v4 = 0; v4 < NP; ++v4)
                                        old[v][v4] = lds128(sa[ub + v] + (j * VEC + v4 * 4) * 4);
                                bool lost = false;
                                bool ok[SB][NP];
#pragma unroll
                                for (int v = 0; v < SB; ++v) {
                                    const int u = ub + v;
                                    const float w = exists[u] ? __uint_as_float(rec[u].y) : 0.f;
#pragma unroll
                                    for (int v4 = 0; v4 < NP; ++v4) {
                                        ok[v][v4] = smem_cas_add_f32x4(
                                            sa[u] + (j * VEC + v4 * 4) * 4, old[v][v4],
                                            w * go[v4 * 4], w * go[v4 * 4 + 1], w * go[v4 * 4 + 2],
                                            w * go[v4 * 4 + 3]);
                                        lost |= !ok[v][v4];
                                    }
                                }
                                if (__any_sync(0xffffffffu, lost)) {
#pragma unroll
                                    for (int v = 0; v < SB; ++v) {
                                        const int u = ub + v;
                                        const float w =
                                            exists[u] ? __uint_as_float(rec[u].y) : 0.f;
#pragma unroll
                                        for (int v4 = 0; v4 < NP; ++v4)
                                            if (!ok[v][v4])
                                                smem_add_f32x4(sa[u] + (j * VEC + v4 * 4) * 4,
                                                               w * go[v4 * 4], w * go[v4 * 4 + 1],
                                                               w * go[v4 * 4 + 2],
                                                               w * go[v4 * 4 + 3], p.status);
                                    }
                                }
                            }
                        } else {
#pragma unroll
                            for (int u = 0; u < U; ++u) {
                                if (!exists[u]) continue;
                                const float w = __uint_as_float(rec[u].y);
                                if (sa[u] != 0u) {
#pragma unroll
                                    for (int v4 = 0; v4 < NP; ++v4)
                                        smem_add_f32x4(sa[u] + (j * VEC + v4 * 4) * 4,
                                                       w * go[v4 * 4], w * go[v4 * 4 + 1],
                                                       w * go[v4 * 4 + 2], w * go[v4 * 4 + 3],
                                                       p.status);
                                } else {
                                    global_red(u, w);
                                }
                            }
                        }
                    };

                    // which form a trip takes: votes over its slots
                    auto classify = [&](int base, int nrow, int& kind, bool& precise) {
                        uint32_t any_res = 0, any_glob = 0, any_prec = 0;
                        for (int u = 0; u < nrow; ++u) {
                            const int slot = base + u * RPI + g;
                            if (slot < slot_end) {
                                const uint32_t a = s_sa[slot];
                                const bool ex = s_rec[slot].x != kNoRow;
                                any_res |= (a & ~15u);
                                any_glob |= (ex && (a & ~15u) == 0u) ? 1u : 0u;
                                any_prec |= ex ? (a & 1u) : 0u;
                            }
                        }
                        const bool r = __any_sync(0xffffffffu, any_res != 0u);
                        const bool gl = __any_sync(0xffffffffu, any_glob != 0u);
                        precise = F32 && __any_sync(0xffffffffu, any_prec != 0u);
                        kind = r ? (gl ? 2 : 1) : 0;
                    };
                    using std::integral_constant;
                    using std::false_type;
                    using std::true_type;
                    auto run = [&](int base, auto unroll_tag, auto guarded_tag) {
                        constexpr int U = decltype(unroll_tag)::value;
                        int kind;
                        bool precise;
                        classify(base, U, kind, precise);
                        if constexpr (decltype(guarded_tag)::value) {
                            // the odd trip at a task's end: one general form per precision
                            if (precise) {
                                if constexpr (F32)
                                    trip(base, unroll_tag, integral_constant<int, 2>{},
                                         true_type{}, true_type{});
                            } else {
                                trip(base, unroll_tag, integral_constant<int, 2>{}, false_type{},
                                     true_type{});
                            }
                        } else if (precise) {
                            if constexpr (F32) {
                                if (kind == 0)
                                    trip(base, unroll_tag, integral_constant<int, 0>{},
                                         true_type{}, false_type{});
                                else if (kind == 1)
                                    trip(base, unroll_tag, integral_constant<int, 1>{},
                                         true_type{}, false_type{});
                                else
                                    trip(base, unroll_tag, integral_constant<int, 2>{},
                                         true_type{}, false_type{});
                            }
                        } else {
                            if (kind == 0)
                                trip(base, unroll_tag, integral_constant<int, 0>{}, false_type{},
                                     false_type{});
                            else if (kind == 1)
                                trip(base, unroll_tag, integral_constant<int, 1>{}, false_type{},
                                     false_type{});
                            else
                                trip(base, unroll_tag, integral_constant<int, 2>{}, false_type{},
                                     false_type{});
                        }
                    };

                    int base = slot_begin;
#pragma unroll 1
                    for (; base + UBIG * RPI <= slot_end; base += UBIG * RPI)
                        run(base, integral_constant<int, UBIG>{}, false_type{});
#pragma unroll 1
                    for (; base < slot_end; base += USMALL * RPI)
                        run(base, integral_constant<int, USMALL>{}, true_type{});
                }
                __syncwarp();

                // ---- phase 3: lane = sample --------------------------------------
                if (active) {
                    const SampleGrad sg = sample_grad<T, 4, 1>(s_dot + lane * 4, geom);
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
    // staging of locations/weights: one bulk copy per task and array, so a task's weights
    // must be whole 16-byte pieces (grad_output rows always are on this path)
    if (!(p.stage && (static_cast<size_t>(p.LP) * e) % 16 == 0)) p.stage = 0;
    // one CTA per SM (shared memory allows no more), fewer when a batch entry has fewer items
    const long long items_per_b =
        static_cast<long long>((p.Q + p.tasks_per_item - 1) / p.tasks_per_item) * p.H;
    const int grid = static_cast<int>(items_per_b < ls.sm_count ? items_per_b : ls.sm_count);
    rp.lv_off = 128;
    rp.warp_off = rp.lv_off + ((static_cast<uint32_t>(p.L) * sizeof(ResLevel) + 127u) & ~127u);
    rp.warp_bytes =
        (res_bwd_warp_bytes(p.stage, spi, p.tasks_per_item, p.D, e) + 127u) & ~127u;
    rp.map_row_bytes = static_cast<uint32_t>(p.D) * 4u;
    rp.trash_off = rp.warp_off + kResBwdWarps * rp.warp_bytes;
    rp.map_off = rp.trash_off + ((rp.map_row_bytes + 127u) & ~127u);
    if (rp.map_off + rp.map_row_bytes > static_cast<uint32_t>(kResMaxSmem))
        return cudaErrorInvalidConfiguration;
    uint32_t cap = (static_cast<uint32_t>(kResMaxSmem) - rp.map_off) & ~15u;
    if (tune.max_resident_bytes >= 0 && static_cast<uint32_t>(tune.max_resident_bytes) < cap)
        cap = static_cast<uint32_t>(tune.max_resident_bytes) & ~15u;
    rp.map_bytes = cap;
    rp.precise_amp = tune.precise_amp;
    switch (dtype) {
        case 0: return launch_res_bwd_typed<float, float>(rp, rowplan.lpr, grid, stream);
        case 1:
            return acc_f32 ? launch_res_bwd_typed<__half, float>(rp, rowplan.lpr, grid, stream)
                           : launch_res_bwd_typed<__half, __half>(rp, rowplan.lpr, grid, stream);
        case 2:
            return acc_f32 ? launch_res_bwd_typed<__nv_bfloat16, float>(rp, rowplan.lpr, grid,
                                                                        stream)
                           : launch_res_bwd_typed<__nv_bfloat16, __nv_bfloat16>(
                                 rp, rowplan.lpr, grid, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace msda

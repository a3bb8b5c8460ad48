// Shared pieces of the "resident level" MSDA kernels for sm_100a.
//
// Work decomposition. One persistent CTA per SM. Batch entries are worked one after the
// other by all CTAs together (so that one entry's value and grad_value rows are what L2 has
// to hold); within an entry its tasks, in (head, query) order, are cut into equal contiguous
// ranges, one per CTA. A unit is the part of a CTA's range that lies in one head: every task
// of a unit has the same (batch entry, head), which is what lets the CTA keep that head's
// small pyramid levels in its own shared memory:
//   backward: fp32 accumulators of grad_value for the resident levels; the scatter into them
//             is a 16-byte compare-and-swap loop in shared memory instead of a vector
//             reduction in L2 (L2 retires ~50 G 128-byte row reductions per second on B200,
//             which is what bounds a backward that sends every row there), and the
//             accumulators are added to global memory once per unit.
// Which pixel rows of which levels are resident is decided on the device from the level
// table (callers may pass it in device memory, where the host cannot read it without a
// synchronisation): levels are taken whole from the smallest up while they fit, the next one
// gets a centred window of pixel rows, the rest go through L2 as before.
//
// The level table is also validated here (positive sizes, start + h*w <= K): a bad table
// sets kStatusBadLevels in the device status word and the kernel returns without touching
// value, grad_value or the outputs.
#pragma once

#include "msda_launch.h"
#include "msda_tile.cuh"

namespace msda {

constexpr int kStatusBadLevels = 4;  // level table inconsistent with K: nothing was computed
constexpr int kStatusAccGiveUp = 8;  // a shared-memory accumulate gave up (never expected)

constexpr int kResMaxSmem = 232448;  // 227 KiB: most dynamic shared memory one CTA can have
constexpr int kCasLimit = 1 << 16;   // bound on retries of one compare-and-swap accumulate

// One level as the resident kernels see it (32 bytes, in shared memory).
struct ResLevel {
    int h, w, start;
    int ry0, ry1;     // pixel rows [ry0, ry1) are resident (ry0 == ry1: none)
    uint32_t roff;    // byte offset of pixel (ry0, 0) inside the resident area
    int pad0, pad1;
};

struct ResParams {
    Params p;
    uint32_t lv_off;         // shared-memory offsets: level table,
    uint32_t warp_off;       //   first warp's private area,
    uint32_t warp_bytes;     //   its size,
    uint32_t trash_off;      //   one scratch accumulator row (stays zero),
    uint32_t map_off;        //   resident area,
    uint32_t map_bytes;      //   its capacity
    uint32_t map_row_bytes;  // bytes of one resident pixel (fp32 accumulator row: 4 * D)
    float precise_amp;       // samples with max(W, H) * |attention| >= this take the
                             // double-precision dot products (fp32 tensors only)
};

// ---------------------------------------------------------------------------
// device side
// ---------------------------------------------------------------------------

// Reads and validates the level table and decides the resident windows. Called by every
// thread of the CTA; returns false (after setting the status bit) when the table is bad.
__device__ __forceinline__ bool res_plan_levels(const ResParams& rp, ResLevel* lv, int* s_bad) {
    const Params& p = rp.p;
    if (threadIdx.x == 0) {
        int bad = 0;
        for (int l = 0; l < p.L; ++l) {
            int hh, ww, ss;
            if (p.use_table) {
                hh = p.lv.h[l]; ww = p.lv.w[l]; ss = p.lv.start[l];
            } else {
                hh = p.shapes_dev[2 * l]; ww = p.shapes_dev[2 * l + 1]; ss = p.start_dev[l];
            }
            if (hh <= 0 || ww <= 0 || ss < 0 ||
                static_cast<long long>(ss) + static_cast<long long>(hh) * ww > p.K)
                bad = 1;
            lv[l].h = hh; lv[l].w = ww; lv[l].start = ss;
            lv[l].ry0 = 0; lv[l].ry1 = 0; lv[l].roff = 0;
        }
        if (!bad) {
            uint32_t used = 0;
            unsigned long long done = 0;
            for (int n = 0; n < p.L; ++n) {
                int best = -1;
                long long best_px = 0;
                for (int l = 0; l < p.L; ++l) {
                    if ((done >> l) & 1ull) continue;
                    const long long px = static_cast<long long>(lv[l].h) * lv[l].w;
                    if (best < 0 || px < best_px) { best = l; best_px = px; }
                }
                done |= 1ull << best;
                const unsigned long long row_line =
                    static_cast<unsigned long long>(lv[best].w) * rp.map_row_bytes;
                const unsigned long long left = rp.map_bytes - used;
                unsigned long long rows = left / row_line;
                if (rows == 0) break;
                if (rows >= static_cast<unsigned long long>(lv[best].h)) {
                    rows = lv[best].h;
                    lv[best].ry0 = 0;
                } else {
                    lv[best].ry0 = (lv[best].h - static_cast<int>(rows)) / 2;
                }
                lv[best].ry1 = lv[best].ry0 + static_cast<int>(rows);
                lv[best].roff = used;
                used += static_cast<uint32_t>(rows * row_line);
                if (lv[best].ry1 - lv[best].ry0 < lv[best].h) break;   // one partial level, then stop
            }
        }
        *s_bad = bad;
        if (bad) atomicOr(p.status, kStatusBadLevels);
    }
    __syncthreads();
    return *s_bad == 0;
}

// Per-lane view of the level its sample belongs to (lane -> sample is fixed for the kernel).
struct ResLane {
    int w, h, start, ry0, ry1;
    uint32_t roff;
};
__device__ __forceinline__ void res_lane_levels(const Params& p, const ResLevel* lv, int lane,
                                                ResLane& a, ResLane& b) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        int tl, s;
        lane_sample_index(p, c, lane, tl, s);
        int l = s / p.P;
        if (l >= p.L) l = p.L - 1;
        ResLane r;
        r.w = lv[l].w; r.h = lv[l].h; r.start = lv[l].start;
        r.ry0 = lv[l].ry0; r.ry1 = lv[l].ry1; r.roff = lv[l].roff;
        if (c == 0) a = r; else b = r;
    }
}

// 16 bytes of shared memory
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "r"(addr));
    return r;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

// One attempt of acc[0..3] += (a, b, c, d): `old` is what the caller read there before.
// Returns true when the sum went in; `old` is then unchanged, otherwise it holds what the
// accumulator holds now. Callers issue the reads of several rows, then these attempts, then
// deal with the (rare) failures through smem_add_f32x4.
__device__ __forceinline__ bool smem_cas_add_f32x4(uint32_t addr, uint4& old, float a, float b,
                                                   float c, float d) {
    const uint32_t n0 = __float_as_uint(__uint_as_float(old.x) + a);
    const uint32_t n1 = __float_as_uint(__uint_as_float(old.y) + b);
    const uint32_t n2 = __float_as_uint(__uint_as_float(old.z) + c);
    const uint32_t n3 = __float_as_uint(__uint_as_float(old.w) + d);
    const uint64_t clo = (static_cast<uint64_t>(old.y) << 32) | old.x;
    const uint64_t chi = (static_cast<uint64_t>(old.w) << 32) | old.z;
    const uint64_t nlo = (static_cast<uint64_t>(n1) << 32) | n0;
    const uint64_t nhi = (static_cast<uint64_t>(n3) << 32) | n2;
    uint64_t olo, ohi;
    asm volatile(
        "{\n\t.reg .b128 cc, nn, oo;\n\t"
        "mov.b128 cc, {%2, %3};\n\t"
        "mov.b128 nn, {%4, %5};\n\t"
        "atom.relaxed.cta.shared::cta.cas.b128 oo, [%6], cc, nn;\n\t"
        "mov.b128 {%0, %1}, oo;\n\t}"
        : "=l"(olo), "=l"(ohi)
        : "l"(clo), "l"(chi), "l"(nlo), "l"(nhi), "r"(addr)
        : "memory");
    return olo == clo && ohi == chi;
}

// acc[0..3] += (a, b, c, d) on four consecutive floats of shared memory, atomically with
// respect to the other warps of the CTA: read, add, 128-bit compare-and-swap, retry on a
// lost race. Retries are bounded; giving up sets *gave_up (never seen in practice: a retry
// only follows another warp's successful update of the same 16 bytes).
__device__ __forceinline__ void smem_add_f32x4(uint32_t addr, float a, float b, float c, float d,
                                               int* status) {
    uint4 o = lds128(addr);
    for (int tries = 0; tries < kCasLimit; ++tries) {
        const uint32_t n0 = __float_as_uint(__uint_as_float(o.x) + a);
        const uint32_t n1 = __float_as_uint(__uint_as_float(o.y) + b);
        const uint32_t n2 = __float_as_uint(__uint_as_float(o.z) + c);
        const uint32_t n3 = __float_as_uint(__uint_as_float(o.w) + d);
        const uint64_t clo = (static_cast<uint64_t>(o.y) << 32) | o.x;
        const uint64_t chi = (static_cast<uint64_t>(o.w) << 32) | o.z;
        const uint64_t nlo = (static_cast<uint64_t>(n1) << 32) | n0;
        const uint64_t nhi = (static_cast<uint64_t>(n3) << 32) | n2;
        uint64_t olo, ohi;
        asm volatile(
            "{\n\t.reg .b128 cc, nn, oo;\n\t"
            "mov.b128 cc, {%2, %3};\n\t"
            "mov.b128 nn, {%4, %5};\n\t"
            "atom.relaxed.cta.shared::cta.cas.b128 oo, [%6], cc, nn;\n\t"
            "mov.b128 {%0, %1}, oo;\n\t}"
            : "=l"(olo), "=l"(ohi)
            : "l"(clo), "l"(chi), "l"(nlo), "l"(nhi), "r"(addr)
            : "memory");
        if (olo == clo && ohi == chi) return;
        o.x = static_cast<uint32_t>(olo);
        o.y = static_cast<uint32_t>(olo >> 32);
        o.z = static_cast<uint32_t>(ohi);
        o.w = static_cast<uint32_t>(ohi >> 32);
    }
    atomicOr(status, kStatusAccGiveUp);
}

// Bilinear set-up of one sample for the resident kernels: the four slot records of
// sample_setup() (offset of the corner's value row in 16-byte units or kNoRow, bilinear
// weight * attention) plus, per corner, the shared-memory address of its accumulator row
// when the corner lies in the level's resident window (0 otherwise).
struct ResCorners {
    uint32_t sa[4];
};
__device__ __forceinline__ void sample_setup_res(float lx, float ly, float a, const ResLane& lv,
                                                 uint32_t row_base, uint32_t H, uint32_t row_units,
                                                 uint32_t map_saddr, uint32_t map_row_bytes,
                                                 uint4& rec01, uint4& rec23, SampleGeom& g,
                                                 ResCorners& rc) {
    sample_setup(lx, ly, a, lv.w, lv.h, row_base, H, row_units, rec01, rec23, g);
    rc.sa[0] = rc.sa[1] = rc.sa[2] = rc.sa[3] = 0u;
    if (g.valid && lv.ry1 > lv.ry0) {
        const int x0 = g.x0, y0 = g.y0;
        const uint32_t base = map_saddr + lv.roff;
        const bool r0 = y0 >= lv.ry0 && y0 < lv.ry1;
        const bool r1 = y0 + 1 >= lv.ry0 && y0 + 1 < lv.ry1;
        const int p00 = (y0 - lv.ry0) * lv.w + x0;
        if (r0 && rec01.x != kNoRow) rc.sa[0] = base + static_cast<uint32_t>(p00) * map_row_bytes;
        if (r0 && rec01.z != kNoRow) rc.sa[1] = base + static_cast<uint32_t>(p00 + 1) * map_row_bytes;
        if (r1 && rec23.x != kNoRow) rc.sa[2] = base + static_cast<uint32_t>(p00 + lv.w) * map_row_bytes;
        if (r1 && rec23.z != kNoRow)
            rc.sa[3] = base + static_cast<uint32_t>(p00 + lv.w + 1) * map_row_bytes;
    }
}

}  // namespace msda

// Shared device-side pieces of the sm_100a multi-scale deformable attention
// (MSDA) kernels: parameter blocks, the per-sample bilinear set-up, 16-byte
// vector loads, vector reductions into global memory, and the bounded
// bulk-copy (TMA) + mbarrier primitives used to stage location/weight tiles.
//
// Semantics follow the reference operator:
//   * pixel coordinates  x = loc_x * W - 0.5,  y = loc_y * H - 0.5
//     (kernels/multi_scale_deformable_attn/op_kernel/msda.h:367-368);
//   * a sample takes part only if  x > -1 && y > -1 && x < W && y < H, which
//     also drops NaN/Inf locations (msda.h:369-390);
//   * corner (y0,x0) needs y0>=0 && x0>=0, (y0,x1) needs y0>=0 && x1<=W-1,
//     (y1,x0) needs y1<=H-1 && x0>=0, (y1,x1) needs y1<=H-1 && x1<=W-1; a
//     missing corner reads as zero and receives no gradient
//     (op_kernel/arch35/multi_scale_deformable_attn.cpp:59-62);
//   * corner weights hh*hw, hh*lw, lh*hw, lh*lw, each times the attention
//     weight (msda.h:492-520).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace msda {

constexpr int kMaxLevels = 64;      // L*P <= 64 implies L <= 64
constexpr int kWarpsPerCta = 8;
constexpr int kThreadsPerCta = kWarpsPerCta * 32;
constexpr int kChunk = 32;          // samples handled by one warp pass
constexpr int kSlots = 4 * kChunk;  // (sample, corner) pairs per warp pass
constexpr int kSlotPad = 64;         // readable (never used) records past the last slot
constexpr int kSpinLimit = 1 << 18; // default bound on mbarrier polling (Params::spin_limit)
constexpr int kDrainLimit = 1 << 20; // bound on waiting for copies already issued after a time-out

// Device status bits, sticky until read by msda_sm100_device_status().
constexpr int kStatusStageTimeout = 1;  // a staged tile never arrived
constexpr int kStatusBadLevels = 4;     // device-resident level table inconsistent with K: kernel did nothing
constexpr int kStatusOutOfBounds = 16;  // MSDA_DEBUG_BOUNDS build: a computed row offset fell outside
                                        // value / grad_value; the access was skipped

// Division by a runtime constant without a divide: q = (n * mul) >> shift, exact
// for 0 <= n < 2^31 (round-up method with a 31 + ceil(log2 d) bit shift).
struct FastDiv {
    uint32_t mul;
    uint32_t shift;
};
inline FastDiv make_fastdiv(uint32_t d) {
    uint32_t s = 0;
    while ((1ull << s) < d) ++s;
    FastDiv f;
    f.shift = 31 + s;
    f.mul = static_cast<uint32_t>(((1ull << f.shift) + d - 1) / d);
    return f;
}
__device__ __forceinline__ uint32_t fd_div(uint32_t n, const FastDiv& f) {
    return static_cast<uint32_t>((static_cast<uint64_t>(n) * f.mul) >> f.shift);
}

// Kernel modes (template parameter): rows per sample, or the fused bilinear variant whose
// phase 1 builds locations and weights from reference points, offsets and logits.
constexpr int kModeBilinear = 4;
constexpr int kModeNearest = 1;
constexpr int kModeFused = 5;

constexpr uint32_t kNoRow = 0xffffffffu;  // slot record of a corner that does not exist

// Level geometry by value. A launch that received the shapes on the host puts
// them here (kernel parameters live in the constant bank); a launch that
// received device pointers leaves use_table = 0 and each CTA reads the two
// small arrays from global memory once.
struct LevelTable {
    int h[kMaxLevels];
    int w[kMaxLevels];
    int start[kMaxLevels];
};

struct Params {
    // forward operands
    const void* value;   // [B, K, H, D]
    const void* loc;     // [B, Q, H, L, P, 2]  (x, y) in [0, 1]
    const void* attn;    // [B, Q, H, L, P]
    void* out;           // [B, Q, H*D]
    // fused variant: loc holds sampling offsets [B,Q,H,L,P,2], attn holds logits [B,Q,H,L,P],
    // grad_loc / grad_attn receive their gradients, and
    const void* ref;     // reference points [B, Q, L, 2]
    float* grad_ref;     // [B, Q, L, 2] fp32, zero-filled by the caller of the kernel
    // backward operands
    const void* grad_out;  // [B, Q, H*D]
    void* grad_value;      // [B, K, H, D]; accumulation target (may be fp32 scratch)
    void* grad_loc;        // like loc
    void* grad_attn;       // like attn
    // level geometry on the device (used when use_table == 0)
    const int* shapes_dev;  // [L, 2] (H, W)
    const int* start_dev;   // [L]
    int B, K, H, D, L, Q, P;
    int LP;             // L * P
    int tasks_per_item; // consecutive (b, q, h) tasks one warp pass covers
    int use_table;
    int pack_rows;      // 1: the forward kernels keep records only for the corners that exist
    int stage;          // 1: each warp bulk-copies its next item's locations/weights to shared
                        // memory while it works on the current one; 0: direct loads
    float precise_amp;  // fp32 backward: samples with max(W, H) * |attention| >= this value
                        // accumulate their dot products in double from the first product on
    int spin_limit;     // polls of a staging barrier before the warp gives up on it (0: every
                        // wait times out at once, which is how the fall-back path is tested)
    long long ntasks;   // B * Q * H
    long long nitems;   // ceil(ntasks / tasks_per_item)
    int* status;        // device status word
    uint32_t row_units;      // offset units per value row: 16-byte pieces, or elements (scalar path)
    uint32_t limit_units;    // B * K * H * row_units: one past the last valid row offset + row
    uint32_t warp_smem;      // bytes of dynamic shared memory per warp
    FastDiv fd_qh, fd_h, fd_lp;  // division by Q*H, H, L*P
    // walk order of the items: 0 = memory order; B > 0 = batch entries interleaved (walk
    // position i -> item (i % B) * walk_items_per_b + i / B)
    uint32_t walk_b, walk_items_per_b;
    FastDiv fd_walk_b;
    LevelTable lv;
};

// ---------------------------------------------------------------------------
// element types
// ---------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int kVec = 4;  // elements in 16 bytes
    __device__ static __forceinline__ float to_f(float v) { return v; }
    __device__ static __forceinline__ float from_f(float v) { return v; }
};
template <> struct Elem<__half> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ float to_f(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte read-only load of a piece of a gathered value row. Rows are reused mostly across
// SMs (through L2); letting them allocate in L1 as well (evict-last) measured a few percent
// faster on pyramids whose smallest levels are hit often, and never slower.
__device__ __forceinline__ uint4 ldg16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::evict_last.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& raw, float (&f)[Elem<T>::kVec]);
template <>
__device__ __forceinline__ void unpack16<float>(const uint4& raw, float (&f)[4]) {
    f[0] = __uint_as_float(raw.x);
    f[1] = __uint_as_float(raw.y);
    f[2] = __uint_as_float(raw.z);
    f[3] = __uint_as_float(raw.w);
}
template <>
__device__ __forceinline__ void unpack16<__half>(const uint4& raw, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& raw, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <typename T>
__device__ __forceinline__ uint4 pack16(const float (&f)[Elem<T>::kVec]);
template <>
__device__ __forceinline__ uint4 pack16<float>(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
}
template <>
__device__ __forceinline__ uint4 pack16<__half>(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------
// reductions into global memory (no return value): one 16-byte vector op per
// lane, so a group of lanes covering one row issues a single full-row request.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void red_add_f32x4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
                 "f"(d)
                 : "memory");
}
__device__ __forceinline__ void red_add_16x8(__half* p, const uint4& v) {
    asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void red_add_16x8(__nv_bfloat16* p, const uint4& v) {
    asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
                 "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Adds VEC consecutive fp32 contributions to an accumulation row whose element
// type is TG (fp32 scratch / fp32 grad_value, or the 16-bit grad_value itself).
template <typename TG, int VEC>
__device__ __forceinline__ void red_add_vec(TG* row, const float (&c)[VEC]);
template <>
__device__ __forceinline__ void red_add_vec<float, 4>(float* row, const float (&c)[4]) {
    red_add_f32x4(row, c[0], c[1], c[2], c[3]);
}
template <>
__device__ __forceinline__ void red_add_vec<float, 8>(float* row, const float (&c)[8]) {
    red_add_f32x4(row, c[0], c[1], c[2], c[3]);
    red_add_f32x4(row + 4, c[4], c[5], c[6], c[7]);
}
template <>
__device__ __forceinline__ void red_add_vec<__half, 8>(__half* row, const float (&c)[8]) {
    red_add_16x8(row, pack16<__half>(c));
}
template <>
__device__ __forceinline__ void red_add_vec<__nv_bfloat16, 8>(__nv_bfloat16* row,
                                                              const float (&c)[8]) {
    red_add_16x8(row, pack16<__nv_bfloat16>(c));
}

// Two fp32 multiply-adds in one instruction (Blackwell's packed fma.rn.f32x2):
// (a.x * b.x + c.x, a.y * b.y + c.y), each rounded once like fmaf.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    uint64_t ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
    uint64_t ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

// Stores two adjacent elements (x at p[0], y at p[1]) with one instruction.
__device__ __forceinline__ void store_pair(float* p, float x, float y) {
    *reinterpret_cast<float2*>(p) = make_float2(x, y);
}
__device__ __forceinline__ void store_pair(__half* p, float x, float y) {
    *reinterpret_cast<__half2*>(p) = __floats2half2_rn(x, y);
}
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float x, float y) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y);
}

__device__ __forceinline__ void red_add_scalar(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void red_add_scalar(__half* p, float v) {
    atomicAdd(p, __float2half_rn(v));
}
__device__ __forceinline__ void red_add_scalar(__nv_bfloat16* p, float v) {
    atomicAdd(p, __float2bfloat16_rn(v));
}

// ---------------------------------------------------------------------------
// bulk copy (TMA, non-tensor form) + mbarrier, all waits bounded
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// global -> this CTA's shared memory; source, destination and size must all be
// multiples of 16 bytes. Plain single-CTA form.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// Polls until the phase with the given parity completes, or `limit` polls have been made.
// Returns false on timeout; the caller falls back to plain loads.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int limit) {
    const uint32_t addr = smem_u32(bar);
    for (int spin = 0; spin < limit; ++spin) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// ---------------------------------------------------------------------------
// per-sample set-up: lane-parallel over the samples of one warp pass
// ---------------------------------------------------------------------------
struct SampleGeom {
    float lw, lh;  // fractional offsets inside the cell
    float a;       // attention weight (0 when the sample is dropped)
    float wf, hf;  // level width / height as floats
    float prob;    // fused variant: the sample's softmax probability, kept for dropped samples too
    int x0, y0;    // top-left pixel of the sample's cell (0 for a dropped sample)
    bool valid;
};

// Produces the four slot records of one sample: rec[c] = {offset of the corner's value row in
// `row_units` units, or kNoRow when that corner does not exist; bits of (bilinear weight *
// attention)}. row_base = (b*K + level_start)*H + h.
__device__ __forceinline__ void sample_setup(float lx, float ly, float a, int Wl, int Hl,
                                             uint32_t row_base, uint32_t H, uint32_t row_units,
                                             uint4& rec01, uint4& rec23, SampleGeom& g) {
    const float wf = static_cast<float>(Wl);
    const float hf = static_cast<float>(Hl);
    const float x = lx * wf - 0.5f;
    const float y = ly * hf - 0.5f;
    const bool valid = (x > -1.f) && (y > -1.f) && (x < wf) && (y < hf);
    const float x0f = floorf(x);
    const float y0f = floorf(y);
    // Fractions from one fused multiply-add each: lx*wf is taken exactly and
    // (x0f + 0.5) is exact, so lw/lh carry one rounding at their own magnitude
    // (< 1) instead of inheriting the rounding of x at magnitude ~W. The
    // gradients multiply these fractions by W*attn*(S differences), which
    // amplifies any error in them.
    const float lw = fmaf(lx, wf, -(x0f + 0.5f));
    const float lh = fmaf(ly, hf, -(y0f + 0.5f));
    const float hw = 1.f - lw;
    const float hh = 1.f - lh;
    // For dropped samples the coordinates may be NaN/Inf: keep the integer
    // conversion away from them.
    const int x0 = valid ? static_cast<int>(x0f) : 0;
    const int y0 = valid ? static_cast<int>(y0f) : 0;
    const bool x0ok = valid && x0 >= 0;
    const bool x1ok = valid && x0 + 1 <= Wl - 1;
    const bool y0ok = valid && y0 >= 0;
    const bool y1ok = valid && y0 + 1 <= Hl - 1;
    const uint32_t step_x = H * row_units;             // next pixel, same head
    const uint32_t step_y = static_cast<uint32_t>(Wl) * step_x;
    // (y0*Wl + x0) may be negative (x0 or y0 == -1); unsigned wrap-around is fine because a
    // record is only used when its corner exists, and then the sum is in range.
    const uint32_t o00 =
        (row_base + static_cast<uint32_t>(y0 * Wl + x0) * H) * row_units;
    // Selects, not multiplications by zero: lw/lh/a may be NaN or Inf here.
    const float aa = valid ? a : 0.f;
    rec01.x = (y0ok && x0ok) ? o00 : kNoRow;
    rec01.y = __float_as_uint(valid ? hh * hw * aa : 0.f);
    rec01.z = (y0ok && x1ok) ? o00 + step_x : kNoRow;
    rec01.w = __float_as_uint(valid ? hh * lw * aa : 0.f);
    rec23.x = (y1ok && x0ok) ? o00 + step_y : kNoRow;
    rec23.y = __float_as_uint(valid ? lh * hw * aa : 0.f);
    rec23.z = (y1ok && x1ok) ? o00 + step_y + step_x : kNoRow;
    rec23.w = __float_as_uint(valid ? lh * lw * aa : 0.f);
    g.lw = valid ? lw : 0.f;
    g.lh = valid ? lh : 0.f;
    g.a = aa;
    g.prob = a;
    g.wf = wf;
    g.hf = hf;
    g.x0 = x0;
    g.y0 = y0;
    g.valid = valid;
}

// MSDA_DEBUG_BOUNDS build (the stand-in for a memory checker where none can be run): every
// row offset a sample produced is checked against the extent of value / grad_value before
// anything is loaded from it or added to it. A violation sets kStatusOutOfBounds in the
// status word and turns the record into "no row", so the access never happens. A correct
// kernel on a consistent level table never trips it; the int32 offset arithmetic is the
// place the reference itself marks as hazardous (op_kernel/msda.h:428).
__device__ __forceinline__ void debug_check_rows(const Params& p, uint4& rec01, uint4& rec23) {
#ifdef MSDA_DEBUG_BOUNDS
    bool bad = false;
    auto check = [&](uint32_t& off) {
        if (off != kNoRow && (off >= p.limit_units || p.limit_units - off < p.row_units)) {
            bad = true;
            off = kNoRow;
        }
    };
    check(rec01.x);
    check(rec01.z);
    check(rec23.x);
    check(rec23.z);
    if (bad) atomicOr(p.status, kStatusOutOfBounds);
#else
    (void)p; (void)rec01; (void)rec23;
#endif
}

// Nearest-pixel variant (geometric kernel attention): the location holds pixel coordinates;
// they are truncated to integers and clamped into the level
// (kernels/geometric_kernel_attention/op_kernel/geometric_kernel_attention.cpp:123-159), so
// every sample has exactly one row. rec.x/.y = {row offset, attention weight bits}.
__device__ __forceinline__ void sample_setup_nearest(float lx, float ly, float a, int Wl, int Hl,
                                                     uint32_t row_base, uint32_t H,
                                                     uint32_t row_units, uint4& rec,
                                                     SampleGeom& g) {
    // __float2int_rz saturates and maps NaN to 0, so any input lands inside the level
    int x = __float2int_rz(lx);
    int y = __float2int_rz(ly);
    x = min(max(x, 0), Wl - 1);
    y = min(max(y, 0), Hl - 1);
    rec.x = (row_base + static_cast<uint32_t>(y * Wl + x) * H) * row_units;
    rec.y = __float_as_uint(a);
    g.lw = g.lh = 0.f;
    g.a = a;
    g.prob = a;
    g.wf = static_cast<float>(Wl);
    g.hf = static_cast<float>(Hl);
    g.x0 = x;
    g.y0 = y;
    g.valid = true;
}

}  // namespace msda

// Work decomposition shared by the forward and backward MSDA kernels.
//
// task  = one (batch, query, head) triple; tasks are numbered (b*Q + q)*H + h,
//         which is also the order of sampling_locations / attention_weights /
//         output / grad_output in memory.
// item  = what one warp handles in one pass: a single task when L*P >= 32
//         (in ceil(L*P/32) chunks of 32 samples), or floor(32 / (L*P))
//         consecutive tasks when L*P < 32, so that the lane-parallel set-up
//         keeps most lanes busy for small L*P. An item's locations and weights
//         are one contiguous range of memory.
// Warps are persistent: warp w of CTA c starts at item c*8 + w and advances by
// gridDim.x*8, so at any moment the whole GPU works on neighbouring queries of
// the same batch entry and that entry's value pyramid stays L2-resident.
//
// While a warp gathers for its current item, the locations and weights of its
// next item are already on their way: one lane issues two bulk copies
// (cp.async.bulk, global -> shared, completion on a per-warp mbarrier) into
// the warp's other staging buffer. Where an item's byte ranges are not
// multiples of 16 (odd L*P with odd task counts, misaligned tensors) the warp
// loads its samples directly instead.
#pragma once

#include "msda_common.cuh"

namespace msda {

// Per-lane level geometry. With lane -> sample fixed for the whole kernel the
// level of a lane never changes, so it is looked up once.
struct LaneLevels {
    int w0, h0, start0;  // chunk 0 (samples 0..31, or the only chunk)
    int w1, h1, start1;  // chunk 1 (samples 32..63)
    int level0;          // level index of the lane's chunk-0 sample (fused variant)
    __device__ __forceinline__ int w(int c) const { return c ? w1 : w0; }
    __device__ __forceinline__ int h(int c) const { return c ? h1 : h0; }
    __device__ __forceinline__ int start(int c) const { return c ? start1 : start0; }
};

// Which (task within the item, sample within the task) a lane handles in a chunk.
__device__ __forceinline__ void lane_sample_index(const Params& p, int chunk, int lane,
                                                  int& task_local, int& s) {
    if (p.tasks_per_item == 1) {
        task_local = 0;
        s = chunk * kChunk + lane;
    } else {
        task_local = static_cast<int>(fd_div(static_cast<uint32_t>(lane), p.fd_lp));
        s = lane - task_local * p.LP;
    }
}

__device__ __forceinline__ LaneLevels load_lane_levels(const Params& p, int lane) {
    LaneLevels lv;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        int tl, s;
        lane_sample_index(p, c, lane, tl, s);
        int l = s / p.P;
        if (l >= p.L) l = p.L - 1;  // inactive lane; any in-range level will do
        int hh, ww, ss;
        if (p.use_table) {
            hh = p.lv.h[l];
            ww = p.lv.w[l];
            ss = p.lv.start[l];
        } else {
            hh = p.shapes_dev[2 * l];
            ww = p.shapes_dev[2 * l + 1];
            ss = p.start_dev[l];
        }
        if (c == 0) {
            lv.h0 = hh; lv.w0 = ww; lv.start0 = ss;
            lv.level0 = l;
        } else {
            lv.h1 = hh; lv.w1 = ww; lv.start1 = ss;
        }
    }
    return lv;
}

// Level tables passed in device memory cannot be checked by the host without a
// synchronisation, so every CTA checks them before it touches anything (L <= 64 entries): a
// size <= 0, a negative start or start + h*w > K sets kStatusBadLevels and makes the kernel
// return. All threads of the CTA must call it.
__device__ __forceinline__ bool device_level_table_ok(const Params& p) {
    if (p.use_table) return true;   // host tables were validated by the entry point
    bool bad = false;
    for (int l = threadIdx.x; l < p.L; l += blockDim.x) {
        const int hh = p.shapes_dev[2 * l], ww = p.shapes_dev[2 * l + 1], ss = p.start_dev[l];
        bad |= hh <= 0 || ww <= 0 || ss < 0 ||
               static_cast<long long>(ss) + static_cast<long long>(hh) * ww > p.K;
    }
    const bool any = __syncthreads_or(bad ? 1 : 0) != 0;
    if (any && threadIdx.x == 0) atomicOr(p.status, kStatusBadLevels);
    return !any;
}

// The sequence of items one warp walks through: warp w of CTA c takes items c*8 + w, then
// + gridDim*8, ... (a CTA's eight warps hold eight consecutive tasks, i.e. with eight heads all
// heads of one query).
struct ItemWalk {
    long long idx, stride, end;
    __device__ __forceinline__ long long item(const Params& p) const { return item_at(p, idx); }
    // Items are walked in memory order, which keeps the batch entry in flight L2-resident, or
    // - when the host found the whole value tensor small enough to stay in L2 anyway - with
    // the batch entries interleaved, so that the reductions of the warps in flight spread
    // over all entries' gradient maps instead of piling onto one entry's few rows.
    __device__ __forceinline__ long long item_at(const Params& p, long long i) const {
        if (p.walk_b == 0) return i;
        const uint32_t q = fd_div(static_cast<uint32_t>(i), p.fd_walk_b);
        const uint32_t r = static_cast<uint32_t>(i) - q * p.walk_b;
        return static_cast<long long>(r) * p.walk_items_per_b + q;
    }
};
__device__ __forceinline__ ItemWalk make_walk(const Params& p, int warp) {
    ItemWalk w;
    w.idx = static_cast<long long>(blockIdx.x) * kWarpsPerCta + warp;
    w.stride = static_cast<long long>(gridDim.x) * kWarpsPerCta;
    w.end = p.nitems;
    return w;
}

// Shared memory of one warp, in this order (all 16-byte aligned):
//   uint2 slot[kSlots + kSlotPad] records of the current chunk (+ padding) 1536 B
//   [backward only] float part[]  partial dot products                   part_bytes
//   uint64_t bar[2]               staging barriers                       16 B
//   T stage[2][3 * SPI]           staged (x, y) pairs then weights, SPI = samples per item
constexpr int kSlotBytes = (kSlots + kSlotPad) * 8;

__host__ __device__ inline uint32_t stage_bytes_per_buffer(int samples_per_item, size_t e) {
    return static_cast<uint32_t>((3 * samples_per_item * e + 15) & ~size_t(15));
}
__host__ __device__ inline uint32_t warp_smem_bytes(int samples_per_item, size_t e,
                                                    uint32_t part_bytes) {
    return kSlotBytes + part_bytes + 16 + 2 * stage_bytes_per_buffer(samples_per_item, e);
}

// Per-warp staging state. Only the two pointers and the flag live in registers; sizes are
// recomputed from the kernel parameters (constant bank) where needed.
template <typename T>
struct WarpStage {
    uint64_t* bar;       // [2], followed by the two buffers
    bool ok;             // staging in use (cleared for good after a timeout)

    __device__ __forceinline__ static uint32_t attn_bytes(const Params& p) {
        return static_cast<uint32_t>(p.tasks_per_item * p.LP * sizeof(T));
    }
    __device__ __forceinline__ unsigned char* buffer(const Params& p, int b) const {
        return reinterpret_cast<unsigned char*>(bar) + 16 +
               b * stage_bytes_per_buffer(p.tasks_per_item * p.LP, sizeof(T));
    }
    __device__ __forceinline__ const T* loc(const Params& p, int b) const {
        return reinterpret_cast<const T*>(buffer(p, b));
    }
    __device__ __forceinline__ const T* attn(const Params& p, int b) const {
        return reinterpret_cast<const T*>(buffer(p, b) + 2 * attn_bytes(p));
    }
    // lane 0 only
    __device__ __forceinline__ void issue(const Params& p, long long item, int b) const {
        const long long spi = static_cast<long long>(p.tasks_per_item) * p.LP;
        const T* gl = static_cast<const T*>(p.loc) + item * spi * 2;
        const T* ga = static_cast<const T*>(p.attn) + item * spi;
        const uint32_t ab = attn_bytes(p);
        unsigned char* dst = buffer(p, b);
        mbar_expect_tx(bar + b, 3 * ab);
        bulk_g2s(dst, gl, 2 * ab, bar + b);
        bulk_g2s(dst + 2 * ab, ga, ab, bar + b);
    }
    // After a time-out on buffer `b` (use number n of the barriers): the warp stops staging,
    // but the copies it has already issued still target its buffers. Wait for them (bounded,
    // with a far larger limit) so that none is in flight when the CTA exits and its shared
    // memory is handed to another CTA. All lanes call it.
    __device__ __forceinline__ void drain(int b, int n, bool next_issued) const {
        mbar_wait(bar + b, (n >> 1) & 1, kDrainLimit);
        if (next_issued) mbar_wait(bar + (b ^ 1), ((n + 1) >> 1) & 1, kDrainLimit);
        __syncwarp();
    }
};

template <typename T>
__device__ __forceinline__ WarpStage<T> warp_stage_init(const Params& p, unsigned char* base,
                                                        int lane) {
    WarpStage<T> st;
    st.bar = reinterpret_cast<uint64_t*>(base);
    st.ok = p.stage != 0;
    if (st.ok) {
        if (lane == 0) {
            mbar_init(st.bar, 1);
            mbar_init(st.bar + 1, 1);
            mbar_fence_init();
        }
        __syncwarp();
    }
    return st;
}

// With one record per sample (CPS == 1) a chunk writes only the first 32 slots; the gather
// loop of a single-task item may read up to a full trip beyond its last sample, so the
// other slots are set to "no row" once.
template <int CPS>
__device__ __forceinline__ void init_unused_slots(uint2* s_slot, int lane) {
    if constexpr (CPS == 1) {
#pragma unroll
        for (int i = kChunk; i < kSlots + kSlotPad; i += 32) s_slot[i + lane] = make_uint2(kNoRow, 0u);
        __syncwarp();
    }
}

// Sum / maximum over the samples of this lane's task. With one task per item that is the whole
// warp (inactive lanes must hold the neutral element); with several tasks per item the
// values go through `scratch` (32 floats of the warp's shared memory) and every lane walks
// its own task's segment.
__device__ __forceinline__ float task_sum(const Params& p, float v, int lane, int tl,
                                          float* scratch) {
    if (p.tasks_per_item == 1) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        return v;
    }
    __syncwarp();
    scratch[lane] = v;
    __syncwarp();
    float acc = 0.f;
    const int begin = min(tl, p.tasks_per_item - 1) * p.LP;
    for (int i = 0; i < p.LP; ++i) acc += scratch[begin + i];
    return acc;
}
__device__ __forceinline__ float task_max(const Params& p, float v, int lane, int tl,
                                          float* scratch) {
    if (p.tasks_per_item == 1) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1)
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
        return v;
    }
    __syncwarp();
    scratch[lane] = v;
    __syncwarp();
    float acc = -INFINITY;
    const int begin = min(tl, p.tasks_per_item - 1) * p.LP;
    for (int i = 0; i < p.LP; ++i) acc = fmaxf(acc, scratch[begin + i]);
    return acc;
}
// The 64 padding records behind the slot array double as 128 floats of per-warp scratch for
// the fused variant (the gather loop may read them as records, but never uses what it reads).
__device__ __forceinline__ float* fused_scratch(uint2* s_slot) {
    return reinterpret_cast<float*>(s_slot + kSlots);
}

// Where this lane's records start and how many records the chunk has, when phase 1 packs
// the existing corners' records (see there).
struct Compaction {
    int first, rows;
};

// Phase 1 of one chunk: lane = sample. Obtains (x, y, weight) — from the staged buffer or
// directly — and leaves the sample's slot records in shared memory: four (bilinear corners)
// for CPS == 4, one (clamped integer pixel) for CPS == 1. Returns whether this lane holds a
// sample; `gi` is its global sample index. FUSED: the staged/loaded pair is a sampling
// offset and the scalar a logit; the location is reference point + offset / (W, H) of the
// level and the weight the softmax of the task's logits (what the callers of MSDA compute
// in separate kernels: mmcv's MultiScaleDeformableAttention.forward).
template <typename T, int CPS, bool FUSED>
__device__ __forceinline__ bool phase1(const Params& p, const LaneLevels& lv, int chunk, int lane,
                                       long long item, int ntask_here, const T* sloc,
                                       const T* sattn, uint2* s_slot, SampleGeom& geom,
                                       long long& gi, Compaction* compact = nullptr) {
    int tl, s;
    lane_sample_index(p, chunk, lane, tl, s);
    const bool active = (tl < ntask_here) && (s < p.LP);
    uint4 rec01 = make_uint4(kNoRow, 0u, kNoRow, 0u);
    uint4 rec23 = rec01;
    geom.lw = geom.lh = geom.a = geom.wf = geom.hf = geom.prob = 0.f;
    geom.valid = false;
    gi = 0;
    float lx = 0.f, ly = 0.f, a = FUSED ? -INFINITY : 0.f;
    uint32_t t = 0;
    if (active) {
        t = static_cast<uint32_t>(item) * p.tasks_per_item + tl;
        gi = static_cast<long long>(t) * p.LP + s;
        if (sloc != nullptr) {
            const int li = tl * p.LP + s;
            lx = Elem<T>::to_f(sloc[2 * li]);
            ly = Elem<T>::to_f(sloc[2 * li + 1]);
            a = Elem<T>::to_f(sattn[li]);
        } else {
            const T* gl = static_cast<const T*>(p.loc);
            lx = Elem<T>::to_f(gl[2 * gi]);
            ly = Elem<T>::to_f(gl[2 * gi + 1]);
            a = Elem<T>::to_f(static_cast<const T*>(p.attn)[gi]);
        }
    }
    if constexpr (FUSED) {
        // softmax over the task's L*P logits (all lanes take part in the reductions)
        float* scratch = fused_scratch(s_slot);
        const float m = task_max(p, a, lane, tl, scratch);
        const float e = active ? __expf(a - m) : 0.f;
        const float sum = task_sum(p, e, lane, tl, scratch);
        a = active ? e / sum : 0.f;
    }
    if (active) {
        const uint32_t b = fd_div(t, p.fd_qh);
        const uint32_t bq = fd_div(t, p.fd_h);          // b * Q + q
        const uint32_t h = t - bq * p.H;
        const int c = (p.tasks_per_item == 1) ? chunk : 0;
        if constexpr (FUSED) {
            const T* ref = static_cast<const T*>(p.ref) +
                           (static_cast<size_t>(bq) * p.L + lv.level0) * 2;
            lx = Elem<T>::to_f(ref[0]) + lx / static_cast<float>(lv.w(c));
            ly = Elem<T>::to_f(ref[1]) + ly / static_cast<float>(lv.h(c));
        }
        const uint32_t row_base =
            (b * static_cast<uint32_t>(p.K) + static_cast<uint32_t>(lv.start(c))) * p.H + h;
        if constexpr (CPS == 4) {
            sample_setup(lx, ly, a, lv.w(c), lv.h(c), row_base, static_cast<uint32_t>(p.H),
                         p.row_units, rec01, rec23, geom);
        } else {
            sample_setup_nearest(lx, ly, a, lv.w(c), lv.h(c), row_base,
                                 static_cast<uint32_t>(p.H), p.row_units, rec01, geom);
        }
        debug_check_rows(p, rec01, rec23);
    }
    if constexpr (CPS == 4) {
        if (compact != nullptr) {
            // Only the corners that exist get a record, packed from slot 0 on in (sample,
            // corner) order; the gather loop then walks compact->rows records instead of
            // 4 per sample (and must not read past them: what follows is stale).
            const bool c0 = rec01.x != kNoRow, c1 = rec01.z != kNoRow;
            const bool c2 = rec23.x != kNoRow, c3 = rec23.z != kNoRow;
            const uint32_t b0 = __ballot_sync(0xffffffffu, c0), b1 = __ballot_sync(0xffffffffu, c1);
            const uint32_t b2 = __ballot_sync(0xffffffffu, c2), b3 = __ballot_sync(0xffffffffu, c3);
            const uint32_t below = (1u << lane) - 1u;
            int pos = __popc(b0 & below) + __popc(b1 & below) + __popc(b2 & below) +
                      __popc(b3 & below);
            const int rows = __popc(b0) + __popc(b1) + __popc(b2) + __popc(b3);
            compact->first = pos;
            compact->rows = rows;
            if (c0) s_slot[pos++] = make_uint2(rec01.x, rec01.y);
            if (c1) s_slot[pos++] = make_uint2(rec01.z, rec01.w);
            if (c2) s_slot[pos++] = make_uint2(rec23.x, rec23.y);
            if (c3) s_slot[pos] = make_uint2(rec23.z, rec23.w);
        } else {
            uint4* dst = reinterpret_cast<uint4*>(s_slot) + 2 * lane;
            dst[0] = rec01;
            dst[1] = rec23;
        }
    } else {
        s_slot[lane] = make_uint2(rec01.x, rec01.y);
    }
    return active;
}

}  // namespace msda

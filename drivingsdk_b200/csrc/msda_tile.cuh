// Work decomposition shared by the forward and backward MSDA kernels.
//
// task  = one (batch, query, head) triple; tasks are numbered (b*Q + q)*H + h,
//         which is also the order of sampling_locations / attention_weights /
//         output / grad_output in memory.
// item  = what one warp handles in one pass: a single task when L*P >= 32
//         (in ceil(L*P/32) chunks of 32 samples), or floor(32 / (L*P))
//         consecutive tasks when L*P < 32, so that the lane-parallel set-up
//         keeps most lanes busy for small L*P.
// tile  = kWarpsPerCta consecutive items, one per warp of a CTA; its locations
//         and weights are one contiguous range, which is what the bulk copy
//         stages into shared memory.
// CTAs walk tiles in increasing order with a grid stride, so at any moment the
// whole GPU works on neighbouring queries of the same batch entry and that
// entry's value pyramid stays L2-resident.
#pragma once

#include "msda_common.cuh"

namespace msda {

// Per-lane level geometry. With lane -> sample fixed for the whole kernel the
// level of a lane never changes, so it is looked up once.
struct LaneLevels {
    int w0, h0, start0;  // chunk 0 (samples 0..31, or the only chunk)
    int w1, h1, start1;  // chunk 1 (samples 32..63)
    __device__ __forceinline__ int w(int c) const { return c ? w1 : w0; }
    __device__ __forceinline__ int h(int c) const { return c ? h1 : h0; }
    __device__ __forceinline__ int start(int c) const { return c ? start1 : start0; }
};

__device__ __forceinline__ void lane_sample_index(const Params& p, int chunk, int lane,
                                                  int& task_local, int& s) {
    if (p.tasks_per_item == 1) {
        task_local = 0;
        s = chunk * kChunk + lane;
    } else {
        task_local = lane / p.LP;
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
        } else {
            lv.h1 = hh; lv.w1 = ww; lv.start1 = ss;
        }
    }
    return lv;
}

// Double-buffered staging of one tile's locations and weights.
template <typename T>
struct Stage {
    T* loc0;        // buffer 0 of the location tile; buffer 1 follows it
    T* attn0;       // buffer 0 of the weight tile; buffer 1 follows it
    uint64_t* bar;  // two barriers
    uint32_t loc_bytes, attn_bytes;
    long long samples_per_tile;
    long long total_samples;
    bool enabled;

    __device__ __forceinline__ bool full(long long tile) const {
        return (tile + 1) * samples_per_tile <= total_samples;
    }
    __device__ __forceinline__ T* loc(int buf) const { return loc0 + buf * 2 * samples_per_tile; }
    __device__ __forceinline__ T* attn(int buf) const { return attn0 + buf * samples_per_tile; }
    __device__ __forceinline__ void issue(const Params& p, long long tile, int buf) const {
        const T* gl = static_cast<const T*>(p.loc) + tile * samples_per_tile * 2;
        const T* ga = static_cast<const T*>(p.attn) + tile * samples_per_tile;
        mbar_expect_tx(bar + buf, loc_bytes + attn_bytes);
        bulk_g2s(loc(buf), gl, loc_bytes, bar + buf);
        bulk_g2s(attn(buf), ga, attn_bytes, bar + buf);
    }
};

// Carves the staging buffers out of dynamic shared memory (16-byte aligned)
// and initialises the barriers. Must be called by all threads of the CTA.
template <typename T>
__device__ __forceinline__ Stage<T> stage_init(const Params& p, unsigned char* smem) {
    Stage<T> st;
    st.samples_per_tile = static_cast<long long>(kWarpsPerCta) * p.tasks_per_item * p.LP;
    st.total_samples = p.ntasks * p.LP;
    st.attn_bytes = static_cast<uint32_t>(st.samples_per_tile * sizeof(T));
    st.loc_bytes = 2 * st.attn_bytes;
    st.enabled = p.stage != 0;
    st.bar = reinterpret_cast<uint64_t*>(smem);
    unsigned char* q = smem + 16;
    st.loc0 = reinterpret_cast<T*>(q);
    st.attn0 = reinterpret_cast<T*>(q + 2 * st.loc_bytes);
    if (st.enabled) {
        if (threadIdx.x == 0) {
            mbar_init(&st.bar[0], 1);
            mbar_init(&st.bar[1], 1);
            mbar_fence_init();
        }
        __syncthreads();
    }
    return st;
}

// Bytes of dynamic shared memory stage_init() consumes for element size e.
__host__ __device__ inline size_t stage_smem_bytes(int tasks_per_item, int LP, size_t e) {
    const size_t samples = static_cast<size_t>(kWarpsPerCta) * tasks_per_item * LP;
    return 16 + 2 * 3 * samples * e;
}

}  // namespace msda

// C-ABI entry points of the sm_100a MSDA library: argument validation, the
// launch plan (what the reference computes in its host tiling functions,
// kernels/multi_scale_deformable_attn/op_host/multi_scale_deformable_attn.cpp:32-114
// and multi_scale_deformable_attn_grad.cpp:35-86), and kernel launches.
// No allocation, no synchronisation (except msda_sm100_device_status).
#include <atomic>
#include <cstring>

#include "../../include/msda_sm100.h"
#include "msda_launch.h"

namespace {

using msda::Params;
using msda::RowPlan;

constexpr int kAbiVersion = 1;
constexpr int kBilinear = 0, kNearest = 1, kFused = 2;
constexpr int kMaxDevices = 64;

__device__ int g_status_word;

std::atomic<int> g_tune_stage{2};   // 0 never, 1 both directions, 2 backward kernels only
std::atomic<int> g_tune_interleave{1};
std::atomic<int> g_tune_cps_fwd{0};
std::atomic<int> g_tune_cps_bwd{0};
std::atomic<int> g_tune_spin{msda::kSpinLimit};
std::atomic<int> g_tune_precise_amp{8};
std::atomic<int> g_tune_debug_rows{0};
std::atomic<int> g_tune_pack{1};
std::atomic<long long> g_launches{0};
thread_local int t_last_cuda_error = 0;
thread_local cudaEvent_t t_prof[4] = {nullptr, nullptr, nullptr, nullptr};

void prof_record(int which, cudaStream_t stream) {
    if (t_prof[which] != nullptr) cudaEventRecord(t_prof[which], stream);
}

struct DeviceInfo {
    std::atomic<int> ready{0};
    int sm_count = 0;
    int* status_ptr = nullptr;
};
DeviceInfo g_dev[kMaxDevices];

int fail_cuda(cudaError_t e) {
    t_last_cuda_error = static_cast<int>(e);
    return MSDA_ERR_CUDA;
}

// Per-device facts (SM count, address of the status word), looked up once.
// Racing first calls do the same idempotent work.
int device_info(const DeviceInfo** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda(e);
    if (dev < 0 || dev >= kMaxDevices) return MSDA_ERR_LIMIT;
    DeviceInfo& d = g_dev[dev];
    if (!d.ready.load(std::memory_order_acquire)) {
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail_cuda(e);
        void* sp = nullptr;
        e = cudaGetSymbolAddress(&sp, g_status_word);
        if (e != cudaSuccess) return fail_cuda(e);
        d.sm_count = sms;
        d.status_ptr = static_cast<int*>(sp);
        d.ready.store(1, std::memory_order_release);
    }
    *out = &d;
    return MSDA_OK;
}

size_t elem_size(int dtype) { return dtype == MSDA_F32 ? 4 : 2; }

bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Is this pointer device-accessible memory (device or managed)? Unregistered
// host memory reports cudaMemoryTypeUnregistered.
int pointer_on_device(const void* p, bool* on_device) {
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *on_device = false;
        return MSDA_OK;
    }
    *on_device = (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged);
    return MSDA_OK;
}

int check_dims(int B, int K, int H, int D, int L, int Q, int P, int dtype) {
    if (dtype != MSDA_F32 && dtype != MSDA_F16 && dtype != MSDA_BF16) return MSDA_ERR_DTYPE;
    if (B <= 0 || K <= 0 || H <= 0 || D <= 0 || L <= 0 || Q <= 0 || P <= 0) return MSDA_ERR_DIMS;
    if (D > 256 || static_cast<long long>(L) * P > 64 || L > msda::kMaxLevels) return MSDA_ERR_LIMIT;
    const long long rows = static_cast<long long>(B) * K * H;
    const long long tasks = static_cast<long long>(B) * Q * H;
    if (rows >= (1LL << 31) || tasks >= (1LL << 31)) return MSDA_ERR_LIMIT;
    return MSDA_OK;
}

RowPlan plan_rows(int D, int dtype, bool ptrs_16B_aligned) {
    RowPlan rp{true, 32, 8};
    const size_t row_bytes = static_cast<size_t>(D) * elem_size(dtype);
    if (!ptrs_16B_aligned || row_bytes % 16 != 0) return rp;
    const size_t pieces = row_bytes / 16;
    if ((pieces & (pieces - 1)) != 0 || pieces > 64) return rp;
    rp.scalar = false;
    rp.lpr = pieces < 32 ? static_cast<int>(pieces) : 32;
    rp.nv = static_cast<int>(pieces) / rp.lpr;
    return rp;
}

// Offsets of value rows travel as 32-bit counts of `row_units`: 16-byte pieces on the vector
// path, elements on the scalar path.
int set_row_units(Params& p, const RowPlan& rp, int dtype) {
    const unsigned long long units =
        rp.scalar ? static_cast<unsigned long long>(p.D)
                  : static_cast<unsigned long long>(p.D) * elem_size(dtype) / 16;
    const unsigned long long rows = static_cast<unsigned long long>(p.B) * p.K * p.H;
    if (rows * units >= 0xffffffffull) return MSDA_ERR_LIMIT;
    p.row_units = static_cast<uint32_t>(units);
    p.limit_units = static_cast<uint32_t>(rows * units);
#ifdef MSDA_DEBUG_BOUNDS
    // test hook of the bounds-checking build: pretend value / grad_value end after this many rows
    const unsigned long long pretend = static_cast<unsigned long long>(g_tune_debug_rows.load());
    if (pretend > 0 && pretend < rows) p.limit_units = static_cast<uint32_t>(pretend * units);
#endif
    return MSDA_OK;
}

// Fills the parts of Params common to both directions.
int fill_common(Params& p, const DeviceInfo* dev, const void* value, const int32_t* shapes,
                const int32_t* starts, const void* loc, const void* attn, int B, int K, int H,
                int D, int L, int Q, int P, int dtype, bool backward) {
    std::memset(&p, 0, sizeof(p));
    p.value = value;
    p.loc = loc;
    p.attn = attn;
    p.B = B; p.K = K; p.H = H; p.D = D; p.L = L; p.Q = Q; p.P = P;
    p.LP = L * P;
    p.tasks_per_item = (p.LP >= msda::kChunk) ? 1 : (msda::kChunk / p.LP);
    p.ntasks = static_cast<long long>(B) * Q * H;
    p.nitems = (p.ntasks + p.tasks_per_item - 1) / p.tasks_per_item;
    p.status = dev->status_ptr;

    bool shapes_dev = false, starts_dev = false;
    pointer_on_device(shapes, &shapes_dev);
    pointer_on_device(starts, &starts_dev);
    if (shapes_dev != starts_dev) return MSDA_ERR_ALIGN;  // both host or both device
    if (shapes_dev) {
        p.use_table = 0;
        p.shapes_dev = shapes;
        p.start_dev = starts;
    } else {
        p.use_table = 1;
        for (int l = 0; l < L; ++l) {
            p.lv.h[l] = shapes[2 * l];
            p.lv.w[l] = shapes[2 * l + 1];
            p.lv.start[l] = starts[l];
            if (p.lv.h[l] <= 0 || p.lv.w[l] <= 0 || p.lv.start[l] < 0 ||
                static_cast<long long>(p.lv.start[l]) + static_cast<long long>(p.lv.h[l]) * p.lv.w[l] > K)
                return MSDA_ERR_DIMS;
        }
    }
    const size_t e = elem_size(dtype);
    // Interleave the batch entries in the walk when all of value stays in L2 whatever the
    // order (16 MiB: measured neutral to harmful from 17 MiB up, a large gain for small maps), every entry holds a whole number of items, and the
    // counters fit the 32-bit fast division.
    p.walk_b = 0;
    p.walk_items_per_b = 0;
    p.fd_walk_b = msda::make_fastdiv(1);
    {
        const long long tasks_per_b = static_cast<long long>(Q) * H;
        const size_t value_bytes = static_cast<size_t>(B) * K * H * D * e;
        if (g_tune_interleave.load() != 0 && B > 1 && value_bytes <= (16u << 20) &&
            tasks_per_b % p.tasks_per_item == 0 && p.nitems < (1ll << 31)) {
            p.walk_b = static_cast<uint32_t>(B);
            p.walk_items_per_b = static_cast<uint32_t>(tasks_per_b / p.tasks_per_item);
            p.fd_walk_b = msda::make_fastdiv(static_cast<uint32_t>(B));
        }
    }
    p.fd_qh = msda::make_fastdiv(static_cast<uint32_t>(Q) * static_cast<uint32_t>(H));
    p.fd_h = msda::make_fastdiv(static_cast<uint32_t>(H));
    p.fd_lp = msda::make_fastdiv(static_cast<uint32_t>(p.LP));
    // Bulk-copy staging needs 16-byte aligned sources and sizes: per item the weights take
    // samples * e bytes and the locations twice that.
    const size_t item_attn_bytes = static_cast<size_t>(p.tasks_per_item) * p.LP * e;
    const int stage_mode = g_tune_stage.load();
    p.stage = ((stage_mode == 1 || (stage_mode == 2 && backward)) && aligned_to(loc, 16) &&
               aligned_to(attn, 16) && item_attn_bytes % 16 == 0)
                  ? 1
                  : 0;
    p.spin_limit = g_tune_spin.load();
    p.pack_rows = g_tune_pack.load() != 0 ? 1 : 0;
    p.precise_amp = static_cast<float>(g_tune_precise_amp.load());
    if (!aligned_to(value, e) || !aligned_to(loc, e) || !aligned_to(attn, e)) return MSDA_ERR_ALIGN;
    return MSDA_OK;
}

int backward_impl(const void* value, const int32_t* shapes, const int32_t* starts, const void* loc,
                  const void* attn, const void* grad_out, void* grad_value, void* grad_loc,
                  void* grad_attn, void* workspace, size_t workspace_bytes, bool use_ws, int mode,
                  const void* ref, float* grad_ref, int B, int K, int H, int D, int L, int Q,
                  int P, int dtype, void* stream_v) {
    // mode: kBilinear = MSDA; kNearest = geometric kernel attention (one clamped integer pixel
    // per sample, no location gradient); kFused = MSDA fed by reference points, offsets (in
    // `loc`) and logits (in `attn`)
    const bool nearest = mode == kNearest;
    if (!value || !shapes || !starts || !loc || !attn || !grad_out || !grad_value || !grad_attn ||
        (!nearest && !grad_loc) || (mode == kFused && (!ref || !grad_ref)))
        return MSDA_ERR_NULL;
    if (mode == kFused && static_cast<long long>(L) * P > 32) return MSDA_ERR_LIMIT;
    int rc = check_dims(B, K, H, D, L, Q, P, dtype);
    if (rc != MSDA_OK) return rc;
    const DeviceInfo* dev = nullptr;
    rc = device_info(&dev);
    if (rc != MSDA_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    Params p;
    rc = fill_common(p, dev, value, shapes, starts, loc, attn, B, K, H, D, L, Q, P, dtype, true);
    if (rc != MSDA_OK) return rc;
    const size_t e = elem_size(dtype);
    if (!aligned_to(grad_out, e) || !aligned_to(grad_value, e) || !aligned_to(grad_attn, e) ||
        (!nearest && !aligned_to(grad_loc, 2 * e)))
        return MSDA_ERR_ALIGN;

    const long long nval = static_cast<long long>(B) * K * H * D;
    const bool acc_f32 = use_ws && dtype != MSDA_F32;
    void* acc = grad_value;
    size_t acc_bytes = static_cast<size_t>(nval) * e;
    if (acc_f32) {
        const size_t need = static_cast<size_t>(nval) * sizeof(float);
        if (!workspace || workspace_bytes < need || !aligned_to(workspace, 16))
            return MSDA_ERR_WORKSPACE;
        acc = workspace;
        acc_bytes = need;
    }
    const bool vec_ok = aligned_to(value, 16) && aligned_to(grad_out, 16) && aligned_to(acc, 16);
    const RowPlan rp = plan_rows(D, dtype, vec_ok);

    rc = set_row_units(p, rp, dtype);
    if (rc != MSDA_OK) return rc;
    p.warp_smem = msda::bwd_warp_smem(p.tasks_per_item * p.LP, e);
    p.grad_out = grad_out;
    p.grad_value = acc;
    p.grad_loc = grad_loc;
    p.grad_attn = grad_attn;

    cudaError_t ce = cudaMemsetAsync(acc, 0, acc_bytes, stream);
    if (ce != cudaSuccess) return fail_cuda(ce);
    prof_record(2, stream);
    const msda::LaunchShape shape{dev->sm_count, g_tune_cps_bwd.load()};
    if (mode == kFused) {
        p.ref = ref;
        p.grad_ref = grad_ref;
        ce = cudaMemsetAsync(grad_ref, 0, static_cast<size_t>(B) * Q * L * 2 * sizeof(float),
                             stream);
        if (ce != cudaSuccess) return fail_cuda(ce);
        ce = msda::launch_fused_backward(p, dtype, acc_f32 ? 1 : 0, rp, shape, stream);
    } else if (nearest) {
        ce = msda::launch_gka_backward(p, dtype, acc_f32 ? 1 : 0, rp, shape, stream);
    } else {
        ce = msda::launch_backward(p, dtype, acc_f32 ? 1 : 0, rp, shape, stream);
    }
    prof_record(3, stream);
    if (ce != cudaSuccess) return fail_cuda(ce);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (acc_f32) {
        ce = msda::launch_downcast(static_cast<const float*>(acc), grad_value, nval, dtype, stream);
        if (ce != cudaSuccess) return fail_cuda(ce);
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return MSDA_OK;
}

int forward_impl(const void* value, const int32_t* spatial_shapes,
                 const int32_t* level_start_index, const void* sampling_locations,
                 const void* attention_weights, void* output, int mode, const void* ref, int B,
                 int K, int H, int D, int L, int Q, int P, int dtype, void* stream_v) {
    if (mode == kFused && (!ref || static_cast<long long>(L) * P > 32))
        return ref ? MSDA_ERR_LIMIT : MSDA_ERR_NULL;
    if (!value || !spatial_shapes || !level_start_index || !sampling_locations ||
        !attention_weights || !output)
        return MSDA_ERR_NULL;
    int rc = check_dims(B, K, H, D, L, Q, P, dtype);
    if (rc != MSDA_OK) return rc;
    const DeviceInfo* dev = nullptr;
    rc = device_info(&dev);
    if (rc != MSDA_OK) return rc;

    Params p;
    rc = fill_common(p, dev, value, spatial_shapes, level_start_index, sampling_locations,
                     attention_weights, B, K, H, D, L, Q, P, dtype, false);
    if (rc != MSDA_OK) return rc;
    if (!aligned_to(output, elem_size(dtype))) return MSDA_ERR_ALIGN;
    p.out = output;
    const RowPlan rp = plan_rows(D, dtype, aligned_to(value, 16) && aligned_to(output, 16));
    rc = set_row_units(p, rp, dtype);
    if (rc != MSDA_OK) return rc;
    p.warp_smem = msda::fwd_warp_smem(p.tasks_per_item * p.LP, elem_size(dtype));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    prof_record(0, stream);
    const msda::LaunchShape shape{dev->sm_count, g_tune_cps_fwd.load()};
    p.ref = ref;
    cudaError_t ce = mode == kFused     ? msda::launch_fused_forward(p, dtype, rp, shape, stream)
                     : mode == kNearest ? msda::launch_gka_forward(p, dtype, rp, shape, stream)
                                        : msda::launch_forward(p, dtype, rp, shape, stream);
    prof_record(1, stream);
    if (ce != cudaSuccess) return fail_cuda(ce);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return MSDA_OK;
}

}  // namespace

namespace msda {
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int note_cuda_error(cudaError_t e) { return fail_cuda(e); }
int device_facts(int* sm_count, int** status_word) {
    const DeviceInfo* d = nullptr;
    const int rc = device_info(&d);
    if (rc != MSDA_OK) return rc;
    if (sm_count != nullptr) *sm_count = d->sm_count;
    if (status_word != nullptr) *status_word = d->status_ptr;
    return MSDA_OK;
}
}  // namespace msda

extern "C" {

int msda_sm100_forward(const void* value, const int32_t* spatial_shapes,
                       const int32_t* level_start_index, const void* sampling_locations,
                       const void* attention_weights, void* output, int B, int K, int H, int D,
                       int L, int Q, int P, int dtype, void* stream) {
    return forward_impl(value, spatial_shapes, level_start_index, sampling_locations,
                        attention_weights, output, kBilinear, nullptr, B, K, H, D, L, Q, P, dtype,
                        stream);
}

int gka_sm100_forward(const void* value, const int32_t* spatial_shapes,
                      const int32_t* level_start_index, const void* sampling_locations,
                      const void* attention_weights, void* output, int B, int K, int H, int D,
                      int L, int Q, int P, int dtype, void* stream) {
    return forward_impl(value, spatial_shapes, level_start_index, sampling_locations,
                        attention_weights, output, kNearest, nullptr, B, K, H, D, L, Q, P, dtype,
                        stream);
}

int msda_sm100_fused_forward(const void* value, const int32_t* spatial_shapes,
                             const int32_t* level_start_index, const void* reference_points,
                             const void* sampling_offsets, const void* attention_logits,
                             void* output, int B, int K, int H, int D, int L, int Q, int P,
                             int dtype, void* stream) {
    return forward_impl(value, spatial_shapes, level_start_index, sampling_offsets,
                        attention_logits, output, kFused, reference_points, B, K, H, D, L, Q, P,
                        dtype, stream);
}

int msda_sm100_fused_backward_ws(const void* value, const int32_t* spatial_shapes,
                                 const int32_t* level_start_index, const void* reference_points,
                                 const void* sampling_offsets, const void* attention_logits,
                                 const void* grad_output, void* grad_value,
                                 float* grad_reference_points, void* grad_sampling_offsets,
                                 void* grad_attention_logits, void* workspace,
                                 size_t workspace_bytes, int B, int K, int H, int D, int L, int Q,
                                 int P, int dtype, void* stream) {
    return backward_impl(value, spatial_shapes, level_start_index, sampling_offsets,
                         attention_logits, grad_output, grad_value, grad_sampling_offsets,
                         grad_attention_logits, workspace, workspace_bytes, true, kFused,
                         reference_points, grad_reference_points, B, K, H, D, L, Q, P, dtype,
                         stream);
}

int gka_sm100_backward_ws(const void* value, const int32_t* spatial_shapes,
                          const int32_t* level_start_index, const void* sampling_locations,
                          const void* attention_weights, const void* grad_output,
                          void* grad_value, void* grad_attn_weight, void* workspace,
                          size_t workspace_bytes, int B, int K, int H, int D, int L, int Q, int P,
                          int dtype, void* stream) {
    return backward_impl(value, spatial_shapes, level_start_index, sampling_locations,
                         attention_weights, grad_output, grad_value, nullptr, grad_attn_weight,
                         workspace, workspace_bytes, true, kNearest, nullptr, nullptr, B, K, H, D,
                         L, Q, P, dtype, stream);
}

int msda_sm100_backward(const void* value, const int32_t* spatial_shapes,
                        const int32_t* level_start_index, const void* sampling_locations,
                        const void* attention_weights, const void* grad_output, void* grad_value,
                        void* grad_sampling_loc, void* grad_attn_weight, int B, int K, int H,
                        int D, int L, int Q, int P, int dtype, void* stream) {
    return backward_impl(value, spatial_shapes, level_start_index, sampling_locations,
                         attention_weights, grad_output, grad_value, grad_sampling_loc,
                         grad_attn_weight, nullptr, 0, false, kBilinear, nullptr, nullptr, B, K, H, D, L,
                         Q, P, dtype, stream);
}

size_t msda_sm100_backward_workspace_bytes(int B, int K, int H, int D, int dtype) {
    if (dtype == MSDA_F32 || B <= 0 || K <= 0 || H <= 0 || D <= 0) return 0;
    return static_cast<size_t>(B) * K * H * D * sizeof(float);
}

int msda_sm100_backward_ws(const void* value, const int32_t* spatial_shapes,
                           const int32_t* level_start_index, const void* sampling_locations,
                           const void* attention_weights, const void* grad_output,
                           void* grad_value, void* grad_sampling_loc, void* grad_attn_weight,
                           void* workspace, size_t workspace_bytes, int B, int K, int H, int D,
                           int L, int Q, int P, int dtype, void* stream) {
    return backward_impl(value, spatial_shapes, level_start_index, sampling_locations,
                         attention_weights, grad_output, grad_value, grad_sampling_loc,
                         grad_attn_weight, workspace, workspace_bytes, true, kBilinear, nullptr, nullptr,
                         B, K, H, D, L, Q, P, dtype, stream);
}

size_t msda_sm100_forward_bytes(int B, int K, int H, int D, int L, int Q, int P, int dtype) {
    const size_t e = elem_size(dtype);
    const size_t v = static_cast<size_t>(B) * K * H * D;
    const size_t s = static_cast<size_t>(B) * Q * H * L * P;
    const size_t o = static_cast<size_t>(B) * Q * H * D;
    return e * (v + 3 * s + o);
}

size_t msda_sm100_backward_bytes(int B, int K, int H, int D, int L, int Q, int P, int dtype) {
    const size_t e = elem_size(dtype);
    const size_t v = static_cast<size_t>(B) * K * H * D;
    const size_t s = static_cast<size_t>(B) * Q * H * L * P;
    const size_t o = static_cast<size_t>(B) * Q * H * D;
    return e * (2 * v + 6 * s + o);
}

int msda_sm100_device_status(int clear) {
    const DeviceInfo* dev = nullptr;
    int rc = device_info(&dev);
    if (rc != MSDA_OK) return rc;
    cudaError_t ce = cudaDeviceSynchronize();
    if (ce != cudaSuccess) return fail_cuda(ce);
    int word = 0;
    ce = cudaMemcpy(&word, dev->status_ptr, sizeof(int), cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) return fail_cuda(ce);
    if (clear) {
        ce = cudaMemset(dev->status_ptr, 0, sizeof(int));
        if (ce != cudaSuccess) return fail_cuda(ce);
    }
    return word;
}

int msda_sm100_tune(int knob, int value) {
    std::atomic<int>* target = nullptr;
    switch (knob) {
        case MSDA_TUNE_STAGE: target = &g_tune_stage; break;
        case MSDA_TUNE_CTAS_PER_SM: target = &g_tune_cps_fwd; break;
        case MSDA_TUNE_CTAS_PER_SM_BWD: target = &g_tune_cps_bwd; break;
        case MSDA_TUNE_INTERLEAVE: target = &g_tune_interleave; break;
        case MSDA_TUNE_SPIN_LIMIT: target = &g_tune_spin; break;
        case MSDA_TUNE_PRECISE_AMP: target = &g_tune_precise_amp; break;
        case MSDA_TUNE_DEBUG_ROW_LIMIT: target = &g_tune_debug_rows; break;
        case MSDA_TUNE_PACK_ROWS: target = &g_tune_pack; break;
        default: return MSDA_ERR_DIMS;
    }
    if (value < 0) return target->load();
    return target->exchange(value);
}

void msda_sm100_profile_events(void* fwd_start, void* fwd_stop, void* bwd_start, void* bwd_stop) {
    t_prof[0] = static_cast<cudaEvent_t>(fwd_start);
    t_prof[1] = static_cast<cudaEvent_t>(fwd_stop);
    t_prof[2] = static_cast<cudaEvent_t>(bwd_start);
    t_prof[3] = static_cast<cudaEvent_t>(bwd_stop);
}

long long msda_sm100_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* msda_sm100_strerror(int status) {
    switch (status) {
        case MSDA_OK: return "ok";
        case MSDA_ERR_NULL: return "a required pointer is NULL";
        case MSDA_ERR_DIMS: return "a dimension or level shape is out of range";
        case MSDA_ERR_LIMIT: return "limit exceeded (D <= 256, L*P <= 64, indices < 2^31)";
        case MSDA_ERR_ALIGN: return "a pointer is misaligned for its element type";
        case MSDA_ERR_DTYPE: return "unknown dtype code";
        case MSDA_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case MSDA_ERR_CUDA: return "a CUDA runtime call failed";
        default: return "unknown status";
    }
}

int msda_sm100_last_cuda_error(void) { return t_last_cuda_error; }

int msda_sm100_abi_version(void) { return kAbiVersion; }

int msda_sm100_debug_bounds(void) {
#ifdef MSDA_DEBUG_BOUNDS
    return 1;
#else
    return 0;
#endif
}

}  // extern "C"

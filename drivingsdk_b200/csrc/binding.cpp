// Torch extension `_C`: the entry points the reference's extension exposes for multi-scale
// deformable attention (and, further down, geometric kernel attention) (mx_driving/csrc/pybind.cpp:110-111, include/csrc/functions.h:58-64)
//     multi_scale_deformable_attn(value, shapes, level_start, loc, attn) -> Tensor
//     multi_scale_deformable_attn_backward(value, shapes, level_start, loc, attn,
//                                          grad_output) -> (Tensor, Tensor, Tensor)
// with the reference binding's checks and messages
// (mx_driving/csrc/MultiScaleDeformableAttn.cpp:28-118). Results are allocated
// here with torch's caching allocator and the work is enqueued on the current
// CUDA stream through the C ABI in include/msda_sm100.h. There is no CPU path:
// non-CUDA tensors are an error.
//
// Differences from the reference binding, all on purpose:
//   * bfloat16 is accepted next to float16/float32;
//   * 16-bit inputs are not upcast to fp32 copies: the kernels read 16-bit
//     operands, do fp32 arithmetic, accumulate grad_value in an fp32 workspace
//     and write 16-bit results (same numerics as the reference's
//     upcast-run-downcast, without the extra passes);
//   * the number of rows of value_spatial_shapes must equal the level dimension
//     of attention_weights (the reference tolerates fewer rows and zero-fills;
//     no test of the reference exercises that).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <atomic>
#include <cstdlib>
#include <tuple>

#include "../../include/conv_ops_sm100.h"
#include "../../include/msda_sm100.h"

namespace {

constexpr int64_t kBatch = 0, kQuery = 1, kHead = 2, kEmbed = 3, kLevel = 3, kPoint = 4;

bool is_float_kind(at::ScalarType t) {
    return t == at::kHalf || t == at::kFloat || t == at::kBFloat16;
}

int dtype_code(at::ScalarType t) {
    if (t == at::kFloat) return MSDA_F32;
    if (t == at::kHalf) return MSDA_F16;
    return MSDA_BF16;
}

struct Dims {
    int B, K, H, D, L, Q, P;
};

Dims check_inputs(const at::Tensor& value, const at::Tensor& shapes, const at::Tensor& starts,
                  const at::Tensor& loc, const at::Tensor& attn) {
    TORCH_CHECK(is_float_kind(value.scalar_type()),
                "value: float16, bfloat16 or float32 tensor expected but got a tensor with dtype: ",
                value.scalar_type());
    TORCH_CHECK(shapes.scalar_type() == at::kInt,
                "value_spatial_shapes: int32 tensor expected but got a tensor with dtype: ",
                shapes.scalar_type());
    TORCH_CHECK(starts.scalar_type() == at::kInt,
                "value_level_start_index: int32 tensor expected but got a tensor with dtype: ",
                starts.scalar_type());
    TORCH_CHECK(is_float_kind(loc.scalar_type()),
                "sampling_locations: float16, bfloat16 or float32 tensor expected but got a tensor "
                "with dtype: ", loc.scalar_type());
    TORCH_CHECK(is_float_kind(attn.scalar_type()),
                "attention_weights: float16, bfloat16 or float32 tensor expected but got a tensor "
                "with dtype: ", attn.scalar_type());
    TORCH_CHECK(value.is_cuda() && loc.is_cuda() && attn.is_cuda(),
                "multi_scale_deformable_attn: value, sampling_locations and attention_weights "
                "must be CUDA tensors (this build has no CPU path)");
    TORCH_CHECK(loc.scalar_type() == value.scalar_type() && attn.scalar_type() == value.scalar_type(),
                "sampling_locations and attention_weights must have value's dtype");
    TORCH_CHECK(value.dim() == 4, "value must be [bs, num_keys, num_heads, embed_dims]");
    TORCH_CHECK(loc.dim() == 6 && loc.size(5) == 2,
                "sampling_locations must be [bs, num_queries, num_heads, num_levels, num_points, 2]");
    TORCH_CHECK(attn.dim() == 5,
                "attention_weights must be [bs, num_queries, num_heads, num_levels, num_points]");
    TORCH_CHECK(value.size(kEmbed) <= 256,
                "The number of embedding dimensions should be less than or equal to 256");
    TORCH_CHECK(loc.size(kLevel) * loc.size(kPoint) <= 64,
                "The product of the number of levels and the number of points should be less than "
                "or equal to 64");
    Dims d;
    d.B = static_cast<int>(value.size(0));
    d.K = static_cast<int>(value.size(1));
    d.H = static_cast<int>(value.size(2));
    d.D = static_cast<int>(value.size(3));
    d.Q = static_cast<int>(loc.size(kQuery));
    d.L = static_cast<int>(loc.size(kLevel));
    d.P = static_cast<int>(loc.size(kPoint));
    TORCH_CHECK(loc.size(kBatch) == d.B && loc.size(kHead) == d.H,
                "sampling_locations batch/head sizes do not match value");
    TORCH_CHECK(attn.size(0) == d.B && attn.size(1) == d.Q && attn.size(2) == d.H &&
                    attn.size(3) == d.L && attn.size(4) == d.P,
                "attention_weights shape does not match sampling_locations");
    TORCH_CHECK(shapes.numel() == 2 * d.L && starts.numel() == d.L,
                "value_spatial_shapes must have one (H, W) row and value_level_start_index one "
                "entry per level of attention_weights");
    TORCH_CHECK(shapes.device() == starts.device(),
                "value_spatial_shapes and value_level_start_index must live on the same device");
    TORCH_CHECK(!shapes.is_cuda() || shapes.device() == value.device(),
                "value_spatial_shapes / value_level_start_index must be CPU tensors or live on "
                "value's device");
    TORCH_CHECK(loc.device() == value.device() && attn.device() == value.device(),
                "sampling_locations and attention_weights must live on value's device");
    return d;
}

// Debugging switch: read the device's sticky status word after every operator call. That
// costs a device synchronisation per call, so it is off unless set_status_checks(true) was
// called or the process started with MSDA_CHECK_STATUS=1.
std::atomic<bool> g_check_status{[] {
    const char* e = std::getenv("MSDA_CHECK_STATUS");
    return e != nullptr && e[0] != '\0' && e[0] != '0';
}()};

void raise_on_error(int rc, const char* what) {
    if (rc == MSDA_OK) {
        if (!g_check_status.load(std::memory_order_relaxed)) return;
        const int status = msda_sm100_device_status(1);
        TORCH_CHECK(status >= 0, what, ": reading the device status failed: ",
                    cudaGetErrorString(static_cast<cudaError_t>(msda_sm100_last_cuda_error())));
        // bit 0 (a staged tile timed out and was fetched with plain loads) leaves the
        // results correct; every other bit means a kernel refused or abandoned work
        TORCH_CHECK((status & ~1) == 0, what, ": device status ", status,
                    " (2: a tensor-core pipeline wait ran out, 4: level table in device memory "
                    "inconsistent with the number of keys, 16: bounds check of the debug build)");
        if (status & 1)
            TORCH_WARN(what, ": a staged tile did not arrive within the poll limit; the kernel "
                             "used plain loads instead");
        return;
    }
    if (rc == MSDA_ERR_CUDA) {
        const auto ce = static_cast<cudaError_t>(msda_sm100_last_cuda_error());
        TORCH_CHECK(false, what, ": CUDA error: ", cudaGetErrorString(ce));
    }
    TORCH_CHECK(false, what, ": ", msda_sm100_strerror(rc));
}

bool set_status_checks(bool on) { return g_check_status.exchange(on); }

}  // namespace

at::Tensor multi_scale_deformable_attn(const at::Tensor& value_in, const at::Tensor& shapes_in,
                                       const at::Tensor& starts_in, const at::Tensor& loc_in,
                                       const at::Tensor& attn_in) {
    const Dims d = check_inputs(value_in, shapes_in, starts_in, loc_in, attn_in);
    const c10::cuda::CUDAGuard guard(value_in.device());
    // the reference op marks its inputs auto-contiguous
    // (kernels/multi_scale_deformable_attn/op_host/multi_scale_deformable_attn.cpp:151-180)
    const at::Tensor value = value_in.contiguous();
    const at::Tensor loc = loc_in.contiguous();
    const at::Tensor attn = attn_in.contiguous();
    const at::Tensor shapes = shapes_in.contiguous();
    const at::Tensor starts = starts_in.contiguous();

    at::Tensor out = at::empty({d.B, d.Q, static_cast<int64_t>(d.H) * d.D}, value.options());
    if (out.numel() == 0) return out;
    const int rc = msda_sm100_forward(
        value.data_ptr(), shapes.data_ptr<int32_t>(), starts.data_ptr<int32_t>(), loc.data_ptr(),
        attn.data_ptr(), out.data_ptr(), d.B, d.K, d.H, d.D, d.L, d.Q, d.P,
        dtype_code(value.scalar_type()), at::cuda::getCurrentCUDAStream().stream());
    raise_on_error(rc, "multi_scale_deformable_attn");
    return out;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> multi_scale_deformable_attn_backward(
    const at::Tensor& value_in, const at::Tensor& shapes_in, const at::Tensor& starts_in,
    const at::Tensor& loc_in, const at::Tensor& attn_in, const at::Tensor& grad_out_in) {
    const Dims d = check_inputs(value_in, shapes_in, starts_in, loc_in, attn_in);
    TORCH_CHECK(is_float_kind(grad_out_in.scalar_type()),
                "grad_output: float16, bfloat16 or float32 tensor expected but got a tensor with "
                "dtype: ", grad_out_in.scalar_type());
    TORCH_CHECK(grad_out_in.is_cuda(), "grad_output must be a CUDA tensor");
    TORCH_CHECK(grad_out_in.numel() == static_cast<int64_t>(d.B) * d.Q * d.H * d.D,
                "grad_output must be [bs, num_queries, num_heads * embed_dims]");
    const c10::cuda::CUDAGuard guard(value_in.device());
    const at::Tensor value = value_in.contiguous();
    const at::Tensor loc = loc_in.contiguous();
    const at::Tensor attn = attn_in.contiguous();
    const at::Tensor shapes = shapes_in.contiguous();
    const at::Tensor starts = starts_in.contiguous();
    const at::Tensor grad_out = grad_out_in.to(value.scalar_type()).contiguous();

    // grad_value is zero-filled by the C-ABI call on the same stream; the other
    // two are fully written by the kernel (the reference allocates them with
    // empty_like too, MultiScaleDeformableAttn.cpp:93-95).
    at::Tensor grad_value = at::empty_like(value);
    at::Tensor grad_loc = at::empty_like(loc);
    at::Tensor grad_attn = at::empty_like(attn);
    if (value.numel() == 0 || loc.numel() == 0) {
        grad_value.zero_();
        return std::make_tuple(grad_value, grad_loc, grad_attn);
    }
    const int dt = dtype_code(value.scalar_type());
    at::Tensor workspace;
    void* ws_ptr = nullptr;
    size_t ws_bytes = msda_sm100_backward_workspace_bytes(d.B, d.K, d.H, d.D, dt);
    if (ws_bytes > 0) {
        workspace = at::empty({static_cast<int64_t>(ws_bytes / sizeof(float))},
                              value.options().dtype(at::kFloat));
        ws_ptr = workspace.data_ptr();
    }
    const int rc = msda_sm100_backward_ws(
        value.data_ptr(), shapes.data_ptr<int32_t>(), starts.data_ptr<int32_t>(), loc.data_ptr(),
        attn.data_ptr(), grad_out.data_ptr(), grad_value.data_ptr(), grad_loc.data_ptr(),
        grad_attn.data_ptr(), ws_ptr, ws_bytes, d.B, d.K, d.H, d.D, d.L, d.Q, d.P, dt,
        at::cuda::getCurrentCUDAStream().stream());
    raise_on_error(rc, "multi_scale_deformable_attn_backward");
    return std::make_tuple(grad_value, grad_loc, grad_attn);
}

// ---------------------------------------------------------------------------
// geometric kernel attention (mx_driving/csrc/GeometricKernelAttentionFunc.cpp:34-118,
// pybind.cpp:131-132): nearest-pixel sampling at integer locations clamped into each level.
// ---------------------------------------------------------------------------
namespace {

Dims check_gka_inputs(const at::Tensor& value, const at::Tensor& shapes, const at::Tensor& starts,
                      const at::Tensor& loc, const at::Tensor& attn) {
    TORCH_CHECK(is_float_kind(value.scalar_type()),
                "value: float16, bfloat16 or float32 tensor expected but got a tensor with dtype: ",
                value.scalar_type());
    TORCH_CHECK(shapes.scalar_type() == at::kInt || shapes.scalar_type() == at::kLong,
                "spatial_spatial_shapes: int32 or int64 tensor expected but got a tensor with "
                "dtype: ", shapes.scalar_type());
    TORCH_CHECK(starts.scalar_type() == at::kInt || starts.scalar_type() == at::kLong,
                "level_start_index: int32 or int64 tensor expected but got a tensor with dtype: ",
                starts.scalar_type());
    TORCH_CHECK(is_float_kind(loc.scalar_type()) || loc.scalar_type() == at::kInt ||
                    loc.scalar_type() == at::kLong,
                "sampling_locations: float16, bfloat16, float32, int32 or int64 tensor expected "
                "but got a tensor with dtype: ", loc.scalar_type());
    TORCH_CHECK(is_float_kind(attn.scalar_type()),
                "attention_weights: float16, bfloat16 or float32 tensor expected but got a tensor "
                "with dtype: ", attn.scalar_type());
    TORCH_CHECK(value.is_cuda() && loc.is_cuda() && attn.is_cuda(),
                "geometric_kernel_attention: value, sampling_locations and attention_weights "
                "must be CUDA tensors (this build has no CPU path)");
    TORCH_CHECK(value.dim() == 4 && loc.dim() == 6 && loc.size(5) == 2 && attn.dim() == 5,
                "geometric_kernel_attention: value [bs, keys, heads, dims], sampling_locations "
                "[bs, queries, heads, levels, points, 2], attention_weights [bs, queries, heads, "
                "levels, points] expected");
    TORCH_CHECK(value.size(kEmbed) <= 256,
                "The number of embedding dimensions should be less than or equal to 256");
    TORCH_CHECK(loc.size(kLevel) * loc.size(kPoint) <= 64,
                "The product of the number of levels and the number of points should be less than "
                "or equal to 64");
    Dims d;
    d.B = static_cast<int>(value.size(0));
    d.K = static_cast<int>(value.size(1));
    d.H = static_cast<int>(value.size(2));
    d.D = static_cast<int>(value.size(3));
    d.Q = static_cast<int>(attn.size(1));
    d.L = static_cast<int>(attn.size(3));
    d.P = static_cast<int>(attn.size(4));
    TORCH_CHECK(attn.size(0) == d.B && attn.size(2) == d.H && loc.size(0) == d.B &&
                    loc.size(1) == d.Q && loc.size(2) == d.H && loc.size(3) == d.L &&
                    loc.size(4) == d.P,
                "sampling_locations / attention_weights shapes do not match value");
    TORCH_CHECK(shapes.numel() == 2 * d.L && starts.numel() == d.L,
                "spatial_shapes must have one (H, W) row and level_start_index one entry per level");
    return d;
}

}  // namespace

void geometric_kernel_attention_forward(const at::Tensor& value_in, const at::Tensor& shapes_in,
                                        const at::Tensor& starts_in, const at::Tensor& loc_in,
                                        const at::Tensor& attn_in, at::Tensor& output) {
    const Dims d = check_gka_inputs(value_in, shapes_in, starts_in, loc_in, attn_in);
    TORCH_CHECK(output.is_cuda() && output.is_contiguous() &&
                    output.scalar_type() == value_in.scalar_type() &&
                    output.numel() == static_cast<int64_t>(d.B) * d.Q * d.H * d.D,
                "output must be a contiguous CUDA tensor [bs, num_queries, num_heads * dims] of "
                "value's dtype");
    const c10::cuda::CUDAGuard guard(value_in.device());
    const at::Tensor value = value_in.contiguous();
    // integer pixel coordinates travel in value's dtype (exact up to 2048 in float16)
    const at::Tensor loc = loc_in.to(value.scalar_type()).contiguous();
    const at::Tensor attn = attn_in.to(value.scalar_type()).contiguous();
    const at::Tensor shapes = shapes_in.to(at::kInt).contiguous();
    const at::Tensor starts = starts_in.to(at::kInt).contiguous();
    if (output.numel() == 0) return;
    const int rc = gka_sm100_forward(
        value.data_ptr(), shapes.data_ptr<int32_t>(), starts.data_ptr<int32_t>(), loc.data_ptr(),
        attn.data_ptr(), output.data_ptr(), d.B, d.K, d.H, d.D, d.L, d.Q, d.P,
        dtype_code(value.scalar_type()), at::cuda::getCurrentCUDAStream().stream());
    raise_on_error(rc, "geometric_kernel_attention_forward");
}

std::tuple<at::Tensor, at::Tensor> geometric_kernel_attention_backward(
    const at::Tensor& value_in, const at::Tensor& shapes_in, const at::Tensor& starts_in,
    const at::Tensor& loc_in, const at::Tensor& attn_in, const at::Tensor& grad_out_in) {
    const Dims d = check_gka_inputs(value_in, shapes_in, starts_in, loc_in, attn_in);
    TORCH_CHECK(is_float_kind(grad_out_in.scalar_type()) && grad_out_in.is_cuda(),
                "grad_output: float16, bfloat16 or float32 CUDA tensor expected");
    TORCH_CHECK(d.D % 8 == 0, "embed_dims must be a multiple of 8, but embed_dims is ", d.D, ".");
    TORCH_CHECK(grad_out_in.numel() == static_cast<int64_t>(d.B) * d.Q * d.H * d.D,
                "grad_output must be [bs, num_queries, num_heads * dims]");
    const c10::cuda::CUDAGuard guard(value_in.device());
    const at::Tensor value = value_in.contiguous();
    const at::Tensor loc = loc_in.to(value.scalar_type()).contiguous();
    const at::Tensor attn = attn_in.to(value.scalar_type()).contiguous();
    const at::Tensor shapes = shapes_in.to(at::kInt).contiguous();
    const at::Tensor starts = starts_in.to(at::kInt).contiguous();
    const at::Tensor grad_out = grad_out_in.to(value.scalar_type()).contiguous();
    at::Tensor grad_value = at::empty_like(value);
    at::Tensor grad_attn = at::empty_like(attn);
    if (value.numel() == 0 || attn.numel() == 0) {
        grad_value.zero_();
        return std::make_tuple(grad_value, grad_attn);
    }
    const int dt = dtype_code(value.scalar_type());
    at::Tensor workspace;
    void* ws_ptr = nullptr;
    const size_t ws_bytes = msda_sm100_backward_workspace_bytes(d.B, d.K, d.H, d.D, dt);
    if (ws_bytes > 0) {
        workspace = at::empty({static_cast<int64_t>(ws_bytes / sizeof(float))},
                              value.options().dtype(at::kFloat));
        ws_ptr = workspace.data_ptr();
    }
    const int rc = gka_sm100_backward_ws(
        value.data_ptr(), shapes.data_ptr<int32_t>(), starts.data_ptr<int32_t>(), loc.data_ptr(),
        attn.data_ptr(), grad_out.data_ptr(), grad_value.data_ptr(), grad_attn.data_ptr(), ws_ptr,
        ws_bytes, d.B, d.K, d.H, d.D, d.L, d.Q, d.P, dt,
        at::cuda::getCurrentCUDAStream().stream());
    raise_on_error(rc, "geometric_kernel_attention_backward");
    return std::make_tuple(grad_value, grad_attn);
}

// ---------------------------------------------------------------------------
// deformable aggregation (mx_driving/csrc/DeformableAggregation.cpp:20-76,
// pybind.cpp:121-122). The kernels are fp32; 16-bit tensors are converted on the way in
// and out, as the reference binding does for its other 16-bit paths.
// ---------------------------------------------------------------------------
namespace {

struct DaDims {
    int B, F, C, A, Pts, cams, scales, G;
};

DaDims check_da_inputs(const at::Tensor& feat, const at::Tensor& shape, const at::Tensor& start,
                       const at::Tensor& loc, const at::Tensor& wts) {
    TORCH_CHECK(feat.is_cuda() && loc.is_cuda() && wts.is_cuda(),
                "deformable_aggregation: mc_ms_feat, sampling_location and weights must be CUDA "
                "tensors (this build has no CPU path)");
    TORCH_CHECK(feat.dim() == 3, "mc_ms_feat.dim() must be 3, but got: ", feat.dim());
    TORCH_CHECK(shape.dim() == 3, "spatial_shape.dim() must be 3, but got: ", shape.dim());
    TORCH_CHECK(start.dim() == 2, "scale_start_index.dim() must be 2, but got: ", start.dim());
    TORCH_CHECK(loc.dim() == 5, "sampling_location.dim() must be 5, but got: ", loc.dim());
    TORCH_CHECK(wts.dim() == 6, "weights.dim() must be 6, but got: ", wts.dim());
    TORCH_CHECK(wts.size(5) % 8 == 0, "weights.sizes()[5] must be multiple of 8, but got: ",
                wts.size(5));
    TORCH_CHECK(is_float_kind(feat.scalar_type()) && is_float_kind(loc.scalar_type()) &&
                    is_float_kind(wts.scalar_type()),
                "deformable_aggregation: float16, bfloat16 or float32 tensors expected");
    TORCH_CHECK(shape.scalar_type() == at::kInt && start.scalar_type() == at::kInt,
                "spatial_shape and scale_start_index must be int32 tensors");
    DaDims d;
    d.B = static_cast<int>(feat.size(0));
    d.F = static_cast<int>(feat.size(1));
    d.C = static_cast<int>(feat.size(2));
    d.A = static_cast<int>(wts.size(1));
    d.Pts = static_cast<int>(wts.size(2));
    d.cams = static_cast<int>(wts.size(3));
    d.scales = static_cast<int>(wts.size(4));
    d.G = static_cast<int>(wts.size(5));
    TORCH_CHECK(wts.size(0) == d.B && loc.size(0) == d.B && loc.size(1) == d.A &&
                    loc.size(2) == d.Pts && loc.size(3) == d.cams && loc.size(4) == 2,
                "sampling_location / weights shapes do not match");
    TORCH_CHECK(shape.size(0) == d.cams && shape.size(1) == d.scales && shape.size(2) == 2 &&
                    start.size(0) == d.cams && start.size(1) == d.scales,
                "spatial_shape must be [cams, scales, 2] and scale_start_index [cams, scales]");
    TORCH_CHECK(d.C % d.G == 0, "the number of channels must be a multiple of the groups");
    return d;
}

void raise_on_da_error(int rc, const char* what) {
    if (rc == MSDA_OK) return;
    if (rc == MSDA_ERR_CUDA) {
        const auto ce = static_cast<cudaError_t>(da_sm100_last_cuda_error());
        TORCH_CHECK(false, what, ": CUDA error: ", cudaGetErrorString(ce));
    }
    TORCH_CHECK(false, what, ": ", msda_sm100_strerror(rc));
}

}  // namespace

at::Tensor deformable_aggregation(const at::Tensor& feat_in, const at::Tensor& shape_in,
                                  const at::Tensor& start_in, const at::Tensor& loc_in,
                                  const at::Tensor& wts_in) {
    const DaDims d = check_da_inputs(feat_in, shape_in, start_in, loc_in, wts_in);
    const c10::cuda::CUDAGuard guard(feat_in.device());
    const at::Tensor feat = feat_in.to(at::kFloat).contiguous();
    const at::Tensor loc = loc_in.to(at::kFloat).contiguous();
    const at::Tensor wts = wts_in.to(at::kFloat).contiguous();
    const at::Tensor shape = shape_in.contiguous();
    const at::Tensor start = start_in.contiguous();
    at::Tensor out = at::empty({d.B, d.A, d.C}, feat.options());
    if (out.numel() == 0) return out.to(feat_in.scalar_type());
    const int rc = da_sm100_forward(feat.data_ptr(), shape.data_ptr<int32_t>(),
                                    start.data_ptr<int32_t>(), loc.data_ptr(), wts.data_ptr(),
                                    out.data_ptr(), d.B, d.F, d.C, d.A, d.Pts, d.cams, d.scales,
                                    d.G, at::cuda::getCurrentCUDAStream().stream());
    raise_on_da_error(rc, "npu_deformable_aggregation");
    return out.to(feat_in.scalar_type());
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> deformable_aggregation_backward(
    const at::Tensor& feat_in, const at::Tensor& shape_in, const at::Tensor& start_in,
    const at::Tensor& loc_in, const at::Tensor& wts_in, const at::Tensor& grad_out_in,
    const at::Tensor& grad_feat_in, const at::Tensor& grad_loc_in, const at::Tensor& grad_wts_in) {
    // the three gradient tensors are accepted for call compatibility with the reference
    // (it fills tensors the caller zeroed); results are returned as new tensors
    (void)grad_feat_in; (void)grad_loc_in; (void)grad_wts_in;
    const DaDims d = check_da_inputs(feat_in, shape_in, start_in, loc_in, wts_in);
    TORCH_CHECK(grad_out_in.is_cuda() && is_float_kind(grad_out_in.scalar_type()) &&
                    grad_out_in.numel() == static_cast<int64_t>(d.B) * d.A * d.C,
                "grad_output must be a CUDA tensor [bs, anchors, channels]");
    const c10::cuda::CUDAGuard guard(feat_in.device());
    const at::Tensor feat = feat_in.to(at::kFloat).contiguous();
    const at::Tensor loc = loc_in.to(at::kFloat).contiguous();
    const at::Tensor wts = wts_in.to(at::kFloat).contiguous();
    const at::Tensor shape = shape_in.contiguous();
    const at::Tensor start = start_in.contiguous();
    const at::Tensor grad_out = grad_out_in.to(at::kFloat).contiguous();
    at::Tensor grad_feat = at::empty_like(feat);
    at::Tensor grad_loc = at::empty_like(loc);
    at::Tensor grad_wts = at::empty_like(wts);
    const int rc = da_sm100_backward(
        feat.data_ptr(), shape.data_ptr<int32_t>(), start.data_ptr<int32_t>(), loc.data_ptr(),
        wts.data_ptr(), grad_out.data_ptr(), grad_feat.data_ptr(), grad_loc.data_ptr(),
        grad_wts.data_ptr(), d.B, d.F, d.C, d.A, d.Pts, d.cams, d.scales, d.G,
        at::cuda::getCurrentCUDAStream().stream());
    raise_on_da_error(rc, "npu_deformable_aggregation_backward");
    return std::make_tuple(grad_feat.to(feat_in.scalar_type()), grad_loc.to(loc_in.scalar_type()),
                           grad_wts.to(wts_in.scalar_type()));
}

// ---------------------------------------------------------------------------
// fused MSDA: reference points + sampling offsets + attention logits in, output out; the
// location arithmetic and the softmax of mmcv's MultiScaleDeformableAttention.forward happen
// inside the kernels. No counterpart in the reference's extension.
// ---------------------------------------------------------------------------
namespace {

Dims check_fused_inputs(const at::Tensor& value, const at::Tensor& shapes,
                        const at::Tensor& starts, const at::Tensor& ref, const at::Tensor& off,
                        const at::Tensor& logits) {
    const Dims d = check_inputs(value, shapes, starts, off, logits);
    TORCH_CHECK(ref.is_cuda() && ref.scalar_type() == value.scalar_type(),
                "reference_points must be a CUDA tensor of value's dtype");
    TORCH_CHECK(ref.dim() == 4 && ref.size(0) == d.B && ref.size(1) == d.Q && ref.size(2) == d.L &&
                    ref.size(3) == 2,
                "reference_points must be [bs, num_queries, num_levels, 2]");
    TORCH_CHECK(static_cast<int64_t>(d.L) * d.P <= 32,
                "the fused operator needs num_levels * num_points <= 32");
    return d;
}

}  // namespace

at::Tensor msda_fused_forward(const at::Tensor& value_in, const at::Tensor& shapes_in,
                              const at::Tensor& starts_in, const at::Tensor& ref_in,
                              const at::Tensor& off_in, const at::Tensor& logits_in) {
    const Dims d = check_fused_inputs(value_in, shapes_in, starts_in, ref_in, off_in, logits_in);
    const c10::cuda::CUDAGuard guard(value_in.device());
    const at::Tensor value = value_in.contiguous();
    const at::Tensor ref = ref_in.contiguous();
    const at::Tensor off = off_in.contiguous();
    const at::Tensor logits = logits_in.contiguous();
    const at::Tensor shapes = shapes_in.contiguous();
    const at::Tensor starts = starts_in.contiguous();
    at::Tensor out = at::empty({d.B, d.Q, static_cast<int64_t>(d.H) * d.D}, value.options());
    if (out.numel() == 0) return out;
    const int rc = msda_sm100_fused_forward(
        value.data_ptr(), shapes.data_ptr<int32_t>(), starts.data_ptr<int32_t>(), ref.data_ptr(),
        off.data_ptr(), logits.data_ptr(), out.data_ptr(), d.B, d.K, d.H, d.D, d.L, d.Q, d.P,
        dtype_code(value.scalar_type()), at::cuda::getCurrentCUDAStream().stream());
    raise_on_error(rc, "msda_fused_forward");
    return out;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> msda_fused_backward(
    const at::Tensor& value_in, const at::Tensor& shapes_in, const at::Tensor& starts_in,
    const at::Tensor& ref_in, const at::Tensor& off_in, const at::Tensor& logits_in,
    const at::Tensor& grad_out_in) {
    const Dims d = check_fused_inputs(value_in, shapes_in, starts_in, ref_in, off_in, logits_in);
    TORCH_CHECK(grad_out_in.is_cuda() && is_float_kind(grad_out_in.scalar_type()) &&
                    grad_out_in.numel() == static_cast<int64_t>(d.B) * d.Q * d.H * d.D,
                "grad_output must be a CUDA tensor [bs, num_queries, num_heads * embed_dims]");
    const c10::cuda::CUDAGuard guard(value_in.device());
    const at::Tensor value = value_in.contiguous();
    const at::Tensor ref = ref_in.contiguous();
    const at::Tensor off = off_in.contiguous();
    const at::Tensor logits = logits_in.contiguous();
    const at::Tensor shapes = shapes_in.contiguous();
    const at::Tensor starts = starts_in.contiguous();
    const at::Tensor grad_out = grad_out_in.to(value.scalar_type()).contiguous();
    at::Tensor grad_value = at::empty_like(value);
    at::Tensor grad_off = at::empty_like(off);
    at::Tensor grad_logits = at::empty_like(logits);
    at::Tensor grad_ref = at::empty(ref.sizes(), ref.options().dtype(at::kFloat));
    const int dt = dtype_code(value.scalar_type());
    at::Tensor workspace;
    void* ws_ptr = nullptr;
    const size_t ws_bytes = msda_sm100_backward_workspace_bytes(d.B, d.K, d.H, d.D, dt);
    if (ws_bytes > 0) {
        workspace = at::empty({static_cast<int64_t>(ws_bytes / sizeof(float))},
                              value.options().dtype(at::kFloat));
        ws_ptr = workspace.data_ptr();
    }
    const int rc = msda_sm100_fused_backward_ws(
        value.data_ptr(), shapes.data_ptr<int32_t>(), starts.data_ptr<int32_t>(), ref.data_ptr(),
        off.data_ptr(), logits.data_ptr(), grad_out.data_ptr(), grad_value.data_ptr(),
        grad_ref.data_ptr<float>(), grad_off.data_ptr(), grad_logits.data_ptr(), ws_ptr, ws_bytes,
        d.B, d.K, d.H, d.D, d.L, d.Q, d.P, dt, at::cuda::getCurrentCUDAStream().stream());
    raise_on_error(rc, "msda_fused_backward");
    return std::make_tuple(grad_value, grad_ref.to(ref.scalar_type()), grad_off, grad_logits);
}

// ---------------------------------------------------------------------------
// add + ReLU and ResNet-stem max pooling (mx_driving/csrc/pybind.cpp: npu_add_relu,
// npu_add_relu_grad, npu_max_pool2d; bindings mx_driving/csrc/AddRelu.cpp:20-32,
// mx_driving/csrc/MaxPool2d.cpp:25-100)
// ---------------------------------------------------------------------------
at::Tensor npu_add_relu(at::Tensor& x, const at::Tensor& y_in) {
    TORCH_CHECK(x.is_cuda() && y_in.is_cuda(),
                "npu_add_relu: x and y must be CUDA tensors (this build has no CPU path)");
    TORCH_CHECK(is_float_kind(x.scalar_type()) && x.scalar_type() == y_in.scalar_type(),
                "npu_add_relu: x and y must share a dtype of float16, bfloat16 or float32");
    TORCH_CHECK(x.sizes() == y_in.sizes(), "npu_add_relu: x and y must have the same shape");
    TORCH_CHECK(x.is_contiguous(), "npu_add_relu: x is updated in place and must be contiguous");
    const c10::cuda::CUDAGuard guard(x.device());
    const at::Tensor y = y_in.contiguous();
    const int rc = addrelu_sm100_forward(x.data_ptr(), y.data_ptr(),
                                         static_cast<size_t>(x.numel()),
                                         dtype_code(x.scalar_type()),
                                         at::cuda::getCurrentCUDAStream().stream());
    raise_on_error(rc, "npu_add_relu");
    return x;
}

at::Tensor npu_add_relu_grad(const at::Tensor& self_in, const at::Tensor& grad_output_in) {
    TORCH_CHECK(self_in.is_cuda() && grad_output_in.is_cuda(),
                "npu_add_relu_grad: CUDA tensors expected (this build has no CPU path)");
    TORCH_CHECK(is_float_kind(self_in.scalar_type()), "npu_add_relu_grad: floating tensors expected");
    TORCH_CHECK(self_in.numel() == grad_output_in.numel(),
                "npu_add_relu_grad: self and grad_output must have the same number of elements");
    const c10::cuda::CUDAGuard guard(self_in.device());
    const at::Tensor self = self_in.contiguous();
    const at::Tensor grad_output = grad_output_in.to(self.scalar_type()).contiguous();
    at::Tensor result = at::empty_like(self);
    const int rc = addrelu_sm100_backward(self.data_ptr(), grad_output.data_ptr(), result.data_ptr(),
                                          static_cast<size_t>(self.numel()),
                                          dtype_code(self.scalar_type()),
                                          at::cuda::getCurrentCUDAStream().stream());
    raise_on_error(rc, "npu_add_relu_grad");
    return result;
}

at::Tensor npu_max_pool2d(const at::Tensor& x_in, int kernel_size, int stride, int padding) {
    TORCH_CHECK(x_in.is_cuda(), "npu_max_pool2d: x must be a CUDA tensor (this build has no CPU path)");
    TORCH_CHECK(is_float_kind(x_in.scalar_type()),
                "x: float32 or float16 tensor expected but got a tensor with dtype: ",
                x_in.scalar_type());
    TORCH_CHECK(kernel_size == 3, "kernel_size: expected 3 but got: ", kernel_size);
    TORCH_CHECK(stride == 2, "stride: expected 2 but got: ", stride);
    TORCH_CHECK(padding == 1, "padding: expected 1 but got: ", padding);
    TORCH_CHECK(x_in.dim() == 4, "x_trans.dim() must be 4, but got: ", x_in.dim());
    const c10::cuda::CUDAGuard guard(x_in.device());
    const at::Tensor x = x_in.contiguous();
    const int64_t N = x.size(0), C = x.size(1), H = x.size(2), W = x.size(3);
    at::Tensor y = at::empty({N, C, (H + 1) / 2, (W + 1) / 2}, x.options());
    if (y.numel() == 0) return y;
    const int rc = maxpool_sm100_forward(x.data_ptr(), y.data_ptr(), static_cast<int>(N),
                                         static_cast<int>(C), static_cast<int>(H),
                                         static_cast<int>(W), dtype_code(x.scalar_type()),
                                         at::cuda::getCurrentCUDAStream().stream());
    raise_on_error(rc, "npu_max_pool2d");
    return y;
}

// ---------------------------------------------------------------------------
// deformable / modulated deformable convolution (mx_driving/csrc/pybind.cpp: deformable_conv2d,
// deformable_conv2d_backward, modulated_deformable_conv2d, modulated_deformable_conv2d_backward;
// bindings mx_driving/csrc/DeformableConv2d.cpp:21-101, ModulatedDeformableConv2d.cpp:26-140).
// Tensors are channels-last as in the reference: x [n, h, w, c], offset [n, ho, wo, dg*2*kh*kw],
// mask [n, ho, wo, dg*kh*kw], weight [co, kh, kw, c/groups]; grad_out is taken as
// [n, ho, wo, co] by both backward functions. Arithmetic is fp32; 16-bit inputs are converted.
// ---------------------------------------------------------------------------
namespace {

struct DcnCall {
    dcn_shape s;
    at::Tensor x, offset, mask, weight;
};

DcnCall check_dcn(const at::Tensor& input, const at::Tensor& offset, const at::Tensor& mask,
                  const at::Tensor& weight, at::IntArrayRef kernel_size, at::IntArrayRef stride,
                  at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups,
                  int64_t deformable_groups) {
    TORCH_CHECK(input.is_cuda() && offset.is_cuda() && weight.is_cuda(),
                "deformable_conv2d: CUDA tensors expected (this build has no CPU path)");
    TORCH_CHECK(input.dim() == 4, "input must to be a 4D Tensor, but got: ", input.dim());
    TORCH_CHECK(offset.dim() == 4, "offset has to be a 4D Tensor, but got: ", offset.dim());
    TORCH_CHECK(weight.dim() == 4, "weight has to be a 4D Tensor, but got: ", weight.dim());
    TORCH_CHECK(kernel_size.size() == 2 && stride.size() == 2 && padding.size() == 2 &&
                    dilation.size() == 2,
                "kernel_size, stride, padding and dilation must have two entries");
    TORCH_CHECK(stride[0] > 0 && stride[1] > 0, "stride must be greater than 0");
    TORCH_CHECK(kernel_size[0] > 0 && kernel_size[1] > 0, "kernel_size must be greater than 0");
    TORCH_CHECK(dilation[0] > 0 && dilation[1] > 0, "dilation must be greater than 0");
    TORCH_CHECK(weight.size(1) == kernel_size[0] && weight.size(2) == kernel_size[1],
                "kernel size mismatch");
    TORCH_CHECK(groups > 0, "groups must be greater than 0");
    TORCH_CHECK(deformable_groups > 0, "deformable_groups must be greater than 0");
    TORCH_CHECK(weight.size(0) % groups == 0, "weight's out channel should be divided by groups");
    TORCH_CHECK(input.size(3) % groups == 0, "input's channel should be divided by groups");
    TORCH_CHECK(weight.size(3) == input.size(3) / groups,
                "weight must be [c_out, kh, kw, c_in / groups]");
    const int64_t taps = kernel_size[0] * kernel_size[1];
    TORCH_CHECK(offset.size(0) == input.size(0) && offset.size(3) == deformable_groups * 2 * taps,
                "offset must be [n, h_out, w_out, deformable_groups * 2 * kh * kw]");
    if (mask.defined()) {
        TORCH_CHECK(mask.is_cuda() && mask.dim() == 4, "mask has to be a 4D Tensor, but got: ", mask.dim());
        TORCH_CHECK(mask.size(0) == offset.size(0) && mask.size(1) == offset.size(1) &&
                        mask.size(2) == offset.size(2) && mask.size(3) == deformable_groups * taps,
                    "The shape of the mask is invalid");
    }
    DcnCall c;
    c.s.N = static_cast<int>(input.size(0));
    c.s.H = static_cast<int>(input.size(1));
    c.s.W = static_cast<int>(input.size(2));
    c.s.C = static_cast<int>(input.size(3));
    c.s.Ho = static_cast<int>(offset.size(1));
    c.s.Wo = static_cast<int>(offset.size(2));
    c.s.Co = static_cast<int>(weight.size(0));
    c.s.kh = static_cast<int>(kernel_size[0]);
    c.s.kw = static_cast<int>(kernel_size[1]);
    c.s.stride_h = static_cast<int>(stride[0]);
    c.s.stride_w = static_cast<int>(stride[1]);
    c.s.pad_h = static_cast<int>(padding[0]);
    c.s.pad_w = static_cast<int>(padding[1]);
    c.s.dil_h = static_cast<int>(dilation[0]);
    c.s.dil_w = static_cast<int>(dilation[1]);
    c.s.groups = static_cast<int>(groups);
    c.s.deform_groups = static_cast<int>(deformable_groups);
    c.x = input.to(at::kFloat).contiguous();
    c.offset = offset.to(at::kFloat).contiguous();
    c.weight = weight.to(at::kFloat).contiguous();
    if (mask.defined()) c.mask = mask.to(at::kFloat).contiguous();
    return c;
}

std::tuple<at::Tensor, at::Tensor> dcn_forward(const char* what, const at::Tensor& input,
                                               const at::Tensor& offset, const at::Tensor& mask,
                                               const at::Tensor& weight, const at::Tensor& bias,
                                               at::IntArrayRef kernel_size, at::IntArrayRef stride,
                                               at::IntArrayRef padding, at::IntArrayRef dilation,
                                               int64_t groups, int64_t deformable_groups) {
    DcnCall c = check_dcn(input, offset, mask, weight, kernel_size, stride, padding, dilation,
                          groups, deformable_groups);
    const c10::cuda::CUDAGuard guard(input.device());
    const dcn_shape& s = c.s;
    at::Tensor out = at::empty({s.N, s.Ho, s.Wo, s.Co}, c.x.options());
    at::Tensor columns = at::empty({s.N, static_cast<int64_t>(s.Ho) * s.Wo, s.groups,
                                    static_cast<int64_t>(s.kh) * s.kw, s.C / s.groups}, c.x.options());
    at::Tensor bias_f;
    if (bias.defined()) {
        TORCH_CHECK(bias.is_cuda() && bias.numel() == s.Co, "bias must be a CUDA tensor [c_out]");
        bias_f = bias.to(at::kFloat).contiguous();
    }
    if (out.numel() > 0) {
        const int rc = dcn_sm100_forward(
            c.x.data_ptr<float>(), c.offset.data_ptr<float>(),
            c.mask.defined() ? c.mask.data_ptr<float>() : nullptr, c.weight.data_ptr<float>(),
            bias_f.defined() ? bias_f.data_ptr<float>() : nullptr, out.data_ptr<float>(),
            columns.data_ptr<float>(), &s, at::cuda::getCurrentCUDAStream().stream());
        raise_on_error(rc, what);
    }
    return std::make_tuple(out.permute({0, 3, 1, 2}).to(input.scalar_type()), columns);
}

struct DcnGrads {
    at::Tensor x, offset, mask, weight, bias;
};

DcnGrads dcn_backward(const char* what, const at::Tensor& input, const at::Tensor& offset,
                      const at::Tensor& mask, const at::Tensor& weight, bool want_bias,
                      const at::Tensor& columns, const at::Tensor& grad_y,
                      at::IntArrayRef kernel_size, at::IntArrayRef stride, at::IntArrayRef padding,
                      at::IntArrayRef dilation, int64_t groups, int64_t deformable_groups) {
    DcnCall c = check_dcn(input, offset, mask, weight, kernel_size, stride, padding, dilation,
                          groups, deformable_groups);
    const dcn_shape& s = c.s;
    TORCH_CHECK(grad_y.is_cuda() && grad_y.dim() == 4 && grad_y.size(0) == s.N && grad_y.size(1) == s.Ho &&
                    grad_y.size(2) == s.Wo && grad_y.size(3) == s.Co,
                "grad_y must be a CUDA tensor [n, h_out, w_out, c_out]");
    const c10::cuda::CUDAGuard guard(input.device());
    const at::Tensor go = grad_y.to(at::kFloat).contiguous();
    const size_t col_bytes = dcn_sm100_columns_bytes(&s);
    at::Tensor cols = columns;
    if (!cols.defined() || static_cast<size_t>(cols.numel()) * 4 != col_bytes || !cols.is_cuda()) {
        // the caller did not keep the forward's columns: compute them again
        at::Tensor out;
        std::tie(out, cols) = dcn_forward(what, input, offset, mask, weight, at::Tensor(),
                                          kernel_size, stride, padding, dilation, groups,
                                          deformable_groups);
    }
    cols = cols.to(at::kFloat).contiguous();
    DcnGrads g;
    g.x = at::empty_like(c.x);
    g.offset = at::empty_like(c.offset);
    g.weight = at::empty_like(c.weight);
    if (c.mask.defined()) g.mask = at::empty_like(c.mask);
    if (want_bias) g.bias = at::empty({s.Co}, c.x.options());
    const size_t ws_bytes = dcn_sm100_backward_workspace_bytes(&s);
    at::Tensor ws = at::empty({static_cast<int64_t>(ws_bytes / 4) + 4}, c.x.options());
    if (g.x.numel() > 0 && go.numel() > 0) {
        const int rc = dcn_sm100_backward(
            c.x.data_ptr<float>(), c.offset.data_ptr<float>(),
            c.mask.defined() ? c.mask.data_ptr<float>() : nullptr, c.weight.data_ptr<float>(),
            cols.data_ptr<float>(), go.data_ptr<float>(), g.x.data_ptr<float>(),
            g.offset.data_ptr<float>(), g.mask.defined() ? g.mask.data_ptr<float>() : nullptr,
            g.weight.data_ptr<float>(), g.bias.defined() ? g.bias.data_ptr<float>() : nullptr,
            ws.data_ptr(), ws_bytes, &s, at::cuda::getCurrentCUDAStream().stream());
        raise_on_error(rc, what);
    }
    return g;
}

}  // namespace

std::tuple<at::Tensor, at::Tensor> deformable_conv2d(
    const at::Tensor& input, const at::Tensor& offset, const at::Tensor& weight,
    at::IntArrayRef kernel_size, at::IntArrayRef stride, at::IntArrayRef padding,
    at::IntArrayRef dilation, int64_t groups, int64_t deformable_groups) {
    return dcn_forward("deformable_conv2d", input, offset, at::Tensor(), weight, at::Tensor(),
                       kernel_size, stride, padding, dilation, groups, deformable_groups);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> deformable_conv2d_backward(
    const at::Tensor& input, const at::Tensor& weight, const at::Tensor& offset,
    const at::Tensor& offset_output, const at::Tensor& grad_y, at::IntArrayRef kernel_size,
    at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups,
    int64_t deformable_groups) {
    DcnGrads g = dcn_backward("deformable_conv2d_backward", input, offset, at::Tensor(), weight,
                              false, offset_output, grad_y, kernel_size, stride, padding,
                              dilation, groups, deformable_groups);
    return std::make_tuple(g.x.permute({0, 3, 1, 2}).to(input.scalar_type()),
                           g.weight.permute({0, 3, 1, 2}).to(weight.scalar_type()),
                           g.offset.permute({0, 3, 1, 2}).to(offset.scalar_type()));
}

std::tuple<at::Tensor, at::Tensor> modulated_deformable_conv2d(
    const at::Tensor& input, const at::Tensor& offset, const at::Tensor& mask,
    const at::Tensor& weight, const c10::optional<at::Tensor>& bias_opt,
    at::IntArrayRef kernel_size, at::IntArrayRef stride, at::IntArrayRef padding,
    at::IntArrayRef dilation, int64_t groups, int64_t deformable_groups, int64_t with_bias) {
    TORCH_CHECK(mask.defined(), "mask has to be a 4D Tensor");
    const at::Tensor bias = (with_bias != 0 && bias_opt.has_value()) ? *bias_opt : at::Tensor();
    return dcn_forward("modulated_deformable_conv2d", input, offset, mask, weight, bias,
                       kernel_size, stride, padding, dilation, groups, deformable_groups);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor>
modulated_deformable_conv2d_backward(
    const at::Tensor& input, const at::Tensor& offset, const at::Tensor& mask,
    const at::Tensor& weight, const c10::optional<at::Tensor>& bias_opt,
    const at::Tensor& offset_output, const at::Tensor& grad_y, at::IntArrayRef kernel_size,
    at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups,
    int64_t deformable_groups, int64_t with_bias) {
    TORCH_CHECK(mask.defined(), "mask has to be a 4D Tensor");
    const bool want_bias = with_bias != 0 && bias_opt.has_value();
    DcnGrads g = dcn_backward("modulated_deformable_conv2d_backward", input, offset, mask, weight,
                              want_bias, offset_output, grad_y, kernel_size, stride, padding,
                              dilation, groups, deformable_groups);
    return std::make_tuple(g.x.permute({0, 3, 1, 2}).to(input.scalar_type()),
                           g.weight.permute({0, 3, 1, 2}).to(weight.scalar_type()),
                           want_bias ? g.bias.to(bias_opt->scalar_type()) : at::Tensor(),
                           g.offset.permute({0, 3, 1, 2}).to(offset.scalar_type()),
                           g.mask.permute({0, 3, 1, 2}).to(mask.scalar_type()));
}

int64_t dcn_use_tensor_cores(int64_t on) { return dcn_sm100_use_tensor_cores(static_cast<int>(on)); }

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "sm_100a multi-scale deformable attention (drop-in for mx_driving._C on this path)";
    m.def("multi_scale_deformable_attn", &multi_scale_deformable_attn,
          "MSDA forward: (value, value_spatial_shapes, value_level_start_index, "
          "sampling_locations, attention_weights) -> output");
    m.def("multi_scale_deformable_attn_backward", &multi_scale_deformable_attn_backward,
          "MSDA backward: (value, value_spatial_shapes, value_level_start_index, "
          "sampling_locations, attention_weights, grad_output) -> "
          "(grad_value, grad_sampling_loc, grad_attn_weight)");
    m.def("geometric_kernel_attention_forward", &geometric_kernel_attention_forward,
          "GKA forward: (value, spatial_shapes, level_start_index, sampling_locations, "
          "attention_weights, output) fills output");
    m.def("geometric_kernel_attention_backward", &geometric_kernel_attention_backward,
          "GKA backward: (value, spatial_shapes, level_start_index, sampling_locations, "
          "attention_weights, grad_output) -> (grad_value, grad_attn_weights)");
    m.def("msda_fused_forward", &msda_fused_forward,
          "fused MSDA forward: (value, spatial_shapes, level_start_index, reference_points, "
          "sampling_offsets, attention_logits) -> output");
    m.def("msda_fused_backward", &msda_fused_backward,
          "fused MSDA backward -> (grad_value, grad_reference_points, grad_sampling_offsets, "
          "grad_attention_logits)");
    m.def("npu_deformable_aggregation", &deformable_aggregation,
          "deformable aggregation forward: (mc_ms_feat, spatial_shape, scale_start_index, "
          "sampling_location, weights) -> output");
    m.def("deformable_conv2d", &deformable_conv2d,
          "(x_nhwc, offset_nhwc, weight_ohwi, kernel_size, stride, padding, dilation, groups, "
          "deformable_groups) -> (out [n, c_out, h_out, w_out] view, offset_output)");
    m.def("deformable_conv2d_backward", &deformable_conv2d_backward,
          "(x_nhwc, weight_ohwi, offset_nhwc, offset_output, grad_y_nhwc, kernel_size, stride, "
          "padding, dilation, groups, deformable_groups) -> (grad_x, grad_weight, grad_offset), "
          "each shaped like the NCHW-style original of its tensor");
    m.def("modulated_deformable_conv2d", &modulated_deformable_conv2d,
          "(x_nhwc, offset_nhwc, mask_nhwc, weight_ohwi, bias, kernel_size, stride, padding, "
          "dilation, groups, deformable_groups, with_bias) -> (out, offset_output)");
    m.def("modulated_deformable_conv2d_backward", &modulated_deformable_conv2d_backward,
          "-> (grad_x, grad_weight, grad_bias, grad_offset, grad_mask)");
    m.def("set_status_checks", &set_status_checks,
          "(on) -> previous setting; when on, every operator call synchronises, reads the "
          "device status word and raises if a kernel refused or abandoned work");
    m.def("device_status", [](bool clear) { return msda_sm100_device_status(clear ? 1 : 0); },
          "(clear) -> the device's sticky status bits (synchronises)");
    m.def("dcn_use_tensor_cores", &dcn_use_tensor_cores,
          "1 / 0 selects the tcgen05 / fp32 FMA product kernels; returns the previous setting");
    m.def("npu_add_relu", &npu_add_relu, "x = relu(x + y) in place; returns x");
    m.def("npu_add_relu_grad", &npu_add_relu_grad, "(out, grad_output) -> grad of either addend");
    m.def("npu_max_pool2d", &npu_max_pool2d, "(x, 3, 2, 1) -> max pooled x (inference only)");
    m.def("npu_deformable_aggregation_backward", &deformable_aggregation_backward,
          "deformable aggregation backward -> (grad_mc_ms_feat, grad_sampling_location, "
          "grad_weights)");
}

/* C ABI of the sm_100a multi-scale deformable attention (MSDA) kernels and of the
 * geometric kernel attention kernels that share their machinery (gka_sm100_*).
 *
 * This library sits where the reference's generated operator API sat:
 * `aclnnMultiScaleDeformableAttn[GetWorkspaceSize]` and
 * `aclnnMultiScaleDeformableAttnGrad[GetWorkspaceSize]`, reached through
 * EXEC_NPU_CMD in mx_driving/csrc/MultiScaleDeformableAttn.cpp:63-64 and
 * :115-116 (dispatch macro: include/csrc/OpApiCommon.h:527-614). A host
 * binding checks dtypes and limits, allocates the results and calls in here.
 *
 * Conventions
 *   - plain pointers and sizes only; every data pointer is DEVICE memory of the
 *     current CUDA device, except `spatial_shapes` and `level_start_index`,
 *     which may be host OR device memory (detected per call; host arrays are
 *     passed to the kernel by value, device arrays are read by the kernel);
 *   - layouts are the reference's (mx_driving/ops/multi_scale_deformable_attn.py:22-44):
 *       value               [B, K, H, D]
 *       spatial_shapes      [L, 2] int32, (height, width) per level
 *       level_start_index   [L]    int32, first key of each level
 *       sampling_locations  [B, Q, H, L, P, 2], (x, y) normalised to [0, 1]
 *       attention_weights   [B, Q, H, L, P]
 *       output, grad_output [B, Q, H*D]
 *     all floating tensors share one dtype (MSDA_F32 / MSDA_F16 / MSDA_BF16);
 *   - work is enqueued on `stream` (a cudaStream_t; NULL = default stream);
 *     nothing here synchronises, allocates or frees;
 *   - the caller owns every buffer; outputs are fully overwritten;
 *   - return value: MSDA_OK or a negative msda_status; nothing is thrown;
 *   - re-entrant: no mutable host state is shared between calls except the
 *     tuning knobs below.
 * Limits (same as the reference binding, MultiScaleDeformableAttn.cpp:46-48):
 *   D <= 256, L * P <= 64. Additionally B*K*H and B*Q*H must be below 2^31.
 */
#ifndef MSDA_SM100_H_
#define MSDA_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum msda_dtype {
    MSDA_F32 = 0,
    MSDA_F16 = 1,
    MSDA_BF16 = 2
} msda_dtype;

typedef enum msda_status {
    MSDA_OK = 0,
    MSDA_ERR_NULL = -1,        /* a required pointer is NULL */
    MSDA_ERR_DIMS = -2,        /* a dimension is <= 0 */
    MSDA_ERR_LIMIT = -3,       /* D > 256, L*P > 64, or an index would overflow */
    MSDA_ERR_ALIGN = -4,       /* a pointer is not aligned to its element size */
    MSDA_ERR_DTYPE = -5,       /* unknown dtype code */
    MSDA_ERR_WORKSPACE = -6,   /* workspace missing or too small */
    MSDA_ERR_CUDA = -7         /* a CUDA runtime call failed; see msda_sm100_last_cuda_error */
} msda_status;

/* Forward. Replaces aclnnMultiScaleDeformableAttn
 * (mx_driving/csrc/MultiScaleDeformableAttn.cpp:63-64; device kernel
 * kernels/multi_scale_deformable_attn/op_kernel/multi_scale_deformable_attn.cpp:349-387).
 * Writes output[B, Q, H*D] in `dtype`. */
int msda_sm100_forward(const void* value, const int32_t* spatial_shapes,
                       const int32_t* level_start_index, const void* sampling_locations,
                       const void* attention_weights, void* output, int B, int K, int H, int D,
                       int L, int Q, int P, int dtype, void* stream);

/* Backward. Replaces aclnnMultiScaleDeformableAttnGrad
 * (mx_driving/csrc/MultiScaleDeformableAttn.cpp:115-116; device kernel
 * kernels/multi_scale_deformable_attn/op_kernel/multi_scale_deformable_attn_grad.cpp:312-341).
 * grad_value [B,K,H,D] is zero-filled on `stream` by this call and then
 * accumulated with atomics in its own dtype; grad_sampling_loc and
 * grad_attn_weight are fully written. */
int msda_sm100_backward(const void* value, const int32_t* spatial_shapes,
                        const int32_t* level_start_index, const void* sampling_locations,
                        const void* attention_weights, const void* grad_output, void* grad_value,
                        void* grad_sampling_loc, void* grad_attn_weight, int B, int K, int H,
                        int D, int L, int Q, int P, int dtype, void* stream);

/* Backward with fp32 accumulation of grad_value for the 16-bit dtypes, which is
 * what the reference does for fp16 (it upcasts, runs the fp32 kernel and casts
 * the three gradients back: MultiScaleDeformableAttn.cpp:103-113). `workspace`
 * is caller-owned device memory of at least
 * msda_sm100_backward_workspace_bytes() bytes, 16-byte aligned; its contents
 * on entry do not matter and are undefined on return. For MSDA_F32 the
 * workspace is not used (it may be NULL) and the call equals
 * msda_sm100_backward. This takes the role of the reference's
 * aclnn...GetWorkspaceSize + workspace tensor
 * (include/csrc/OpApiCommon.h:585-610). */
size_t msda_sm100_backward_workspace_bytes(int B, int K, int H, int D, int dtype);
int msda_sm100_backward_ws(const void* value, const int32_t* spatial_shapes,
                           const int32_t* level_start_index, const void* sampling_locations,
                           const void* attention_weights, const void* grad_output,
                           void* grad_value, void* grad_sampling_loc, void* grad_attn_weight,
                           void* workspace, size_t workspace_bytes, int B, int K, int H, int D,
                           int L, int Q, int P, int dtype, void* stream);

/* Backward for callers that cannot allocate device memory. It has no counterpart
 * in the reference (there the framework allocates the operator's workspace for
 * it). Who needs it: a host whose device memory is fully planned before the
 * first operator runs — an inference/training runtime that owns all memory in
 * its own arena, a plug-in inside such a process, a latency-critical loop where
 * calling the device allocator is forbidden — and that therefore cannot hand a
 * workspace to msda_sm100_backward_ws(). The fp32 accumulation scratch lives
 * inside the library instead: one static device array of
 * MSDA_SM100_STATIC_SCRATCH_BYTES bytes, reserved by the driver on every GPU
 * that loads this library and held until the process exits.
 *   - Same operands, results and numerics as msda_sm100_backward_ws(); the
 *     caller still passes every input and output. For MSDA_F32 no scratch is
 *     involved and the call equals msda_sm100_backward().
 *   - Limit: 4 * B*K*H*D bytes must not exceed MSDA_SM100_STATIC_SCRATCH_BYTES
 *     (16-bit dtypes); larger problems are refused with MSDA_ERR_WORKSPACE
 *     before anything is enqueued.
 *   - It calls no allocation or free routine. The first call on each device
 *     looks up the array's device address (and makes the driver load the
 *     module there); make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps whatever the last
 *     call left in it; each call zero-fills the part it uses, on `stream`,
 *     before accumulating. Two calls that overlap on the GPU (different
 *     streams, or different host threads without stream ordering) race on it:
 *     serialise them. */
#define MSDA_SM100_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
size_t msda_sm100_static_scratch_bytes(void);
int msda_sm100_backward_static(const void* value, const int32_t* spatial_shapes,
                               const int32_t* level_start_index, const void* sampling_locations,
                               const void* attention_weights, const void* grad_output,
                               void* grad_value, void* grad_sampling_loc, void* grad_attn_weight,
                               int B, int K, int H, int D, int L, int Q, int P, int dtype,
                               void* stream);

/* Fused MSDA: the operator together with the arithmetic its callers run around it
 * (mmcv's MultiScaleDeformableAttention.forward): sampling location = reference point +
 * offset / (W, H) of the level, attention weight = softmax of the logits over levels*points.
 * No counterpart in the reference library (its models call the plain operator); it removes
 * the softmax and location kernels and the two intermediate tensors between them.
 *   reference_points [B, Q, L, 2] (x, y) in [0, 1]; sampling_offsets [B, Q, H, L, P, 2] in
 *   pixels; attention_logits [B, Q, H, L, P]; all in `dtype`. Limit: L * P <= 32.
 * Backward: grad_value as msda_sm100_backward_ws (same workspace rule); grad_sampling_offsets
 * and grad_attention_logits in `dtype`, fully written; grad_reference_points [B, Q, L, 2] in
 * FLOAT32 (summed over heads and points with atomics; zero-filled by the call). */
int msda_sm100_fused_forward(const void* value, const int32_t* spatial_shapes,
                             const int32_t* level_start_index, const void* reference_points,
                             const void* sampling_offsets, const void* attention_logits,
                             void* output, int B, int K, int H, int D, int L, int Q, int P,
                             int dtype, void* stream);
int msda_sm100_fused_backward_ws(const void* value, const int32_t* spatial_shapes,
                                 const int32_t* level_start_index, const void* reference_points,
                                 const void* sampling_offsets, const void* attention_logits,
                                 const void* grad_output, void* grad_value,
                                 float* grad_reference_points, void* grad_sampling_offsets,
                                 void* grad_attention_logits, void* workspace,
                                 size_t workspace_bytes, int B, int K, int H, int D, int L, int Q,
                                 int P, int dtype, void* stream);

/* Geometric kernel attention (nearest-pixel sampling), forward. Replaces
 * aclnnGeometricKernelAttention (mx_driving/csrc/GeometricKernelAttentionFunc.cpp:34-57;
 * device kernel kernels/geometric_kernel_attention/op_kernel/geometric_kernel_attention.cpp).
 * Same layouts as above, but sampling_locations holds PIXEL coordinates (x, y) of each
 * level (in `dtype`), which are truncated to integers and clamped into the level:
 *   output[b,q,h,:] = sum_{l,p} attention[b,q,h,l,p] * value[b, start_l + y*W_l + x, h, :]. */
int gka_sm100_forward(const void* value, const int32_t* spatial_shapes,
                      const int32_t* level_start_index, const void* sampling_locations,
                      const void* attention_weights, void* output, int B, int K, int H, int D,
                      int L, int Q, int P, int dtype, void* stream);

/* Geometric kernel attention, backward. Replaces aclnnGeometricKernelAttnGrad
 * (mx_driving/csrc/GeometricKernelAttentionFunc.cpp:59-118). grad_value is zero-filled here
 * and accumulated in fp32 (in `workspace` for the 16-bit dtypes: same size rule as
 * msda_sm100_backward_workspace_bytes; unused for MSDA_F32); grad_attn_weight is fully
 * written; sampling locations have no gradient. */
int gka_sm100_backward_ws(const void* value, const int32_t* spatial_shapes,
                          const int32_t* level_start_index, const void* sampling_locations,
                          const void* attention_weights, const void* grad_output,
                          void* grad_value, void* grad_attn_weight, void* workspace,
                          size_t workspace_bytes, int B, int K, int H, int D, int L, int Q, int P,
                          int dtype, void* stream);

/* Deformable aggregation (multi-camera, multi-scale feature sampling with per-group
 * weights), fp32. Replaces aclnnDeformableAggregation / aclnnDeformableAggregationGrad
 * (mx_driving/csrc/DeformableAggregation.cpp:49-50, 72-74; device kernels
 * kernels/deformable_aggregation/op_kernel/deformable_aggregation{,_grad}.cpp).
 *   feat [B, F, C]; spatial_shape [cams, scales, 2] (h, w) and scale_start [cams, scales]
 *   (int32, host or device); sampling_location [B, A, Pts, cams, 2] (w, h) in (0, 1);
 *   weights [B, A, Pts, cams, scales, G]; out / grad_out [B, A, C].
 * A sample counts only if 0 < w < 1 and 0 < h < 1. Limits: C <= 256, C % G == 0, G <= 32,
 * scales <= 32, cams * scales <= 64. Forward zero-fills `out` on `stream` and adds partial sums
 * into it (the order of the fp32 additions is not fixed); backward zero-fills grad_feat on
 * `stream` and fully writes grad_sampling_location and grad_weights. */
int da_sm100_forward(const void* feat, const int32_t* spatial_shape, const int32_t* scale_start,
                     const void* sampling_location, const void* weights, void* out, int B, int F,
                     int C, int A, int Pts, int cams, int scales, int G, void* stream);
int da_sm100_backward(const void* feat, const int32_t* spatial_shape, const int32_t* scale_start,
                      const void* sampling_location, const void* weights, const void* grad_out,
                      void* grad_feat, void* grad_sampling_location, void* grad_weights, int B,
                      int F, int C, int A, int Pts, int cams, int scales, int G, void* stream);
int da_sm100_last_cuda_error(void);

/* Algorithmic (compulsory) bytes one call moves: every operand read once and
 * every result written once. Used by benchmarks for the bandwidth roofline. */
size_t msda_sm100_forward_bytes(int B, int K, int H, int D, int L, int Q, int P, int dtype);
size_t msda_sm100_backward_bytes(int B, int K, int H, int D, int L, int Q, int P, int dtype);

/* Measured ceilings for the operations that bound these kernels (no counterpart in the
 * reference). Times, on the current device, (a) gathers of random rows of gather_row_bytes
 * with 16-byte vector loads and (b) red.global.add.v4.f32 reductions of random rows of
 * red_row_bytes (each 64, 128, 256 or 512) over `buffer` (caller-owned device memory, 16-byte
 * aligned, >= 1 MiB; it is zero-filled and left zero; a size that fits in L2, e.g. 32 MiB,
 * gives the L2 <-> SM rates the MSDA kernels run against) and returns rows per second.
 * Launches a handful of short kernels on `stream` and waits for them. */
int msda_sm100_probe_row_rates(void* buffer, size_t buffer_bytes, int gather_row_bytes,
                               int red_row_bytes, double* gather_rows_per_s,
                               double* red_rows_per_s, void* stream);

/* Sticky device-side status of the current device. Bit 0 (value 1): a staged
 * location/weight tile did not arrive within the polling limit and the kernel
 * fell back to direct loads (results are still correct). Bit 1 (value 2): a
 * pipeline barrier of the tensor-core matrix product (conv_ops_sm100.h) timed
 * out and the CTA stopped early (that call's results are undefined). Bit 2 (value 4): a
 * kernel found the level table it was given in DEVICE memory inconsistent with K (a size
 * <= 0, a negative start, or start + h*w > K) and returned without reading value or writing
 * any result (tables passed in host memory are checked by the entry point, which returns
 * MSDA_ERR_DIMS). Bit 4 (value 16): debug-bounds build only, see msda_sm100_debug_bounds().
 * Synchronises the device. clear != 0 resets it. Returns the status word
 * (>= 0) or a negative msda_status. */
int msda_sm100_device_status(int clear);

/* Tuning knobs, process-wide. Returns the previous value, or MSDA_ERR_DIMS for
 * an unknown knob. Values < 0 only query.
 *   MSDA_TUNE_STAGE          a warp bulk-copies (TMA) its next item's locations/weights into
 *                            shared memory while it works on the current item (never where
 *                            sizes are not multiples of 16): 2 = in the backward kernels only
 *                            (default: measured 3-9 % faster forward kernels than with it),
 *                            1 = in both directions, 0 = direct loads everywhere
 *   MSDA_TUNE_CTAS_PER_SM    persistent CTAs per SM for the forward kernel
 *                            (default 0 = as many as are resident at once)
 *   MSDA_TUNE_CTAS_PER_SM_BWD  same for the backward kernel
 *   MSDA_TUNE_INTERLEAVE     1 = when the whole value tensor is at most 16 MiB (it stays in L2
 *                            whatever the order), walk the (batch, query, head) tasks with
 *                            the batch entries interleaved, so that concurrent reductions
 *                            spread over all entries' gradient maps (default); 0 = always
 *                            walk in memory order
 *   MSDA_TUNE_SPIN_LIMIT     polls of a staging barrier before a warp gives the staged tile
 *                            up, sets status bit 0 and carries on with direct loads (default
 *                            262144). 0 makes every wait run out at once: the way to exercise
 *                            that path without any fault; results stay correct.
 *   MSDA_TUNE_PRECISE_AMP    fp32 tensors: samples with max(W, H) * |attention| >= this value
 *                            accumulate their dot products <value row, grad_out> in double
 *                            from the first product on, the others form the per-lane sums in
 *                            fp32 (default 8; 0 = all samples in double). The location
 *                            gradient multiplies those dot products by W * attention.
 *   MSDA_TUNE_DEBUG_ROW_LIMIT  bounds-checking build only (see msda_sm100_debug_bounds): when
 *                            > 0 the checks behave as if value / grad_value had only this many
 *                            (key, head) rows, so that a test can see them fire on a
 *                            correct problem. Ignored by the normal build.
 *   MSDA_TUNE_PACK_ROWS      1 (default): the forward kernels of the bilinear operators keep a
 *                            record only for the corners that exist and walk those; 0 = one
 *                            record per (sample, corner), missing ones skipped one by one.
 *                            Same results either way. */
typedef enum msda_tune {
    MSDA_TUNE_STAGE = 0,
    MSDA_TUNE_CTAS_PER_SM = 1,
    MSDA_TUNE_CTAS_PER_SM_BWD = 2,
    MSDA_TUNE_INTERLEAVE = 3,
    MSDA_TUNE_SPIN_LIMIT = 4,
    MSDA_TUNE_PRECISE_AMP = 5,
    MSDA_TUNE_DEBUG_ROW_LIMIT = 6,
    MSDA_TUNE_PACK_ROWS = 7
} msda_tune;
int msda_sm100_tune(int knob, int value);

/* Optional timing hook for benchmarks, per host thread. While set, every
 * forward call records (fwd_start, fwd_stop) and every backward call records
 * (bwd_start, bwd_stop) — all cudaEvent_t created by the caller — immediately
 * around its main kernel launch, on the launch stream, so that the kernel can
 * be timed without the zero-fill or the down-conversion. Pass NULLs to clear.
 * An event pair must not be reused before the caller has read it. */
void msda_sm100_profile_events(void* fwd_start, void* fwd_stop, void* bwd_start, void* bwd_stop);

/* Number of kernels this library has launched since load (all threads). */
long long msda_sm100_launch_count(void);

const char* msda_sm100_strerror(int status);
/* cudaError_t of the most recent failing runtime call on this thread (0 if none). */
int msda_sm100_last_cuda_error(void);
/* ABI version of this header: bumps on any signature change. */
int msda_sm100_abi_version(void);
/* 1 when this build of the library was compiled with -DMSDA_DEBUG_BOUNDS: the MSDA and
 * geometric-kernel-attention kernels then check every row offset they compute against the
 * extent of value / grad_value (and every shared-memory accumulator address against its
 * area) before using it; a violation sets bit 4 (value 16) of the device status word and the
 * access is skipped. The reference has no such switch; it flags the same offset arithmetic
 * as hazardous (kernels/multi_scale_deformable_attn/op_kernel/msda.h:428). */
int msda_sm100_debug_bounds(void);

#ifdef __cplusplus
}
#endif

#endif /* MSDA_SM100_H_ */

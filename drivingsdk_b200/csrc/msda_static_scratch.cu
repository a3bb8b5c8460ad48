// Backward entry point for callers that must not allocate device memory.
//
// The 16-bit backward accumulates grad_value in fp32 scratch memory that the caller of
// msda_sm100_backward_ws() has to provide. Some hosts cannot provide it: an inference or
// training runtime that has handed every byte of device memory to its own arena before the
// first operator runs, a plug-in loaded into a process whose memory plan is fixed ahead of
// time, or a real-time loop in which a call into the device allocator (and the implicit
// synchronisation it may bring) is not allowed. For them this file keeps the scratch inside
// the library: one statically sized array in device memory, reserved by the driver when this
// module is loaded on a GPU and held until the process exits. The price is a fixed upper
// limit on the problem size and the loss of concurrency (see the header).
//
// In host code the name of a __device__ array is only a handle for the runtime, not a
// device address, so the address that kernels and cudaMemsetAsync may use is looked up with
// cudaGetSymbolAddress() — once per device, with that device current — and cached.
#include <atomic>

#include <cuda_runtime.h>

#include "../../include/msda_sm100.h"
#include "msda_launch.h"

namespace {

constexpr size_t kScratchBytes = MSDA_SM100_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

struct ScratchAddress {
    std::atomic<int> ready{0};
    void* ptr = nullptr;
};
ScratchAddress g_scratch_of_device[kMaxDevices];

// Device address of the scratch array on the current device. The first call on a device
// resolves the symbol (which also makes the driver load this module there); racing first
// calls do the same idempotent work. Returns a cudaError_t.
cudaError_t scratch_address(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    ScratchAddress& slot = g_scratch_of_device[dev];
    if (!slot.ready.load(std::memory_order_acquire)) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        if (p == nullptr) return cudaErrorInvalidSymbol;
        slot.ptr = p;
        slot.ready.store(1, std::memory_order_release);
    }
    *out = slot.ptr;
    return cudaSuccess;
}

}  // namespace

extern "C" {

size_t msda_sm100_static_scratch_bytes(void) { return kScratchBytes; }

int msda_sm100_backward_static(const void* value, const int32_t* spatial_shapes,
                               const int32_t* level_start_index, const void* sampling_locations,
                               const void* attention_weights, const void* grad_output,
                               void* grad_value, void* grad_sampling_loc, void* grad_attn_weight,
                               int B, int K, int H, int D, int L, int Q, int P, int dtype,
                               void* stream) {
    // An unknown dtype code is refused before anything else, so that it is reported as such
    // whatever the sizes are.
    if (dtype != MSDA_F32 && dtype != MSDA_F16 && dtype != MSDA_BF16) return MSDA_ERR_DTYPE;
    // Size check next, in 64-bit arithmetic and without touching the device: the fp32
    // accumulation buffer of this problem must fit into the static array.
    if (B > 0 && K > 0 && H > 0 && D > 0 && dtype != MSDA_F32) {
        const unsigned long long need = 4ull * static_cast<unsigned long long>(B) *
                                        static_cast<unsigned long long>(K) *
                                        static_cast<unsigned long long>(H) *
                                        static_cast<unsigned long long>(D);
        if (need > kScratchBytes) return MSDA_ERR_WORKSPACE;
    }
    void* scratch = nullptr;
    if (dtype != MSDA_F32) {  // fp32 problems accumulate in grad_value itself: no scratch
        const cudaError_t e = scratch_address(&scratch);
        if (e != cudaSuccess) {
            cudaGetLastError();                  // leave no sticky error behind
            return msda::note_cuda_error(e);     // msda_sm100_last_cuda_error() reports it
        }
    }
    // Everything else — validation, zero-filling the part of the scratch that is used,
    // the kernel, the conversion into grad_value — is the workspace entry point's job.
    return msda_sm100_backward_ws(value, spatial_shapes, level_start_index, sampling_locations,
                                  attention_weights, grad_output, grad_value, grad_sampling_loc,
                                  grad_attn_weight, scratch, scratch ? kScratchBytes : 0, B, K, H,
                                  D, L, Q, P, dtype, stream);
}

}  // extern "C"

// MSDA forward for sm_100a: out[b,q,h,:] = sum over (level, point) of
// attention * bilinear(value[b, level], location), zero outside the level.
// Replaces the reference's forward device kernel and its host tiling
// (kernels/multi_scale_deformable_attn/op_kernel/multi_scale_deformable_attn.cpp:116-250,
//  op_host/multi_scale_deformable_attn.cpp:32-114).
//
// One warp per (batch, query, head) task (several tasks per warp when L*P < 32).
//   phase 1  lane = sample: take (x, y, weight) — bulk-copied to shared memory
//            while the previous item was being gathered — and leave one
//            8-byte record per corner in shared memory: {offset of the value
//            row, bilinear weight * attention}.
//   phase 2  lane = (row slot, 16-byte piece of the row): the warp reads
//            32/LPR whole rows per instruction (LPR lanes x 16 bytes = one
//            contiguous row), four instructions in flight, and accumulates
//            in fp32 registers.
//   epilogue the row-slot groups are summed with xor shuffles and one group
//            writes the D outputs as 16-byte stores.
// Rows whose byte length is not 16 * 2^k take the SCALAR instantiation: lane =
// channel (mod 32), one row per instruction.
#include "msda_fwd_kernel.cuh"

namespace msda {

uint32_t fwd_warp_smem(int samples_per_item, size_t elem) {
    return warp_smem_bytes(samples_per_item, elem, 0);
}

cudaError_t launch_forward(const Params& p, int dtype, const RowPlan& rp, const LaunchShape& ls,
                           cudaStream_t stream) {
    return launch_forward_cps<4>(p, dtype, rp, ls, stream);
}

}  // namespace msda

// C[M, N] = sum_k A[m, k] * B[n, k] on the sm_100a tensor cores with fp32 accuracy.
//
// Operands are fp32 in global memory with k contiguous. A TF32 tensor-core product keeps only
// 10 mantissa bits of each operand, which is not enough for a convolution whose results are
// compared with an fp32 implementation at 1e-4, so every operand is split in two TF32-exact
// parts, v = hi + lo with hi = v rounded towards zero to TF32 and lo = v - hi (exact in fp32),
// and three products are accumulated per tile: lo*hi + hi*lo + hi*hi (lo*lo is below fp32
// resolution). Accumulation is fp32, in tensor memory.
//
// A work item is one 128 x BN tile of C (BN = 64, 128 or 256) over one part of K; the kernel is
// persistent (one CTA per SM, items dealt round-robin) and walks K in stages of 16 or 32 k (one
// swizzled shared-memory row per operand row):
//   warp 0        producer: one lane issues the two TMA tile loads of a stage
//   warp 1        MMA: one lane issues the k-slices x 3 products of tcgen05.mma per stage and
//                 commits the stage's "empty" barrier; owns the tensor-memory allocation, which
//                 holds two accumulators used alternately
//   warps 2..5    splitters: write the lo part of the raw tile into a second buffer at the same
//                 offsets (so the swizzle pattern does not matter; the raw tile itself serves
//                 as the hi part because the tensor core ignores the low 13 mantissa bits),
//                 then hand the stage to the MMA warp
//   warps 6..9    epilogue: tcgen05.ld of a finished accumulator (warp q reads lanes
//                 32q..32q+31), bias, stores (or reductions when K is cut across items), then
//                 hand the accumulator back; this overlaps the products of the next item
// Operands may also be stored with the row index contiguous (the grad_weight product): 3-D TMA
// maps and the 32-byte-chunk swizzle, same pipeline.
// Out-of-range parts of a tile (M, N or K tails) are zero-filled by TMA and masked in the
// epilogue. A single-product mode (PASSES == 1) skips the split and uses the freed shared
// memory for twice as many stages. Every barrier wait is bounded: on a timeout the CTA raises
// the library's sticky status word, stops issuing work, waits (bounded) for its own copies,
// frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "gemm_sm100.h"
#include "msda_common.cuh"

namespace msda {
namespace {

constexpr int BM = 128;
// k extent of a stage in fp32 elements: one swizzled shared-memory row per operand row.
// The three-product mode doubles a stage's footprint (lo parts), so it uses 64-byte rows to
// keep four stages in flight; two were not enough to cover the TMA latency.
constexpr int kBkSplit = 16;                // 64-byte rows, 64-byte swizzle
constexpr int kBkPlain = 32;                // 128-byte rows, 128-byte swizzle
constexpr int kGemmThreads = 320;           // producer, MMA, 4 splitter and 4 epilogue warps
constexpr int kStatusGemmTimeout = 2;       // bit in the sticky status word
constexpr int kWaitLimit = 1 << 22;

// A stage holds the raw A and B tiles and, for the three-product mode, their lo parts.
template <int BN, int PASSES>
struct Tile {
    static constexpr int BK = (PASSES == 3) ? kBkSplit : kBkPlain;
    static constexpr int kRowBytes = BK * 4;
    static constexpr int kTileABytes = BM * kRowBytes;
    static constexpr int kTileBBytes = BN * kRowBytes;
    static constexpr int kStageBytes = (PASSES == 3 ? 2 : 1) * (kTileABytes + kTileBBytes);
    static constexpr int kFit = (192 * 1024) / kStageBytes;
    static constexpr int kStages = kFit > 8 ? 8 : kFit;
    // + barriers and the tensor-memory address, + slack to align the tiles to 1 KiB
    static constexpr int kSmemBytes = kStages * kStageBytes + 256 + 1024;
};

__device__ __forceinline__ bool gemm_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (int spin = 0; spin < kWaitLimit; ++spin) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
        if (spin > 1024) __nanosleep(64);
    }
    return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 2-D tiled TMA load into this CTA's shared memory; coordinates are (k, row).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}

// The same for a 3-D map; used for operands whose contiguous index is the row (m or n):
// coordinates are (0, k, row / 32).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory operand descriptor: k-major rows of ROW_BYTES (128 or 64) swizzled at that
// width, 8-row groups 8 * ROW_BYTES apart.
template <int ROW_BYTES>
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
    static_assert(ROW_BYTES == 128 || ROW_BYTES == 64, "row width");
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);            // start address
    d |= static_cast<uint64_t>((8 * ROW_BYTES) >> 4) << 32;              // stride between 8-row groups
    d |= 1ull << 46;                                                     // descriptor version (sm_100)
    d |= static_cast<uint64_t>(ROW_BYTES == 128 ? 2 : 4) << 61;          // 128- / 64-byte swizzle
    return d;
}

// Descriptor of a row-contiguous ("MN-major") operand tile: 128-byte lines of 32 consecutive
// m (or n) for one k. For 32-bit operands the tensor core takes this form only with the
// "128-byte swizzle on 32-byte chunks" pattern, whose groups are four lines (four k) of
// 512 bytes; groups follow each other along k, the next 32 m (or n) start `block_bytes`
// further on.
__device__ __forceinline__ uint64_t operand_desc_mn(uint32_t smem_addr, uint32_t block_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(block_bytes >> 4) << 16;      // leading offset: next 32 rows
    d |= static_cast<uint64_t>(512 >> 4) << 32;               // stride offset: next 4 k
    d |= 1ull << 46;
    d |= 1ull << 61;                                          // 128-byte swizzle, 32-byte chunks
    return d;
}

// Instruction descriptor: TF32 x TF32 -> fp32, M = 128, N = BN; both operands k-major, or
// both row-contiguous (bits 15 and 16).
template <int BN>
__device__ __forceinline__ uint32_t instr_desc(bool mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (mn_major ? (3u << 15) : 0u) |
           (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                     "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct TcParams {
    float* C;
    long long ldc;
    const float* bias;
    int M, N, K;
    int kb_per_split;   // k-blocks (of BK) per work item
    int n_splits;       // parts K is cut into
    int n_tiles;        // tiles along N
    int total_tiles;    // tiles of C; work item w = split * total_tiles + tile, tile = m_tile * n_tiles + n_tile
    int mn_major;       // operands are row-contiguous (A[k][m], B[k][n]) instead of k-contiguous
    int reduce;         // add into C with reductions (K is cut across work items)
    int* status;
};

// One work item: a 128 x BN tile of C over one part of K.
struct WorkItem {
    int m0, n0, kb_begin, num_kb, split;
};
template <int BN, int BK>
__device__ __forceinline__ WorkItem work_item(const TcParams& p, int w) {
    const int split = w / p.total_tiles;
    const int tile = w - split * p.total_tiles;
    WorkItem it;
    it.split = split;
    // tiles that share a row block of A are neighbours in the order, so A comes from HBM once
    it.m0 = (tile / p.n_tiles) * BM;
    it.n0 = (tile % p.n_tiles) * BN;
    const int kb_total = (p.K + BK - 1) / BK;
    it.kb_begin = split * p.kb_per_split;
    it.num_kb = min(kb_total, it.kb_begin + p.kb_per_split) - it.kb_begin;
    return it;
}

// PASSES == 3: hi/lo split, fp32-class accuracy; PASSES == 1: one TF32 product per tile.
// Persistent: CTA c takes work items c, c + gridDim.x, ...; the accumulator alternates between
// two tensor-memory buffers so that the epilogue of one item overlaps the products of the next.
template <int BN, int PASSES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const TcParams p) {
    using T = Tile<BN, PASSES>;
    constexpr int kStages = T::kStages;
    constexpr int BK = T::BK;
    constexpr int kTileABytes = T::kTileABytes;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base_u32 = smem_u32(smem_raw);
    uint8_t* tiles = smem_raw + ((1024u - (base_u32 & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + kStages * T::kStageBytes);
    uint64_t* full_raw = bars;                      // TMA landed
    uint64_t* full_split = bars + kStages;          // lo parts written
    uint64_t* empty = bars + 2 * kStages;           // the MMAs that read the stage have finished
    uint64_t* accum_full = bars + 3 * kStages;      // [2] every MMA of the item has finished
    uint64_t* accum_empty = bars + 3 * kStages + 2; // [2] the epilogue has read the accumulator
    static_assert((3 * kStages + 5) * 8 + 8 <= 256, "barrier area");
    uint64_t* drained = bars + 3 * kStages + 4;     // abort path only: the issued MMAs have retired
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * kStages + 5);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_items = p.total_tiles * p.n_splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_raw[s], 1);
            mbar_init(&full_split[s], 4);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&accum_full[a], 1);
            mbar_init(&accum_empty[a], 4);
        }
        mbar_init(drained, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::
                         "r"(smem_u32(tmem_slot)), "r"(static_cast<uint32_t>(2 * BN))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    auto stage_ptr = [&](int s) { return tiles + s * T::kStageBytes; };
    auto give_up = [&]() {
        atomicOr(p.status, kStatusGemmTimeout);
        *abort_flag = 1;
    };

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t it = 0;   // k-blocks issued so far, over all items
            for (int w = blockIdx.x; w < total_items && !*abort_flag; w += gridDim.x) {
                const WorkItem wi = work_item<BN, BK>(p, w);
                for (int i = 0; i < wi.num_kb && !*abort_flag; ++i, ++it) {
                    const int s = it % kStages;
                    const uint32_t round = it / kStages;
                    if (!gemm_wait(&empty[s], (round & 1u) ^ 1u)) {
                        give_up();
                        break;
                    }
                    uint8_t* st = stage_ptr(s);
                    mbar_expect_tx(&full_raw[s], kTileABytes + T::kTileBBytes);
                    const int k0 = (wi.kb_begin + i) * BK;
                    if (p.mn_major) {
                        tma_load_3d(st, &map_a, 0, k0, wi.m0 / 32, &full_raw[s]);
                        tma_load_3d(st + kTileABytes, &map_b, 0, k0, wi.n0 / 32, &full_raw[s]);
                    } else {
                        tma_load_2d(st, &map_a, k0, wi.m0, &full_raw[s]);
                        tma_load_2d(st + kTileABytes, &map_b, k0, wi.n0, &full_raw[s]);
                    }
                }
            }
            // Let the copies that were issued land before the CTA goes away, whoever gave up
            // (when nothing went wrong these phases have completed and the waits return at once).
            const uint32_t first = it > static_cast<uint32_t>(kStages) ? it - kStages : 0u;
            for (uint32_t j = first; j < it; ++j)
                gemm_wait(&full_raw[j % kStages], (j / kStages) & 1u);
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc<BN>(p.mn_major != 0);
            uint32_t it = 0, item = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x, ++item) {
                const WorkItem wi = work_item<BN, BK>(p, w);
                const uint32_t acc = item & 1u, use = item >> 1;
                const uint32_t tmem_d = tmem_base + acc * BN;
                // the epilogue must have drained this accumulator's previous item
                if (*abort_flag || !gemm_wait(&accum_empty[acc], (use & 1u) ^ 1u)) {
                    give_up();
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int i = 0; i < wi.num_kb; ++i, ++it) {
                    const int s = it % kStages;
                    const uint32_t round = it / kStages;
                    if (*abort_flag || !gemm_wait(&full_split[s], round & 1u)) {
                        give_up();
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_hi = smem_u32(stage_ptr(s));
                    const uint32_t b_hi = a_hi + kTileABytes;
                    const uint32_t a_lo = b_hi + T::kTileBBytes;   // only present when PASSES == 3
                    const uint32_t b_lo = a_lo + kTileABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / 8; ++kk) {
                        uint64_t dah, dal, dbh, dbl;
                        if (p.mn_major) {
                            const uint32_t off = kk * 1024;       // next group of 8 k
                            constexpr uint32_t kBlock = BK * 128;  // 32 rows x BK k
                            dah = operand_desc_mn(a_hi + off, kBlock);
                            dal = operand_desc_mn(a_lo + off, kBlock);
                            dbh = operand_desc_mn(b_hi + off, kBlock);
                            dbl = operand_desc_mn(b_lo + off, kBlock);
                        } else {
                            const uint32_t off = kk * 32;         // 8 TF32 values along k
                            dah = operand_desc<T::kRowBytes>(a_hi + off);
                            dal = operand_desc<T::kRowBytes>(a_lo + off);
                            dbh = operand_desc<T::kRowBytes>(b_hi + off);
                            dbl = operand_desc<T::kRowBytes>(b_lo + off);
                        }
                        const uint32_t fresh = (i > 0 || kk > 0) ? 1u : 0u;
                        if (PASSES == 3) {
                            mma_tf32(tmem_d, dal, dbh, idesc, fresh);
                            mma_tf32(tmem_d, dah, dbl, idesc, 1u);
                            mma_tf32(tmem_d, dah, dbh, idesc, 1u);
                        } else {
                            // the tensor core reads the upper 19 bits of each fp32 operand
                            mma_tf32(tmem_d, dah, dbh, idesc, fresh);
                        }
                    }
                    mma_commit(&empty[s]);   // arrives when these MMAs no longer read the stage
                }
                if (ok) mma_commit(&accum_full[acc]);
            }
            if (!ok || *abort_flag) {
                // Abandoning work: the MMAs already issued still write tensor memory and read
                // the stages. Wait (bounded) until they have retired, so that the tensor
                // memory is not handed back underneath them.
                mma_commit(drained);
                gemm_wait(drained, 0u);
            }
        }
    } else if (warp < 6) {
        // ---------------- splitters ----------------
        const int t = threadIdx.x - 64;          // 0..127
        uint32_t it = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
            const WorkItem wi = work_item<BN, BK>(p, w);
            for (int i = 0; i < wi.num_kb; ++i, ++it) {
                const int s = it % kStages;
                const uint32_t round = it / kStages;
                if (*abort_flag || !gemm_wait(&full_raw[s], round & 1u)) {
                    if (lane == 0) give_up();
                    ok = false;
                    break;
                }
                if (PASSES == 3) {
                    // The tensor core uses the upper 19 bits of an fp32 operand (sign, exponent,
                    // 10 mantissa bits) and ignores the rest, so the raw tile already acts as the
                    // hi part; only lo = v - hi has to be produced. Raw A and B are contiguous,
                    // and so are their lo parts behind them.
                    const uint8_t* raw = stage_ptr(s);
                    uint8_t* lo_buf = stage_ptr(s) + kTileABytes + T::kTileBBytes;
#pragma unroll 4
                    for (int v = t; v < (kTileABytes + T::kTileBBytes) / 16; v += 128) {
                        const uint4 x = *reinterpret_cast<const uint4*>(raw + v * 16);
                        uint4 lo;
                        lo.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(x.x & 0xffffe000u));
                        lo.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(x.y & 0xffffe000u));
                        lo.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(x.z & 0xffffe000u));
                        lo.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(x.w & 0xffffe000u));
                        *reinterpret_cast<uint4*>(lo_buf + v * 16) = lo;
                    }
                    // make the generic-proxy writes visible to the tensor core's reads
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_split[s]);
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;                       // tensor-memory lane quarter of this warp
        const bool vec_ok = (p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        uint32_t item = 0;
        for (int w = blockIdx.x; w < total_items; w += gridDim.x, ++item) {
            const WorkItem wi = work_item<BN, BK>(p, w);
            const uint32_t acc = item & 1u, use = item >> 1;
            if (*abort_flag || !gemm_wait(&accum_full[acc], use & 1u)) {
                if (lane == 0) give_up();
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m = wi.m0 + 32 * q + lane;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_load_32(tmem_base + (static_cast<uint32_t>(32 * q) << 16) + acc * BN + c * 32, r);
                if (m >= p.M) continue;
                const int n_first = wi.n0 + c * 32;
                float* row = p.C + static_cast<long long>(m) * p.ldc;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const int n = n_first + j;
                    if (n >= p.N) break;
                    float v[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        v[e] = __uint_as_float(r[j + e]);
                        // with K cut across work items the first part carries the bias
                        if (p.bias != nullptr && wi.split == 0 && n + e < p.N) v[e] += p.bias[n + e];
                    }
                    if (vec_ok && n + 3 < p.N) {
                        if (p.reduce) red_add_f32x4(row + n, v[0], v[1], v[2], v[3]);
                        else *reinterpret_cast<float4*>(row + n) = make_float4(v[0], v[1], v[2], v[3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (n + e < p.N) {
                                if (p.reduce) atomicAdd(row + n + e, v[e]);
                                else row[n + e] = v[e];
                            }
                        }
                    }
                }
            }
            // hand the accumulator back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&accum_empty[acc]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(static_cast<uint32_t>(2 * BN))
                     : "memory");
    }
}

// ------------------------------- host side -------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::atomic<EncodeTiledFn> g_encode{nullptr};

cudaError_t encode_fn(EncodeTiledFn* out) {
    EncodeTiledFn fn = g_encode.load(std::memory_order_acquire);
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (q != cudaDriverEntryPointSuccess || sym == nullptr) return cudaErrorNotSupported;
        fn = reinterpret_cast<EncodeTiledFn>(sym);
        g_encode.store(fn, std::memory_order_release);
    }
    *out = fn;
    return cudaSuccess;
}

// [rows, K] fp32 matrix with k contiguous -> map with boxes of (bk k) x (box_rows rows),
// swizzled at the width of a box row
cudaError_t make_map(CUtensorMap* map, const float* base, long long row_stride, int rows, int K,
                     int box_rows, int bk) {
    EncodeTiledFn fn = nullptr;
    cudaError_t e = encode_fn(&fn);
    if (e != cudaSuccess) return e;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride) * 4};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(bk), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims,
                          strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          bk * 4 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// [K, rows] fp32 matrix with the row index contiguous (element (row, k) at base[k * k_stride +
// row]) seen as [rows / 32][K][32]: one box brings (box_rows / 32) blocks of bk k x 32 rows, each
// k a 128-byte line swizzled in 32-byte chunks. rows must be a multiple of 32.
cudaError_t make_map_mn(CUtensorMap* map, const float* base, long long k_stride, int rows, int K,
                        int box_rows, int bk) {
    EncodeTiledFn fn = nullptr;
    cudaError_t e = encode_fn(&fn);
    if (e != cudaSuccess) return e;
    const cuuint64_t dims[3] = {32, static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows / 32)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(k_stride) * 4, 128};
    const cuuint32_t box[3] = {32, static_cast<cuuint32_t>(bk), static_cast<cuuint32_t>(box_rows / 32)};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims,
                          strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

bool k_major_ok(const GemmArgs& g) {
    return g.a_k == 1 && g.b_k == 1 && g.a_row % 4 == 0 && g.b_row % 4 == 0 &&
           g.a_row * 4 < (1ll << 40) && g.b_row * 4 < (1ll << 40);
}
bool mn_major_ok(const GemmArgs& g) {
    return g.a_row == 1 && g.b_row == 1 && g.a_k % 4 == 0 && g.b_k % 4 == 0 && g.M % 32 == 0 &&
           g.N % 32 == 0 && g.a_k * 4 < (1ll << 40) && g.b_k * 4 < (1ll << 40);
}

template <int BN, int PASSES>
cudaError_t launch(const GemmArgs& g, int splits, int* status, cudaStream_t stream) {
    // per device and cheap, so set on every launch (a process may drive several devices)
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, PASSES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Tile<BN, PASSES>::kSmemBytes);
    if (e != cudaSuccess) return e;
    CUtensorMap map_a, map_b;
    constexpr int BK = Tile<BN, PASSES>::BK;
    const bool mn_major = !k_major_ok(g);
    e = mn_major ? make_map_mn(&map_a, g.A, g.a_k, g.M, g.K, BM, BK)
                             : make_map(&map_a, g.A, g.a_row, g.M, g.K, BM, BK);
    if (e != cudaSuccess) return e;
    e = mn_major ? make_map_mn(&map_b, g.B, g.b_k, g.N, g.K, BN, BK)
                 : make_map(&map_b, g.B, g.b_row, g.N, g.K, BN, BK);
    if (e != cudaSuccess) return e;
    const int kb_total = (g.K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > kb_total) splits = kb_total;
    TcParams p;
    p.C = g.C;
    p.ldc = g.ldc;
    p.bias = g.bias;
    p.M = g.M;
    p.N = g.N;
    p.K = g.K;
    p.kb_per_split = (kb_total + splits - 1) / splits;
    p.n_splits = (kb_total + p.kb_per_split - 1) / p.kb_per_split;   // no part is empty
    p.reduce = p.n_splits > 1 ? 1 : 0;
    p.status = status;
    p.n_tiles = (g.N + BN - 1) / BN;
    p.mn_major = mn_major ? 1 : 0;
    const long long tiles = static_cast<long long>((g.M + BM - 1) / BM) * p.n_tiles;
    if (tiles * p.n_splits >= (1ll << 31)) return cudaErrorInvalidValue;
    p.total_tiles = static_cast<int>(tiles);
    int dev = 0, sms = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    const long long items = tiles * p.n_splits;
    const dim3 grid(static_cast<unsigned>(items < sms ? items : sms));   // one CTA per SM
    gemm_tc_kernel<BN, PASSES><<<grid, kGemmThreads, Tile<BN, PASSES>::kSmemBytes, stream>>>(map_a, map_b, p);
    return cudaGetLastError();
}

}  // namespace

bool gemm_tc_supported(const GemmArgs& g) {
    if (g.M <= 0 || g.N <= 0 || g.K <= 0) return false;
    if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B)) % 16 != 0) return false;
    return k_major_ok(g) || mn_major_ok(g);
}

cudaError_t gemm_tc(const GemmArgs& g, int splits, int passes, int* status_word,
                    cudaStream_t stream) {
    if (!gemm_tc_supported(g) || status_word == nullptr) return cudaErrorInvalidValue;
    if (passes != 1 && passes != 3) return cudaErrorInvalidValue;
    // widest tile that N fills to at least three quarters; measured on B200 at N = 512 and
    // N = 4608: 256-wide tiles are 10-40 % faster than 128-wide ones in both modes
    const int bn = g.N > 128 + 64 ? 256 : (g.N > 64 + 32 ? 128 : 64);
    if (passes == 3) {
        if (bn == 256) return launch<256, 3>(g, splits, status_word, stream);
        if (bn == 128) return launch<128, 3>(g, splits, status_word, stream);
        return launch<64, 3>(g, splits, status_word, stream);
    }
    if (bn == 256) return launch<256, 1>(g, splits, status_word, stream);
    if (bn == 128) return launch<128, 1>(g, splits, status_word, stream);
    return launch<64, 1>(g, splits, status_word, stream);
}

}  // namespace msda

// Deformable / modulated deformable 2-D convolution for sm_100a, fp32, channels-last.
//
// The operator is a data-dependent gather followed by a dense product, and is built that way:
//   forward   gather kernel: columns[m, g, tap, c] = mask * bilinear(x[n], p(m, tap))
//             product:       out[m, co] = sum columns[m, g, :] . weight[co, :]  (+ bias)
//   backward  product:       grad_columns = grad_out x weight
//             scatter kernel: grad_x (+= through reductions), grad_offset, grad_mask
//             product:       grad_weight = grad_out^T x columns
// m runs over the N * Ho * Wo output pixels. The gather and scatter kernels are the part that
// is specific to this operator; they move whole channel rows (C / deform_groups contiguous
// floats per corner) as 16-byte pieces, a group of lanes per (pixel, deformable group, tap),
// and are bound by L2 / HBM traffic. The products go to the tensor cores (gemm_tc) when the
// operands meet its alignment rules, else to the fp32 FMA kernel.
//
// Replaces kernels/deformable_conv2d/op_kernel/deformable_conv2d.cpp (gather :223-420, product
// :206-221) and deformable_conv2d_grad.cpp of the reference, and the aclnn calls of
// mx_driving/csrc/DeformableConv2d.cpp:59-60, 92-94 and ModulatedDeformableConv2d.cpp.
#include <atomic>
#include <cstdint>

#include "../../include/conv_ops_sm100.h"
#include "gemm_sm100.h"
#include "msda_launch.h"

namespace {

using msda::FastDiv;
using msda::fd_div;

constexpr int kThreads = 256;

struct DcnParams {
    const float* x;
    const float* offset;
    const float* mask;      // null: not modulated
    float* columns;         // forward: written; backward: grad_columns, read
    float* grad_x;
    float* grad_offset;
    float* grad_mask;
    int H, W, C;
    int Wo, HoWo;
    int K, kw;              // taps, taps per kernel row
    int sh, sw, ph, pw, dh, dw;
    int DG, Cd;             // deformable groups, channels per deformable group
    int Cg, G;              // channels per weight group, weight groups
    int pieces;             // Cd / VEC (VEC = 4 floats per piece, or 1 for odd channel counts)
    int lpi_log2;           // lanes per item = 1 << lpi_log2
    uint32_t items;         // M * DG * K
    FastDiv fd_K, fd_DG, fd_HoWo, fd_Wo, fd_kw, fd_Cg;
};

struct Sample {
    float w[4];        // corner weights (bilinear, times the mask in the forward)
    const float* row[4];  // corner rows of x (this deformable group's channels), null if missing
    float lh, lw;
    bool valid;
};

// Position, corners and weights of item (m, dg, k); every lane of the item's group computes
// the same thing. Fractions come from the fp32 position as in the reference
// (deformable_conv2d.cpp:253-262: floor, then position - floor).
__device__ __forceinline__ void item_setup(const DcnParams& p, uint32_t item, uint32_t* m_out,
                                           uint32_t* dg_out, uint32_t* k_out, float* mask_out,
                                           Sample* s) {
    const uint32_t t = fd_div(item, p.fd_K);
    const uint32_t k = item - t * p.K;
    const uint32_t m = fd_div(t, p.fd_DG);
    const uint32_t dg = t - m * p.DG;
    const uint32_t n = fd_div(m, p.fd_HoWo);
    const uint32_t r = m - n * p.HoWo;
    const uint32_t ho = fd_div(r, p.fd_Wo);
    const uint32_t wo = r - ho * p.Wo;
    const uint32_t ki = fd_div(k, p.fd_kw);
    const uint32_t kj = k - ki * p.kw;
    const float2 d = *reinterpret_cast<const float2*>(
        p.offset + (static_cast<size_t>(m) * p.DG + dg) * (2 * p.K) + 2 * k);
    const float py = static_cast<float>(static_cast<int>(ho) * p.sh - p.ph + static_cast<int>(ki) * p.dh) + d.x;
    const float px = static_cast<float>(static_cast<int>(wo) * p.sw - p.pw + static_cast<int>(kj) * p.dw) + d.y;
    *mask_out = p.mask ? p.mask[(static_cast<size_t>(m) * p.DG + dg) * p.K + k] : 1.f;
    *m_out = m;
    *dg_out = dg;
    *k_out = k;
    const float Hf = static_cast<float>(p.H), Wf = static_cast<float>(p.W);
    s->valid = (py > -1.f) && (px > -1.f) && (py < Hf) && (px < Wf);  // false for NaN
    const float fy = floorf(py), fx = floorf(px);
    const float lh = s->valid ? py - fy : 0.f, lw = s->valid ? px - fx : 0.f;
    const float hh = 1.f - lh, hw = 1.f - lw;
    s->lh = lh;
    s->lw = lw;
    const int y0 = s->valid ? static_cast<int>(fy) : 0, x0 = s->valid ? static_cast<int>(fx) : 0;
    const bool top = y0 >= 0, bottom = y0 + 1 <= p.H - 1, left = x0 >= 0, right = x0 + 1 <= p.W - 1;
    const float* plane = p.x + static_cast<size_t>(n) * p.H * p.W * p.C + static_cast<size_t>(dg) * p.Cd;
    const ptrdiff_t at = (static_cast<ptrdiff_t>(y0) * p.W + x0) * p.C;
    const ptrdiff_t dx = p.C, dy = static_cast<ptrdiff_t>(p.W) * p.C;
    s->row[0] = (s->valid && top && left) ? plane + at : nullptr;
    s->row[1] = (s->valid && top && right) ? plane + at + dx : nullptr;
    s->row[2] = (s->valid && bottom && left) ? plane + at + dy : nullptr;
    s->row[3] = (s->valid && bottom && right) ? plane + at + dy + dx : nullptr;
    s->w[0] = hh * hw;
    s->w[1] = hh * lw;
    s->w[2] = lh * hw;
    s->w[3] = lh * lw;
}

// A piece of a channel row: VEC consecutive floats, kept in a float4 (unused parts zero).
template <int VEC>
__device__ __forceinline__ float4 load_piece(const float* row, int piece) {
    if (row == nullptr) return make_float4(0.f, 0.f, 0.f, 0.f);
    if (VEC == 4) {
        const uint4 r = msda::ldg16(row + 4 * piece);
        return make_float4(__uint_as_float(r.x), __uint_as_float(r.y), __uint_as_float(r.z),
                           __uint_as_float(r.w));
    }
    return make_float4(__ldg(row + piece), 0.f, 0.f, 0.f);
}
template <int VEC>
__device__ __forceinline__ float4 load_column_piece(const float* p) {
    if (VEC == 4) return *reinterpret_cast<const float4*>(p);
    return make_float4(*p, 0.f, 0.f, 0.f);
}
template <int VEC>
__device__ __forceinline__ void store_column_piece(float* p, const float4& v) {
    if (VEC == 4) *reinterpret_cast<float4*>(p) = v;
    else *p = v.x;
}
template <int VEC>
__device__ __forceinline__ void red_piece(float* p, float a, float b, float c, float d) {
    if (VEC == 4) msda::red_add_f32x4(p, a, b, c, d);
    else atomicAdd(p, a);
}

// index of channel c of (m, tap k) in the columns tensor [M, G, K, Cg]
__device__ __forceinline__ size_t column_index(const DcnParams& p, uint32_t m, uint32_t k,
                                               uint32_t c) {
    const uint32_t g = fd_div(c, p.fd_Cg);
    const uint32_t cg = c - g * p.Cg;
    return ((static_cast<size_t>(m) * p.G + g) * p.K + k) * p.Cg + cg;
}

template <bool BACKWARD, int VEC>
__global__ void __launch_bounds__(kThreads, 4)
dcn_sample_kernel(const DcnParams p) {
    const int lane = threadIdx.x & 31;
    const int lpi = 1 << p.lpi_log2;
    const int sub = lane & (lpi - 1);            // piece lane within the item
    const int slot = lane >> p.lpi_log2;         // item within the warp
    const uint32_t items_per_warp = 32u >> p.lpi_log2;
    const uint32_t warp = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    const uint32_t warps = (gridDim.x * kThreads) >> 5;

    for (uint32_t first = warp * items_per_warp; first < p.items; first += warps * items_per_warp) {
        const uint32_t item = first + slot;
        const bool live = item < p.items;
        uint32_t m = 0, dg = 0, k = 0;
        float mk = 0.f;
        Sample s;
        if (live) {
            item_setup(p, item, &m, &dg, &k, &mk, &s);
        } else {
            s.valid = false;
            s.lh = s.lw = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                s.row[c] = nullptr;
                s.w[c] = 0.f;
            }
        }
        if (!BACKWARD) {
            if (live) {
                for (int piece = sub; piece < p.pieces; piece += lpi) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (s.valid) {
                        float4 v[4];
#pragma unroll
                        for (int c = 0; c < 4; ++c) v[c] = load_piece<VEC>(s.row[c], piece);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float w = s.w[c] * mk;
                            acc.x = fmaf(w, v[c].x, acc.x);
                            acc.y = fmaf(w, v[c].y, acc.y);
                            acc.z = fmaf(w, v[c].z, acc.z);
                            acc.w = fmaf(w, v[c].w, acc.w);
                        }
                    }
                    store_column_piece<VEC>(p.columns + column_index(p, m, k, dg * p.Cd + VEC * piece), acc);
                }
            }
        } else {
            // dots of the column gradient with the sample and with its derivatives
            float d_val = 0.f, d_dy = 0.f, d_dx = 0.f;
            if (live && s.valid) {
                const float hh = 1.f - s.lh, hw = 1.f - s.lw;
                float* grow[4];
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    grow[c] = s.row[c] ? p.grad_x + (s.row[c] - p.x) : nullptr;
                for (int piece = sub; piece < p.pieces; piece += lpi) {
                    const float4 g = load_column_piece<VEC>(
                        p.columns + column_index(p, m, k, dg * p.Cd + VEC * piece));
                    float4 v[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) v[c] = load_piece<VEC>(s.row[c], piece);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if (grow[c] != nullptr) {
                            const float w = s.w[c] * mk;
                            red_piece<VEC>(grow[c] + VEC * piece, w * g.x, w * g.y, w * g.z, w * g.w);
                        }
                    }
                    const float gx[4] = {g.x, g.y, g.z, g.w};
                    const float v0[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
                    const float v1[4] = {v[1].x, v[1].y, v[1].z, v[1].w};
                    const float v2[4] = {v[2].x, v[2].y, v[2].z, v[2].w};
                    const float v3[4] = {v[3].x, v[3].y, v[3].z, v[3].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float val = s.w[0] * v0[e] + s.w[1] * v1[e] + s.w[2] * v2[e] + s.w[3] * v3[e];
                        const float dy = hw * (v2[e] - v0[e]) + s.lw * (v3[e] - v1[e]);
                        const float dx = hh * (v1[e] - v0[e]) + s.lh * (v3[e] - v2[e]);
                        d_val = fmaf(gx[e], val, d_val);
                        d_dy = fmaf(gx[e], dy, d_dy);
                        d_dx = fmaf(gx[e], dx, d_dx);
                    }
                }
            }
            for (int o = lpi >> 1; o > 0; o >>= 1) {
                d_val += __shfl_xor_sync(0xffffffffu, d_val, o);
                d_dy += __shfl_xor_sync(0xffffffffu, d_dy, o);
                d_dx += __shfl_xor_sync(0xffffffffu, d_dx, o);
            }
            if (live && sub == 0) {
                const size_t at = (static_cast<size_t>(m) * p.DG + dg) * p.K + k;
                *reinterpret_cast<float2*>(p.grad_offset + 2 * at) = 
                    s.valid ? make_float2(mk * d_dy, mk * d_dx) : make_float2(0.f, 0.f);
                if (p.grad_mask != nullptr) p.grad_mask[at] = d_val;
            }
        }
    }
}

// grad_bias[c] = sum over rows of grad_out[r, c]
__global__ void __launch_bounds__(kThreads)
column_sum_kernel(const float* __restrict__ a, int rows, int cols, int rows_per_block,
                  float* __restrict__ sums) {
    const int c = blockIdx.y * kThreads + threadIdx.x;
    if (c >= cols) return;
    const int r0 = blockIdx.x * rows_per_block;
    const int r1 = min(rows, r0 + rows_per_block);
    float acc = 0.f;
    for (int r = r0; r < r1; ++r) acc += a[static_cast<size_t>(r) * cols + c];
    atomicAdd(sums + c, acc);
}

std::atomic<int> g_use_tc{1};

struct Derived {
    long long M;
    int K, Kd, Cg, Cog, Cd;
};

int check_shape(const dcn_shape* s, Derived* d) {
    if (s == nullptr) return MSDA_ERR_NULL;
    if (s->N <= 0 || s->H <= 0 || s->W <= 0 || s->C <= 0 || s->Ho <= 0 || s->Wo <= 0 || s->Co <= 0 ||
        s->kh <= 0 || s->kw <= 0 || s->stride_h <= 0 || s->stride_w <= 0 || s->dil_h <= 0 ||
        s->dil_w <= 0 || s->pad_h < 0 || s->pad_w < 0 || s->groups <= 0 || s->deform_groups <= 0)
        return MSDA_ERR_DIMS;
    if (s->C % s->groups != 0 || s->Co % s->groups != 0 || s->C % s->deform_groups != 0)
        return MSDA_ERR_DIMS;
    const int ho = (s->H + 2 * s->pad_h - (s->dil_h * (s->kh - 1) + 1)) / s->stride_h + 1;
    const int wo = (s->W + 2 * s->pad_w - (s->dil_w * (s->kw - 1) + 1)) / s->stride_w + 1;
    if (ho != s->Ho || wo != s->Wo) return MSDA_ERR_DIMS;
    d->M = static_cast<long long>(s->N) * s->Ho * s->Wo;
    d->K = s->kh * s->kw;
    d->Cg = s->C / s->groups;
    d->Cog = s->Co / s->groups;
    d->Cd = s->C / s->deform_groups;
    d->Kd = d->K * d->Cg;
    // 32-bit item and pixel counters in the kernels
    if (d->M * s->deform_groups * d->K >= (1ll << 31) || d->M * s->C * d->K >= (1ll << 40))
        return MSDA_ERR_LIMIT;
    return MSDA_OK;
}

// 16-byte pieces need every row piece and every column piece to start on a 16-byte boundary
int piece_width(const dcn_shape* s, const Derived& d) {
    return (d.Cg % 4 == 0 && d.Cd % 4 == 0 && s->C % 4 == 0) ? 4 : 1;
}

void fill_params(const dcn_shape* s, const Derived& d, DcnParams* p) {
    p->H = s->H;
    p->W = s->W;
    p->C = s->C;
    p->Wo = s->Wo;
    p->HoWo = s->Ho * s->Wo;
    p->K = d.K;
    p->kw = s->kw;
    p->sh = s->stride_h;
    p->sw = s->stride_w;
    p->ph = s->pad_h;
    p->pw = s->pad_w;
    p->dh = s->dil_h;
    p->dw = s->dil_w;
    p->DG = s->deform_groups;
    p->Cd = d.Cd;
    p->Cg = d.Cg;
    p->G = s->groups;
    p->pieces = d.Cd / piece_width(s, d);
    int l = 0;
    while ((1 << l) < p->pieces && l < 5) ++l;
    p->lpi_log2 = l;
    p->items = static_cast<uint32_t>(d.M * s->deform_groups * d.K);
    p->fd_K = msda::make_fastdiv(d.K);
    p->fd_DG = msda::make_fastdiv(s->deform_groups);
    p->fd_HoWo = msda::make_fastdiv(p->HoWo);
    p->fd_Wo = msda::make_fastdiv(s->Wo);
    p->fd_kw = msda::make_fastdiv(s->kw);
    p->fd_Cg = msda::make_fastdiv(d.Cg);
}

template <bool BACKWARD, int VEC>
int launch_sample_vec(const DcnParams& p, int sms, cudaStream_t stream) {
    const uint32_t items_per_warp = 32u >> p.lpi_log2;
    const long long warps_needed = (static_cast<long long>(p.items) + items_per_warp - 1) / items_per_warp;
    const long long ctas_needed = (warps_needed + kThreads / 32 - 1) / (kThreads / 32);
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
        &per_sm, dcn_sample_kernel<BACKWARD, VEC>, kThreads, 0);
    if (e != cudaSuccess) return msda::note_cuda_error(e);
    if (per_sm < 1) per_sm = 1;
    const long long cap = static_cast<long long>(sms) * per_sm;
    const unsigned grid = static_cast<unsigned>(ctas_needed < cap ? ctas_needed : cap);
    dcn_sample_kernel<BACKWARD, VEC><<<grid, kThreads, 0, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return msda::note_cuda_error(e);
    msda::count_launches(1);
    return MSDA_OK;
}

template <bool BACKWARD>
int launch_sample(const DcnParams& p, int vec, int sms, cudaStream_t stream) {
    return vec == 4 ? launch_sample_vec<BACKWARD, 4>(p, sms, stream)
                    : launch_sample_vec<BACKWARD, 1>(p, sms, stream);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) % 16) == 0; }

// One product, on the tensor cores when allowed and possible.
int product(const msda::GemmArgs& g, int splits, int* status_word, cudaStream_t stream) {
    cudaError_t e;
    const int mode = g_use_tc.load(std::memory_order_relaxed);
    if (mode != 0 && msda::gemm_tc_supported(g)) {
        e = msda::gemm_tc(g, splits, mode == 2 ? 1 : 3, status_word, stream);
    } else {
        e = msda::gemm_simt(g, stream);
    }
    if (e != cudaSuccess) return msda::note_cuda_error(e);
    msda::count_launches(1);
    return MSDA_OK;
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Into how many parts to cut K for a product with few output tiles, so that the persistent
// kernel's CTAs (one per SM) all finish together: the smallest count whose work items fill
// their last round of `sms` to at least 90 %, else the count that fills it best.
int balanced_splits(long long tiles, int sms, int max_splits) {
    if (max_splits < 1) max_splits = 1;
    if (max_splits > 64) max_splits = 64;
    int best = 1;
    double best_fill = 0.0;
    for (int s = 1; s <= max_splits; ++s) {
        const long long items = tiles * s;
        const long long rounds = (items + sms - 1) / sms;
        const double fill = static_cast<double>(items) / static_cast<double>(rounds * sms);
        if (fill >= 0.9) return s;
        if (fill > best_fill) {
            best_fill = fill;
            best = s;
        }
    }
    return best;
}

// Layout of the backward's scratch memory.
struct Workspace {
    size_t grad_columns, weight_t, total;
};
Workspace plan_workspace(const dcn_shape* s, const Derived& d) {
    Workspace w;
    size_t at = 0;
    w.grad_columns = at;
    at += round_up(static_cast<size_t>(d.M) * s->groups * d.Kd * 4, 256);
    w.weight_t = at;       // per group [Kd, Cog]
    at += round_up(static_cast<size_t>(s->Co) * d.Kd * 4, 256);
    w.total = at;
    return w;
}

// The exported products: argument checks, optional K split with its zero-fill.
int public_product(const float* A, long long a_row, long long a_k, const float* B, long long b_row,
                   long long b_k, float* C, long long ldc, const float* bias, int M, int N, int K,
                   int splits, void* stream_v) {
    if (A == nullptr || B == nullptr || C == nullptr) return MSDA_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || ldc < N) return MSDA_ERR_DIMS;
    int* status_word = nullptr;
    int rc = msda::device_facts(nullptr, &status_word);
    if (rc != MSDA_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    msda::GemmArgs g{};
    g.A = A;
    g.a_row = a_row;
    g.a_k = a_k;
    g.B = B;
    g.b_row = b_row;
    g.b_k = b_k;
    g.C = C;
    g.ldc = ldc;
    g.bias = bias;
    g.M = M;
    g.N = N;
    g.K = K;
    const bool tc = g_use_tc.load(std::memory_order_relaxed) != 0 && msda::gemm_tc_supported(g);
    if (!tc) splits = 1;
    if (splits > 1) {
        if (ldc != N) return MSDA_ERR_DIMS;   // the zero-fill below covers a dense C
        const cudaError_t e = cudaMemsetAsync(C, 0, static_cast<size_t>(M) * N * 4, stream);
        if (e != cudaSuccess) return msda::note_cuda_error(e);
    }
    return product(g, splits, status_word, stream);
}

}  // namespace

extern "C" {

int dcn_sm100_use_tensor_cores(int on) {
    if (on >= 0 && on <= 2) return g_use_tc.exchange(on, std::memory_order_relaxed);
    return g_use_tc.load(std::memory_order_relaxed);
}

int gemm_nt_sm100_f32(const float* A, long long lda, const float* B, long long ldb, float* C,
                      long long ldc, const float* bias, int M, int N, int K, int splits,
                      void* stream_v) {
    if (M > 0 && N > 0 && K > 0 && (lda < K || ldb < K)) return MSDA_ERR_DIMS;
    return public_product(A, lda, 1, B, ldb, 1, C, ldc, bias, M, N, K, splits, stream_v);
}

int gemm_tn_sm100_f32(const float* A, long long lda, const float* B, long long ldb, float* C,
                      long long ldc, int M, int N, int K, int splits, void* stream_v) {
    if (M > 0 && N > 0 && K > 0 && (lda < M || ldb < N)) return MSDA_ERR_DIMS;
    return public_product(A, 1, lda, B, 1, ldb, C, ldc, nullptr, M, N, K, splits, stream_v);
}

size_t dcn_sm100_columns_bytes(const dcn_shape* s) {
    Derived d;
    if (check_shape(s, &d) != MSDA_OK) return 0;
    return static_cast<size_t>(d.M) * s->groups * d.Kd * sizeof(float);
}

size_t dcn_sm100_backward_workspace_bytes(const dcn_shape* s) {
    Derived d;
    if (check_shape(s, &d) != MSDA_OK) return 0;
    return plan_workspace(s, d).total;
}

int dcn_sm100_forward(const float* x, const float* offset, const float* mask, const float* weight,
                      const float* bias, float* out, float* columns, const dcn_shape* s,
                      void* stream_v) {
    if (x == nullptr || offset == nullptr || weight == nullptr || out == nullptr || columns == nullptr)
        return MSDA_ERR_NULL;
    Derived d;
    int rc = check_shape(s, &d);
    if (rc != MSDA_OK) return rc;
    if (reinterpret_cast<uintptr_t>(offset) % 8 != 0) return MSDA_ERR_ALIGN;
    if (piece_width(s, d) == 4 && (!aligned16(x) || !aligned16(columns))) return MSDA_ERR_ALIGN;
    int sms = 0;
    int* status_word = nullptr;
    rc = msda::device_facts(&sms, &status_word);
    if (rc != MSDA_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    DcnParams p{};
    fill_params(s, d, &p);
    p.x = x;
    p.offset = offset;
    p.mask = mask;
    p.columns = columns;
    rc = launch_sample<false>(p, piece_width(s, d), sms, stream);
    if (rc != MSDA_OK) return rc;

    const long long ld_cols = static_cast<long long>(s->groups) * d.Kd;
    bool zeroed = false;
    for (int g = 0; g < s->groups; ++g) {
        msda::GemmArgs a{};
        a.A = columns + static_cast<size_t>(g) * d.Kd;
        a.a_row = ld_cols;
        a.a_k = 1;
        a.B = weight + static_cast<size_t>(g) * d.Cog * d.Kd;
        a.b_row = d.Kd;
        a.b_k = 1;
        a.C = out + static_cast<size_t>(g) * d.Cog;
        a.ldc = s->Co;
        a.bias = bias ? bias + static_cast<size_t>(g) * d.Cog : nullptr;
        a.M = static_cast<int>(d.M);
        a.N = d.Cog;
        a.K = d.Kd;
        // few output tiles (small batches): cut K so that every SM has work
        int splits = 1;
        if (g_use_tc.load(std::memory_order_relaxed) != 0 && msda::gemm_tc_supported(a)) {
            const long long tiles = ((d.M + 127) / 128) * static_cast<long long>((d.Cog + 255) / 256);
            if (2 * tiles <= sms) splits = balanced_splits(tiles, sms, (d.Kd + 255) / 256);
            if (splits > 1 && !zeroed) {
                const cudaError_t e = cudaMemsetAsync(out, 0, static_cast<size_t>(d.M) * s->Co * 4, stream);
                if (e != cudaSuccess) return msda::note_cuda_error(e);
                zeroed = true;
            }
        }
        rc = product(a, splits, status_word, stream);
        if (rc != MSDA_OK) return rc;
    }
    return MSDA_OK;
}

int dcn_sm100_backward(const float* x, const float* offset, const float* mask,
                       const float* weight, const float* columns, const float* grad_out,
                       float* grad_x, float* grad_offset, float* grad_mask, float* grad_weight,
                       float* grad_bias, void* workspace, size_t workspace_bytes,
                       const dcn_shape* s, void* stream_v) {
    if (x == nullptr || offset == nullptr || weight == nullptr || columns == nullptr ||
        grad_out == nullptr || grad_x == nullptr || grad_offset == nullptr ||
        grad_weight == nullptr || workspace == nullptr)
        return MSDA_ERR_NULL;
    if ((mask == nullptr) != (grad_mask == nullptr)) return MSDA_ERR_NULL;
    Derived d;
    int rc = check_shape(s, &d);
    if (rc != MSDA_OK) return rc;
    const Workspace ws = plan_workspace(s, d);
    if (workspace_bytes < ws.total) return MSDA_ERR_WORKSPACE;
    if (!aligned16(workspace) || reinterpret_cast<uintptr_t>(offset) % 8 != 0 ||
        reinterpret_cast<uintptr_t>(grad_offset) % 8 != 0)
        return MSDA_ERR_ALIGN;
    if (piece_width(s, d) == 4 && (!aligned16(x) || !aligned16(grad_x) || !aligned16(columns)))
        return MSDA_ERR_ALIGN;
    int sms = 0;
    int* status_word = nullptr;
    rc = msda::device_facts(&sms, &status_word);
    if (rc != MSDA_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    char* wsp = static_cast<char*>(workspace);
    float* grad_columns = reinterpret_cast<float*>(wsp + ws.grad_columns);
    float* weight_t = reinterpret_cast<float*>(wsp + ws.weight_t);
    const long long ld_cols = static_cast<long long>(s->groups) * d.Kd;
    const int M = static_cast<int>(d.M);
    const bool tc = g_use_tc.load(std::memory_order_relaxed) != 0;

    cudaError_t e = cudaMemsetAsync(grad_x, 0, static_cast<size_t>(s->N) * s->H * s->W * s->C * 4, stream);
    if (e != cudaSuccess) return msda::note_cuda_error(e);

    // 1. grad_columns[m, g, :] = grad_out[m, g's outputs] x weight[g's outputs, :]
    for (int g = 0; g < s->groups; ++g) {
        const float* wg = weight + static_cast<size_t>(g) * d.Cog * d.Kd;
        msda::GemmArgs a{};
        a.A = grad_out + static_cast<size_t>(g) * d.Cog;
        a.a_row = s->Co;
        a.a_k = 1;
        a.C = grad_columns + static_cast<size_t>(g) * d.Kd;
        a.ldc = ld_cols;
        a.M = M;
        a.N = d.Kd;
        a.K = d.Cog;
        // B(n = kd, k = co) = weight[co, kd]; with k contiguous after a transpose
        float* wt = weight_t + static_cast<size_t>(g) * d.Cog * d.Kd;
        msda::GemmArgs probe = a;
        probe.B = wt;
        probe.b_row = d.Cog;
        probe.b_k = 1;
        if (tc && msda::gemm_tc_supported(probe)) {
            e = msda::transpose_f32(wg, d.Kd, wt, d.Cog, d.Cog, d.Kd, stream);
            if (e != cudaSuccess) return msda::note_cuda_error(e);
            msda::count_launches(1);
            a = probe;
        } else {
            a.B = wg;
            a.b_row = 1;
            a.b_k = d.Kd;
        }
        rc = product(a, 1, status_word, stream);
        if (rc != MSDA_OK) return rc;
    }

    // 2. scatter: grad_x, grad_offset, grad_mask
    DcnParams p{};
    fill_params(s, d, &p);
    p.x = x;
    p.offset = offset;
    p.mask = mask;
    p.columns = grad_columns;
    p.grad_x = grad_x;
    p.grad_offset = grad_offset;
    p.grad_mask = grad_mask;
    rc = launch_sample<true>(p, piece_width(s, d), sms, stream);
    if (rc != MSDA_OK) return rc;

    // 3. grad_weight[co, kd] = sum over m of grad_out[m, co] * columns[m, g, kd]: both operands
    //    are stored pixel row by pixel row, i.e. with the row index (co, kd) contiguous and
    //    k = m strided. The tensor-core kernel takes that form directly (K cut over CTAs so
    //    that every SM has work); operands that miss its alignment rules go to the FMA kernel.
    {
        bool zeroed = false;
        for (int g = 0; g < s->groups; ++g) {
            msda::GemmArgs a{};
            a.A = grad_out + static_cast<size_t>(g) * d.Cog;
            a.a_row = 1;
            a.a_k = s->Co;
            a.B = columns + static_cast<size_t>(g) * d.Kd;
            a.b_row = 1;
            a.b_k = ld_cols;
            a.C = grad_weight + static_cast<size_t>(g) * d.Cog * d.Kd;
            a.ldc = d.Kd;
            a.M = d.Cog;
            a.N = d.Kd;
            a.K = M;
            int splits = 1;
            if (tc && msda::gemm_tc_supported(a)) {
                const long long tiles = ((d.Cog + 127) / 128) * static_cast<long long>((d.Kd + 255) / 256);
                splits = balanced_splits(tiles, sms, (M + 1023) / 1024);
                if (splits > 1 && !zeroed) {
                    e = cudaMemsetAsync(grad_weight, 0, static_cast<size_t>(s->Co) * d.Kd * 4, stream);
                    if (e != cudaSuccess) return msda::note_cuda_error(e);
                    zeroed = true;
                }
            }
            rc = product(a, splits, status_word, stream);
            if (rc != MSDA_OK) return rc;
        }
    }

    // 4. grad_bias
    if (grad_bias != nullptr) {
        e = cudaMemsetAsync(grad_bias, 0, static_cast<size_t>(s->Co) * 4, stream);
        if (e != cudaSuccess) return msda::note_cuda_error(e);
        const int rows_per_block = 256;
        const dim3 grid((M + rows_per_block - 1) / rows_per_block, (s->Co + kThreads - 1) / kThreads);
        column_sum_kernel<<<grid, kThreads, 0, stream>>>(grad_out, M, s->Co, rows_per_block, grad_bias);
        e = cudaGetLastError();
        if (e != cudaSuccess) return msda::note_cuda_error(e);
        msda::count_launches(1);
    }
    return MSDA_OK;
}

}  // extern "C"

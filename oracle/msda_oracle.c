/* CPU oracle for multi-scale deformable attention (MSDA), forward and backward.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product path may call this file;
 * it exists so that tests, the smoke check and the benchmark's CPU-baseline
 * leg can check the CUDA kernels against an independent statement of the
 * reference's algorithm.
 *
 * It restates, in double precision and plain loops, what the reference defines:
 *   - the CPU golden of the reference's unit test: per level, bilinear
 *     grid_sample(align_corners=False, padding_mode="zeros") at 2*loc-1, i.e.
 *     pixel coordinate loc*size - 0.5, weighted by the attention weights and
 *     summed over levels and points
 *     (tests/torch/test_multi_scale_deformable_attn.py:34-64), gradients by
 *     differentiating that expression (:67-76);
 *   - the device kernel's explicit rules, which agree with the golden: a sample
 *     counts only if x > -1, y > -1, x < W, y < H
 *     (kernels/multi_scale_deformable_attn/op_kernel/msda.h:367-390); corner
 *     existence and weights
 *     (op_kernel/arch35/multi_scale_deformable_attn.cpp:59-78); gradient
 *     algebra (op_kernel/arch35/multi_scale_deformable_attn_grad.cpp:105-142,
 *     op_kernel/multi_scale_deformable_attn_grad.cpp:215-242).
 * Parity is pinned: tests/golden/ holds outputs of the reference's own golden
 * functions on seeded inputs, and tests/test_oracle.py checks this file
 * against them.
 *
 * Layouts: value [B,K,H,D]; shapes [L,2] (H,W); starts [L];
 * loc [B,Q,H,L,P,2] (x,y); attn [B,Q,H,L,P]; out/grad_out [B,Q,H*D].
 * Inputs are float (already rounded to the dtype under test); results double.
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <string.h>

/* ---- a minimal parallel-for over [0, n) with POSIX threads ---------------- */
static int g_threads = 1;
void msda_oracle_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
int msda_oracle_get_threads(void) { return g_threads; }

typedef void (*range_fn)(long begin, long end, void* ctx);
typedef struct {
    range_fn fn;
    void* ctx;
    long begin, end;
} job_t;
static void* job_main(void* arg) {
    job_t* j = (job_t*)arg;
    j->fn(j->begin, j->end, j->ctx);
    return NULL;
}
static void parallel_for(long n, range_fn fn, void* ctx) {
    int nt = g_threads;
    if (nt > n) nt = (int)(n > 0 ? n : 1);
    if (nt <= 1) {
        fn(0, n, ctx);
        return;
    }
    pthread_t th[256];
    job_t jobs[256];
    for (int i = 0; i < nt; ++i) {
        jobs[i].fn = fn;
        jobs[i].ctx = ctx;
        jobs[i].begin = n * i / nt;
        jobs[i].end = n * (i + 1) / nt;
        if (pthread_create(&th[i], NULL, job_main, &jobs[i]) != 0) {
            /* could not start a thread: run this share inline */
            fn(jobs[i].begin, jobs[i].end, ctx);
            th[i] = 0;
            jobs[i].fn = NULL;
        }
    }
    for (int i = 0; i < nt; ++i)
        if (jobs[i].fn) pthread_join(th[i], NULL);
}

typedef struct {
    const float *value, *loc, *attn, *grad_out;
    const int *shapes, *starts;
    double *out, *grad_value, *grad_loc, *grad_attn;
    int B, K, H, D, L, Q, P;
} args_t;

typedef struct {
    int ok[4];      /* corner exists */
    size_t row[4];  /* pixel index y*W + x inside the level */
    double w[4];    /* bilinear weight (no attention factor) */
    double lw, lh;
    int valid;
} corners_t;

static void corners(double lx, double ly, int Hl, int Wl, corners_t* c) {
    const double x = lx * (double)Wl - 0.5;
    const double y = ly * (double)Hl - 0.5;
    memset(c, 0, sizeof(*c));
    /* written so that NaN compares false, as in the reference */
    c->valid = (x > -1.0) && (y > -1.0) && (x < (double)Wl) && (y < (double)Hl);
    if (!c->valid) return;
    const double x0f = floor(x), y0f = floor(y);
    const long x0 = (long)x0f, y0 = (long)y0f, x1 = x0 + 1, y1 = y0 + 1;
    const double lw = x - x0f, lh = y - y0f, hw = 1.0 - lw, hh = 1.0 - lh;
    c->lw = lw;
    c->lh = lh;
    c->w[0] = hh * hw; c->w[1] = hh * lw; c->w[2] = lh * hw; c->w[3] = lh * lw;
    c->ok[0] = (y0 >= 0 && x0 >= 0);
    c->ok[1] = (y0 >= 0 && x1 <= Wl - 1);
    c->ok[2] = (y1 <= Hl - 1 && x0 >= 0);
    c->ok[3] = (y1 <= Hl - 1 && x1 <= Wl - 1);
    if (c->ok[0]) c->row[0] = (size_t)(y0 * Wl + x0);
    if (c->ok[1]) c->row[1] = (size_t)(y0 * Wl + x1);
    if (c->ok[2]) c->row[2] = (size_t)(y1 * Wl + x0);
    if (c->ok[3]) c->row[3] = (size_t)(y1 * Wl + x1);
}

static void forward_range(long begin, long end, void* ctx) {
    const args_t* A = (const args_t*)ctx;
    const float *value = A->value, *loc = A->loc, *attn = A->attn;
    const int *shapes = A->shapes, *starts = A->starts;
    double* out = A->out;
    const int K = A->K, H = A->H, D = A->D, L = A->L, Q = A->Q, P = A->P;
    for (long t = begin; t < end; ++t) {
        const int h = (int)(t % H);
        const int b = (int)(t / ((long)Q * H));
        double* o = out + (size_t)t * D;
        for (int d = 0; d < D; ++d) o[d] = 0.0;
        for (int l = 0; l < L; ++l) {
            const int Hl = shapes[2 * l], Wl = shapes[2 * l + 1];
            for (int p = 0; p < P; ++p) {
                const size_t si = ((size_t)t * L + l) * P + p;
                corners_t c;
                corners((double)loc[2 * si], (double)loc[2 * si + 1], Hl, Wl, &c);
                if (!c.valid) continue;
                const double a = (double)attn[si];
                for (int k = 0; k < 4; ++k) {
                    if (!c.ok[k]) continue;
                    const float* v =
                        value + (((size_t)b * K + starts[l] + c.row[k]) * H + h) * (size_t)D;
                    const double w = c.w[k] * a;
                    for (int d = 0; d < D; ++d) o[d] += w * (double)v[d];
                }
            }
        }
    }
}

void msda_oracle_forward(const float* value, const int* shapes, const int* starts,
                         const float* loc, const float* attn, double* out, int B, int K, int H,
                         int D, int L, int Q, int P) {
    args_t A;
    memset(&A, 0, sizeof(A));
    A.value = value; A.shapes = shapes; A.starts = starts; A.loc = loc; A.attn = attn;
    A.out = out;
    A.B = B; A.K = K; A.H = H; A.D = D; A.L = L; A.Q = Q; A.P = P;
    parallel_for((long)B * Q * H, forward_range, &A);
}

/* one (batch, head) pair owns a disjoint set of grad_value rows, so pairs can
 * run on different threads without atomics */
static void backward_range(long begin, long end, void* ctx) {
    const args_t* A = (const args_t*)ctx;
    const float *value = A->value, *loc = A->loc, *attn = A->attn, *grad_out = A->grad_out;
    const int *shapes = A->shapes, *starts = A->starts;
    double *grad_value = A->grad_value, *grad_loc = A->grad_loc, *grad_attn = A->grad_attn;
    const int K = A->K, H = A->H, D = A->D, L = A->L, Q = A->Q, P = A->P;
    for (long bh = begin; bh < end; ++bh) {
        const int b = (int)(bh / H), h = (int)(bh % H);
        for (int q = 0; q < Q; ++q) {
            const size_t t = ((size_t)b * Q + q) * H + h;
            const float* go = grad_out + t * D;
            for (int l = 0; l < L; ++l) {
                const int Hl = shapes[2 * l], Wl = shapes[2 * l + 1];
                for (int p = 0; p < P; ++p) {
                    const size_t si = (t * L + l) * P + p;
                    corners_t c;
                    corners((double)loc[2 * si], (double)loc[2 * si + 1], Hl, Wl, &c);
                    double ga = 0.0, gx = 0.0, gy = 0.0;
                    if (c.valid) {
                        const double a = (double)attn[si];
                        double S[4] = {0.0, 0.0, 0.0, 0.0};
                        for (int k = 0; k < 4; ++k) {
                            if (!c.ok[k]) continue;
                            const size_t off =
                                (((size_t)b * K + starts[l] + c.row[k]) * H + h) * (size_t)D;
                            const float* v = value + off;
                            double* gv = grad_value + off;
                            const double w = c.w[k] * a;
                            double s = 0.0;
                            for (int d = 0; d < D; ++d) {
                                gv[d] += w * (double)go[d];
                                s += (double)v[d] * (double)go[d];
                            }
                            S[k] = s;
                        }
                        const double hw = 1.0 - c.lw, hh = 1.0 - c.lh;
                        ga = c.w[0] * S[0] + c.w[1] * S[1] + c.w[2] * S[2] + c.w[3] * S[3];
                        gx = (double)Wl * a * (hh * (S[1] - S[0]) + c.lh * (S[3] - S[2]));
                        gy = (double)Hl * a * (hw * (S[2] - S[0]) + c.lw * (S[3] - S[1]));
                    }
                    grad_attn[si] = ga;
                    grad_loc[2 * si] = gx;
                    grad_loc[2 * si + 1] = gy;
                }
            }
        }
    }
}

void msda_oracle_backward(const float* value, const int* shapes, const int* starts,
                          const float* loc, const float* attn, const float* grad_out,
                          double* grad_value, double* grad_loc, double* grad_attn, int B, int K,
                          int H, int D, int L, int Q, int P) {
    const size_t nval = (size_t)B * K * H * D;
    for (size_t i = 0; i < nval; ++i) grad_value[i] = 0.0;
    args_t A;
    memset(&A, 0, sizeof(A));
    A.value = value; A.shapes = shapes; A.starts = starts; A.loc = loc; A.attn = attn;
    A.grad_out = grad_out;
    A.grad_value = grad_value; A.grad_loc = grad_loc; A.grad_attn = grad_attn;
    A.B = B; A.K = K; A.H = H; A.D = D; A.L = L; A.Q = Q; A.P = P;
    parallel_for((long)B * H, backward_range, &A);
}

/* Distance of every sample's pixel coordinates from the nearest cell boundary
 * (an integer), min over x and y. grad_loc is discontinuous there (the two
 * one-sided derivatives differ), so parity checks skip samples that sit within
 * float rounding of a boundary. */
void msda_oracle_kink_distance(const int* shapes, const float* loc, double* dist, int B, int H,
                               int L, int Q, int P) {
    const long ntask = (long)B * Q * H;
    for (long t = 0; t < ntask; ++t)
        for (int l = 0; l < L; ++l)
            for (int p = 0; p < P; ++p) {
                const size_t si = ((size_t)t * L + l) * P + p;
                const double x = (double)loc[2 * si] * shapes[2 * l + 1] - 0.5;
                const double y = (double)loc[2 * si + 1] * shapes[2 * l] - 0.5;
                const double dx = fabs(x - nearbyint(x)), dy = fabs(y - nearbyint(y));
                dist[si] = (dx < dy) ? dx : dy;
                if (!(dist[si] == dist[si])) dist[si] = 0.0; /* NaN: treat as on a kink */
            }
}

/* ---- geometric kernel attention (nearest-pixel sibling of MSDA) -----------------------
 * Restates the reference's CPU golden (tests/torch/test_geometric_kernel_attention.py:44-103):
 * sampling locations are integer pixel coordinates (x, y), clamped into [0, W-1] x [0, H-1]
 * of their level (the golden converts them with .long(), i.e. truncation, first);
 *   out[b,q,h,:]      = sum_{l,p} attn * value[b, start_l + y*W_l + x, h, :]
 *   grad_value[row,:] += attn * grad_out[b,q,h,:]
 *   grad_attn         = <value[row,:], grad_out[b,q,h,:]>.
 * Pinned by tests/golden/gka_golden.npz (outputs of that golden). */
static size_t gka_row(const float* loc, size_t si, int Hl, int Wl) {
    long x = (long)loc[2 * si], y = (long)loc[2 * si + 1];
    if (x < 0) x = 0;
    if (x > Wl - 1) x = Wl - 1;
    if (y < 0) y = 0;
    if (y > Hl - 1) y = Hl - 1;
    return (size_t)(y * Wl + x);
}

void gka_oracle_forward(const float* value, const int* shapes, const int* starts,
                        const float* loc, const float* attn, double* out, int B, int K, int H,
                        int D, int L, int Q, int P) {
    const long ntask = (long)B * Q * H;
    for (long t = 0; t < ntask; ++t) {
        const int h = (int)(t % H);
        const int b = (int)(t / ((long)Q * H));
        double* o = out + (size_t)t * D;
        for (int d = 0; d < D; ++d) o[d] = 0.0;
        for (int l = 0; l < L; ++l)
            for (int p = 0; p < P; ++p) {
                const size_t si = ((size_t)t * L + l) * P + p;
                const size_t row = gka_row(loc, si, shapes[2 * l], shapes[2 * l + 1]);
                const float* v = value + (((size_t)b * K + starts[l] + row) * H + h) * (size_t)D;
                const double a = (double)attn[si];
                for (int d = 0; d < D; ++d) o[d] += a * (double)v[d];
            }
    }
}

void gka_oracle_backward(const float* value, const int* shapes, const int* starts,
                         const float* loc, const float* attn, const float* grad_out,
                         double* grad_value, double* grad_attn, int B, int K, int H, int D, int L,
                         int Q, int P) {
    const size_t nval = (size_t)B * K * H * D;
    for (size_t i = 0; i < nval; ++i) grad_value[i] = 0.0;
    const long ntask = (long)B * Q * H;
    for (long t = 0; t < ntask; ++t) {
        const int h = (int)(t % H);
        const int b = (int)(t / ((long)Q * H));
        const float* go = grad_out + (size_t)t * D;
        for (int l = 0; l < L; ++l)
            for (int p = 0; p < P; ++p) {
                const size_t si = ((size_t)t * L + l) * P + p;
                const size_t row = gka_row(loc, si, shapes[2 * l], shapes[2 * l + 1]);
                const size_t off = (((size_t)b * K + starts[l] + row) * H + h) * (size_t)D;
                const double a = (double)attn[si];
                double s = 0.0;
                for (int d = 0; d < D; ++d) {
                    grad_value[off + d] += a * (double)go[d];
                    s += (double)value[off + d] * (double)go[d];
                }
                grad_attn[si] = s;
            }
    }
}

/* ---- deformable aggregation ------------------------------------------------------------
 * Restates the reference's numpy golden of the forward
 * (tests/torch/test_deformable_aggregation.py:33-125): for every (batch, anchor, point, cam,
 * scale) a sample at loc = (w, h), skipped unless 0 < w < 1 and 0 < h < 1; pixel
 * coordinates loc * size - 0.5; bilinear corners that fall outside the map read as zero; the
 * interpolated C-vector is multiplied group-wise by weights[..., group] and summed into
 * out[b, anchor, :]. The backward is the derivative of that expression (the reference has no
 * CPU golden for it): grad_feat scatter, grad_weights[..., g] = <interpolated group g,
 * grad_out group g>, grad_loc from the bilinear slopes, summed over scales and channels.
 * Forward pinned by tests/golden/da_golden.npz (outputs of the reference golden); backward
 * cross-checked against autograd of an independent PyTorch restatement in the tests.
 * feat [B,F,C]; shapes [cams,scales,2] (h,w); starts [cams,scales]; loc [B,A,Pts,cams,2]
 * (w,h); wts [B,A,Pts,cams,scales,G]. */
static void da_sample(const float* feat, const int* shapes, const int* starts, const float* loc,
                      const float* wts, const float* grad_out, double* out, double* grad_feat,
                      double* grad_loc, double* grad_wts, int b, int a, int pt, int cam, int sc,
                      int F, int C, int A, int Pts, int cams, int scales, int G) {
    const size_t pc = (((size_t)b * A + a) * Pts + pt) * cams + cam;
    const size_t wi = (pc * scales + sc) * G;
    const double lw_n = (double)loc[2 * pc], lh_n = (double)loc[2 * pc + 1];
    const int cpg = C / G;
    if (grad_wts)
        for (int g = 0; g < G; ++g) grad_wts[wi + g] = 0.0;
    if (!(lw_n > 0.0 && lw_n < 1.0 && lh_n > 0.0 && lh_n < 1.0)) return;
    const int map = cam * scales + sc;
    const int Hm = shapes[2 * map], Wm = shapes[2 * map + 1];
    corners_t c;
    corners(lw_n, lh_n, Hm, Wm, &c);
    if (!c.valid) return;
    const float* rows[4] = {0, 0, 0, 0};
    double* grows[4] = {0, 0, 0, 0};
    for (int k = 0; k < 4; ++k)
        if (c.ok[k]) {
            const size_t off = ((size_t)b * F + starts[map] + c.row[k]) * (size_t)C;
            rows[k] = feat + off;
            if (grad_feat) grows[k] = grad_feat + off;
        }
    const double hw = 1.0 - c.lw, hh = 1.0 - c.lh;
    double gx = 0.0, gy = 0.0;
    for (int ch = 0; ch < C; ++ch) {
        const int g = ch / cpg;
        const double wt = (double)wts[wi + g];
        double v[4];
        for (int k = 0; k < 4; ++k) v[k] = rows[k] ? (double)rows[k][ch] : 0.0;
        const double val = c.w[0] * v[0] + c.w[1] * v[1] + c.w[2] * v[2] + c.w[3] * v[3];
        if (out) out[((size_t)b * A + a) * C + ch] += val * wt;
        if (grad_out) {
            const double go = (double)grad_out[((size_t)b * A + a) * C + ch];
            for (int k = 0; k < 4; ++k)
                if (grows[k]) grows[k][ch] += c.w[k] * wt * go;
            grad_wts[wi + g] += val * go;
            gx += go * wt * (double)Wm * (hh * (v[1] - v[0]) + c.lh * (v[3] - v[2]));
            gy += go * wt * (double)Hm * (hw * (v[2] - v[0]) + c.lw * (v[3] - v[1]));
        }
    }
    if (grad_loc) {
        grad_loc[2 * pc] += gx;
        grad_loc[2 * pc + 1] += gy;
    }
}

void da_oracle_forward(const float* feat, const int* shapes, const int* starts, const float* loc,
                       const float* wts, double* out, int B, int F, int C, int A, int Pts,
                       int cams, int scales, int G) {
    for (size_t i = 0; i < (size_t)B * A * C; ++i) out[i] = 0.0;
    for (int b = 0; b < B; ++b)
        for (int a = 0; a < A; ++a)
            for (int pt = 0; pt < Pts; ++pt)
                for (int cam = 0; cam < cams; ++cam)
                    for (int sc = 0; sc < scales; ++sc)
                        da_sample(feat, shapes, starts, loc, wts, 0, out, 0, 0, 0, b, a, pt, cam,
                                  sc, F, C, A, Pts, cams, scales, G);
}

void da_oracle_backward(const float* feat, const int* shapes, const int* starts,
                        const float* loc, const float* wts, const float* grad_out,
                        double* grad_feat, double* grad_loc, double* grad_wts, int B, int F,
                        int C, int A, int Pts, int cams, int scales, int G) {
    for (size_t i = 0; i < (size_t)B * F * C; ++i) grad_feat[i] = 0.0;
    for (size_t i = 0; i < (size_t)B * A * Pts * cams * 2; ++i) grad_loc[i] = 0.0;
    for (int b = 0; b < B; ++b)
        for (int a = 0; a < A; ++a)
            for (int pt = 0; pt < Pts; ++pt)
                for (int cam = 0; cam < cams; ++cam)
                    for (int sc = 0; sc < scales; ++sc)
                        da_sample(feat, shapes, starts, loc, wts, grad_out, 0, grad_feat,
                                  grad_loc, grad_wts, b, a, pt, cam, sc, F, C, A, Pts, cams,
                                  scales, G);
}

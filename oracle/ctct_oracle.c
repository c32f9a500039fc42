/*
 * CPU oracle for the CTC-Transducer loss -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the reference project's algorithm (maxwellzh/warp-ctct):
 * ref_ctct.py for the lattice recursions and gathers, csrc/gather.cu:311-374 for
 * the occupancy gradient, warp_ctct/__init__.py for the dense scatter that autograd
 * performs, csrc/simple.cu:20-26 and csrc/binding.cpp:198-219,251-253 for the
 * log-add joiner.  Only the test-suite, the smoke check and the benchmark's CPU
 * baseline may call into this library; the product never does.
 *
 * Parity pin: tests/test_oracle.py compares these functions with tables, costs and
 * autograd gradients produced by the reference's ref_ctct.py (the .npz files under tests/golden/).
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -shared).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define REAL float
#define SUF(n) CAT(n, _f32)
#define EXP expf
#define LOG logf
#define LOG1P log1pf
#include "ctct_oracle_impl.inc"
#undef REAL
#undef SUF
#undef EXP
#undef LOG
#undef LOG1P

#define REAL double
#define SUF(n) CAT(n, _f64)
#define EXP exp
#define LOG log
#define LOG1P log1p
#include "ctct_oracle_impl.inc"
#undef REAL
#undef SUF
#undef EXP
#undef LOG
#undef LOG1P

static void set_threads(int nthreads) {
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#else
    (void)nthreads;
#endif
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Vocabulary index the reference gathers for (context u, slot k): an index tensor
 * filled with 0, [:,1:,1] = labels, [:,:U,2] = labels (warp_ctct/__init__.py:124-127,
 * ref_ctct.py:223-230).  ys is one utterance's padded label row of length U1-1. */
static inline int slot_index(const int *ys, int U1, int u, int k) {
    if (k == 1 && u >= 1) return ys[u - 1];
    if (k == 2 && u < U1 - 1) return ys[u];
    return 0;
}

/* collect_units, ref_ctct.py:223-230: (N,T,U1,V) -> (N,T,U1,3), pure copy. */
int oracle_collect_units(const float *lp, const int *ys, int N, int T, int U1, int V, float *out,
                         int nthreads) {
    set_threads(nthreads);
    const long rows = (long)N * T * U1;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r) {
        const int u = (int)(r % U1);
        const int n = (int)(r / ((long)T * U1));
        const int *y = ys + (size_t)n * (U1 - 1);
        const float *src = lp + (size_t)r * V;
        for (int k = 0; k < 3; ++k) out[(size_t)r * 3 + k] = src[slot_index(y, U1, u, k)];
    }
    return 0;
}

/* One utterance's table in one of the four layouts of ref_ctct.py.
 * which: 0 fw_simple, 1 bw_simple ((T+1) x (2U+1)); 2 fw_shift, 3 bw_shift ((T-U+1) x (2U+1)).
 * Returns the log-likelihood through *ll. */
int oracle_table_f32(const float *g3, int su, const int *ys, int T, int U, int which, float *table,
                     float *ll) {
    if (T < U || U < 1) return -1;
    switch (which) {
    case 0: *ll = fw_simple_f32(g3, su, ys, T, U, table); break;
    case 1: *ll = bw_simple_f32(g3, su, ys, T, U, table); break;
    case 2: *ll = fw_shift_f32(g3, su, ys, T, U, table); break;
    case 3: *ll = bw_shift_f32(g3, su, ys, T, U, table); break;
    default: return -2;
    }
    return 0;
}

int oracle_table_f64(const float *g3, int su, const int *ys, int T, int U, int which, double *table,
                     double *ll) {
    if (T < U || U < 1) return -1;
    switch (which) {
    case 0: *ll = fw_simple_f64(g3, su, ys, T, U, table); break;
    case 1: *ll = bw_simple_f64(g3, su, ys, T, U, table); break;
    case 2: *ll = fw_shift_f64(g3, su, ys, T, U, table); break;
    case 3: *ll = bw_shift_f64(g3, su, ys, T, U, table); break;
    default: return -2;
    }
    return 0;
}

/* Batch forward of the reference's extension entry point ctct_loss_fwd
 * (csrc/binding.cpp:31-100): costs[n] = -betas[n,0,0]; when want_grad, grads =
 * occupancy gradient w.r.t. the gathered log-probs, zeros outside t<lx, u<=ly.
 * Where the reference leaves the result undefined: an utterance with lx < ly has no alignment
 * (cost +inf, zero gradient); one without labels (ly == 0) has exactly one, all blanks at
 * context 0 (cost = minus the sum of those log-probs, gradient -1 on each of them; its table
 * in ref_ctct.py:6-36 never sets the cell it reads the likelihood from). */
#define DEFINE_CTCT_FWD(REAL, SFX)                                                               \
    int oracle_ctct_fwd_##SFX(const float *g3, const int *ys, const int *lx, const int *ly,      \
                              int N, int T, int U1, int want_grad, REAL *costs, REAL *grads,     \
                              int nthreads) {                                                    \
        set_threads(nthreads);                                                                   \
        int bad = 0;                                                                             \
        if (want_grad) memset(grads, 0, sizeof(REAL) * (size_t)N * T * U1 * 3);                  \
        _Pragma("omp parallel for schedule(dynamic)") for (int n = 0; n < N; ++n) {              \
            const int Tn = lx[n], Un = ly[n];                                                    \
            if (Un == 0 && Tn >= 0 && Tn <= T) {                                                 \
                REAL s = 0;                                                                      \
                for (int t = 0; t < Tn; ++t) s += (REAL)g3[(((size_t)n * T + t) * U1) * 3];      \
                costs[n] = -s;                                                                   \
                if (want_grad && isfinite((double)s))                                            \
                    for (int t = 0; t < Tn; ++t) grads[(((size_t)n * T + t) * U1) * 3] = (REAL)-1; \
                continue;                                                                        \
            }                                                                                    \
            if (Tn > T || Un > U1 - 1 || Tn < Un || Un < 1) {                                    \
                costs[n] = INFINITY;                                                             \
                continue;                                                                        \
            }                                                                                    \
            const size_t cells = (size_t)(Tn - Un + 1) * (2 * Un + 1);                           \
            REAL *B = (REAL *)malloc(sizeof(REAL) * cells);                                      \
            REAL *A = want_grad ? (REAL *)malloc(sizeof(REAL) * cells) : NULL;                   \
            if (!B || (want_grad && !A)) {                                                       \
                bad = 1;                                                                         \
                free(A);                                                                         \
                free(B);                                                                         \
                continue;                                                                        \
            }                                                                                    \
            const float *g = g3 + (size_t)n * T * U1 * 3;                                        \
            const int *y = ys + (size_t)n * (U1 - 1);                                            \
            costs[n] = -bw_shift_##SFX(g, U1, y, Tn, Un, B);                                     \
            if (want_grad) {                                                                     \
                fw_shift_##SFX(g, U1, y, Tn, Un, A);                                             \
                fill_grad_##SFX(g, U1, y, Tn, Un, A, B, grads + (size_t)n * T * U1 * 3);         \
            }                                                                                    \
            free(A);                                                                             \
            free(B);                                                                             \
        }                                                                                        \
        return bad ? -3 : 0;                                                                     \
    }
DEFINE_CTCT_FWD(float, f32)
DEFINE_CTCT_FWD(double, f64)

/* What autograd does after CTCTLoss.backward (warp_ctct/__init__.py:31-33, and the
 * backward of the gather at :131): dense[n,t,u,:] = 0, then for each slot k add
 * grad_out[n] * grads[n,t,u,k] at the slot's vocabulary index; slots that share
 * an index add up.  half_round != 0 reproduces fp16 inputs: every scaled value is
 * rounded to fp16 before the scatter and sums are rounded to fp16 again. */
static float to_half_and_back(float x) {
    /* round-to-nearest-even float -> IEEE binary16 -> float, in integer arithmetic */
    uint32_t b;
    memcpy(&b, &x, 4);
    uint32_t sign = b & 0x80000000u;
    uint32_t a = b & 0x7fffffffu;
    float r;
    if (a >= 0x7f800000u) return x;          /* inf / nan */
    if (a >= 0x477ff000u) {                  /* rounds to >= 65520 -> inf */
        uint32_t inf = sign | 0x7f800000u;
        memcpy(&r, &inf, 4);
        return r;
    }
    if (a < 0x38800000u) {                   /* subnormal half: quantum 2^-24 */
        float ax = fabsf(x);
        float q = ax * 16777216.0f;          /* exact scaling */
        q = nearbyintf(q);                   /* ties-to-even in default mode */
        r = q / 16777216.0f;
        return sign ? -r : r;
    }
    uint32_t lsb = (a >> 13) & 1u;
    a += 0xfffu + lsb;
    a &= ~0x1fffu;
    a |= sign;
    memcpy(&r, &a, 4);
    return r;
}

float oracle_round_half(float x) { return to_half_and_back(x); }

int oracle_scatter_dense(const float *grads3, const int *ys, const float *grad_out, int N, int T,
                         int U1, int V, int half_round, float *dense, int nthreads) {
    set_threads(nthreads);
    const long rows = (long)N * T * U1;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r) {
        const int u = (int)(r % U1);
        const int n = (int)(r / ((long)T * U1));
        const int *y = ys + (size_t)n * (U1 - 1);
        float *dst = dense + (size_t)r * V;
        memset(dst, 0, sizeof(float) * (size_t)V);
        for (int k = 0; k < 3; ++k) {
            float v = grad_out[n] * grads3[(size_t)r * 3 + k];
            const int idx = slot_index(y, U1, u, k);
            if (half_round) {
                v = to_half_and_back(v);
                dst[idx] = to_half_and_back(dst[idx] + v);
            } else {
                dst[idx] += v;
            }
        }
    }
    return 0;
}

/* Whole hot path on host memory, as the benchmark's CPU baseline runs it:
 * gather -> beta/alpha tables -> occupancy gradient -> dense scatter. */
int oracle_ctct_loss_f32(const float *lp, const int *ys, const int *lx, const int *ly, int N,
                         int T, int U1, int V, const float *grad_out, float *costs, float *dense,
                         int nthreads) {
    const size_t n3 = (size_t)N * T * U1 * 3;
    float *g3 = (float *)malloc(sizeof(float) * n3);
    float *gr = (float *)malloc(sizeof(float) * n3);
    if (!g3 || !gr) {
        free(g3);
        free(gr);
        return -3;
    }
    int rc = oracle_collect_units(lp, ys, N, T, U1, V, g3, nthreads);
    if (!rc) rc = oracle_ctct_fwd_f32(g3, ys, lx, ly, N, T, U1, dense != NULL, costs, gr, nthreads);
    if (!rc && dense) rc = oracle_scatter_dense(gr, ys, grad_out, N, T, U1, V, 0, dense, nthreads);
    free(g3);
    free(gr);
    return rc;
}

/* ------------------------------------------------------------------------- *
 * log-add joiner ("simple" loss)
 * ------------------------------------------------------------------------- */

/* den[b,i,j] = log sum_k exp(f[b,i,k] + g[b,j,k]); f (B,M,K), g (B,Nc,K) contiguous.
 * This is log_matmul(f, g^T) of warp_ctct/__init__.py:195-200 / csrc/logmatmul.cu:44-146. */
#define DEFINE_LOGMM(REAL, SFX)                                                                  \
    int oracle_log_matmul_##SFX(const float *f, const float *g, int B, int M, int Nc, int K,     \
                                REAL *out, int nthreads) {                                       \
        set_threads(nthreads);                                                                   \
        const long cells = (long)B * M * Nc;                                                     \
        _Pragma("omp parallel for schedule(static)") for (long c = 0; c < cells; ++c) {          \
            const int j = (int)(c % Nc);                                                         \
            const int i = (int)((c / Nc) % M);                                                   \
            const int b = (int)(c / ((long)Nc * M));                                             \
            out[c] = logdot_##SFX(f + ((size_t)b * M + i) * K, g + ((size_t)b * Nc + j) * K, 1, K); \
        }                                                                                        \
        return 0;                                                                                \
    }
DEFINE_LOGMM(float, f32)
DEFINE_LOGMM(double, f64)

/* collect_separate, ref_ctct.py:206-220 (warp_ctct/__init__.py:204-215):
 * f (N,T,V) -> cf (N,T,U1) [col 0 = blank, col k = ys[k-1]];  g (N,U1,V) -> cg (N,U1,3). */
int oracle_collect_separate(const float *f, const float *g, const int *ys, int N, int T, int U1,
                            int V, float *cf, float *cg) {
    for (int n = 0; n < N; ++n) {
        const int *y = ys + (size_t)n * (U1 - 1);
        for (int t = 0; t < T; ++t)
            for (int u = 0; u < U1; ++u)
                cf[((size_t)n * T + t) * U1 + u] = f[((size_t)n * T + t) * V + (u == 0 ? 0 : y[u - 1])];
        for (int u = 0; u < U1; ++u)
            for (int k = 0; k < 3; ++k)
                cg[((size_t)n * U1 + u) * 3 + k] = g[((size_t)n * U1 + u) * V + slot_index(y, U1, u, k)];
    }
    return 0;
}

/* The log-prob the simple kernels compose on the fly, csrc/simple.cu:20-26 (with den)
 * and csrc/simple_unnorm.cu:20-25 (den == NULL):
 *   slot 0: f[n,t,0]   + g[n,u,0] - den[n,t,u]
 *   slot 1: f[n,t,u]   + g[n,u,1] - den[n,t,u]
 *   slot 2: f[n,t,u+1] + g[n,u,2] - den[n,t,u]
 * The (u=0, slot 1) and (u=U1-1, slot 2) entries are never read by the lattice; they are
 * composed from column 0 of cf so that the tensor is fully defined. */
int oracle_compose_simple(const float *cf, const float *cg, const float *den, int N, int T, int U1,
                          float *g3) {
    for (int n = 0; n < N; ++n)
        for (int t = 0; t < T; ++t)
            for (int u = 0; u < U1; ++u) {
                const size_t r = ((size_t)n * T + t) * U1 + u;
                const float *frow = cf + ((size_t)n * T + t) * U1;
                const float *gk = cg + ((size_t)n * U1 + u) * 3;
                const float d = den ? den[r] : 0.0f;
                const float f1 = frow[u];
                const float f2 = u + 1 < U1 ? frow[u + 1] : frow[0];
                if (den) {
                    g3[r * 3 + 0] = frow[0] + gk[0] - d;
                    g3[r * 3 + 1] = f1 + gk[1] - d;
                    g3[r * 3 + 2] = f2 + gk[2] - d;
                } else {
                    g3[r * 3 + 0] = frow[0] + gk[0];
                    g3[r * 3 + 1] = f1 + gk[1];
                    g3[r * 3 + 2] = f2 + gk[2];
                }
            }
    return 0;
}

/* Reductions of csrc/binding.cpp:198,209-219 from grads (N,T,U1,3):
 *   grad_den = -sum_k grads;  grad_cg = sum_t grads;
 *   grad_cf[...,0] = sum_u grads[...,0];  grad_cf[...,k] = grads[...,k,1] + grads[...,k-1,2]. */
int oracle_simple_reduce(const float *grads, int N, int T, int U1, float *grad_cf, float *grad_cg,
                         float *grad_den) {
    memset(grad_cg, 0, sizeof(float) * (size_t)N * U1 * 3);
    for (int n = 0; n < N; ++n)
        for (int t = 0; t < T; ++t) {
            const float *gr = grads + ((size_t)n * T + t) * U1 * 3;
            float *cfr = grad_cf + ((size_t)n * T + t) * U1;
            float blank = 0.0f;
            for (int u = 0; u < U1; ++u) {
                blank += gr[u * 3];
                if (grad_den) grad_den[((size_t)n * T + t) * U1 + u] = -(gr[u * 3] + gr[u * 3 + 1] + gr[u * 3 + 2]);
                for (int k = 0; k < 3; ++k) grad_cg[((size_t)n * U1 + u) * 3 + k] += gr[u * 3 + k];
                if (u >= 1) cfr[u] = gr[u * 3 + 1] + gr[(u - 1) * 3 + 2];
            }
            cfr[0] = blank;
        }
    return 0;
}

/* Backward of the log-semiring product, the formula of csrc/binding.cpp:251-253:
 *   grad_f[b,i,k] = exp(f[b,i,k]) * sum_j (grad_den[b,i,j] / exp(den[b,i,j])) * exp(g[b,j,k])
 *   grad_g[b,j,k] = exp(g[b,j,k]) * sum_i (grad_den[b,i,j] / exp(den[b,i,j])) * exp(f[b,i,k])
 * evaluated in double as sum of exp(f + g - den) * grad_den.  Accumulates (+=) into the
 * outputs so the caller can pre-load the scatter of the lattice gradients. */
int oracle_log_matmul_backward(const float *grad_den, const float *f, const float *g,
                               const float *den, int B, int M, int Nc, int K, double *grad_f,
                               double *grad_g, int nthreads) {
    set_threads(nthreads);
    for (int b = 0; b < B; ++b) {
#pragma omp parallel for schedule(static)
        for (int k = 0; k < K; ++k) {
            for (int i = 0; i < M; ++i) {
                const double fv = f[((size_t)b * M + i) * K + k];
                double acc = 0.0;
                for (int j = 0; j < Nc; ++j) {
                    const size_t c = ((size_t)b * M + i) * Nc + j;
                    const double w = exp(fv + (double)g[((size_t)b * Nc + j) * K + k] - (double)den[c]) *
                                     (double)grad_den[c];
                    acc += w;
                    if (grad_g) grad_g[((size_t)b * Nc + j) * K + k] += w;
                }
                if (grad_f) grad_f[((size_t)b * M + i) * K + k] += acc;
            }
        }
    }
    return 0;
}

// Gradient kernels.
//
//  k_fill_grad   : occupancy gradient w.r.t. the three gathered log-probs of every (n,t,u),
//                  the quantity the reference's k_fill_grad produces (csrc/gather.cu:311-374),
//                  evaluated from the normalised tables of lattice.cuh.
//  k_scatter_*   : the dense (N,T,U+1,V) gradient in ONE pass of 16-byte stores: zeros
//                  everywhere except <= 3 patched columns per row.  Replaces what autograd does
//                  for the reference after CTCTLoss.backward (warp_ctct/__init__.py:31-33): a
//                  multiply, a cast, a memset of the full tensor and a scatter_add.
//  k_export_tables: test hook, tables in natural-log units and unshifted coordinates.
#pragma once

#include "common.cuh"

namespace ctct {

struct GradArgs {
    const float *G;    // [N][T][3][U1p]
    const float *TAB;  // [N][T][4][U1p]
    const int *OFF;    // [N][T][2][NL]
    const float *llf;  // [N][2]
    const int *lli;    // [N][2]
    const int *ys, *lx, *ly;
    float *out;        // internal [N][T][3][U1p] or reference [N][T][U1][3]
    int T, U1, U1p, NL, C;
    int ref_layout;
};

// One thread per (t,u) of one utterance (blockIdx.y).  Every arc (state at t) -> (state at
// t+1) contributes exp2(alpha + logp + beta - loglik); arcs outside the band contribute an
// exact 0 because one of the two variables is "impossible" there, so the reference's band
// guards (gather.cu:335-337,355-359) need no restating.
__global__ void __launch_bounds__(256) k_fill_grad(const GradArgs a) {
    const int n = blockIdx.y;
    const int cells = a.T * a.U1;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= cells) return;
    const int t = idx / a.U1;
    const int u = idx - t * a.U1;
    const int U1p = a.U1p, U = a.U1 - 1;
    const int Tn = max(0, min(a.lx[n], a.T));
    const int Un = max(0, min(a.ly[n], U));
    const int64_t nt = static_cast<int64_t>(n) * a.T + t;

    float g0 = 0.0f, g1 = 0.0f, g2 = 0.0f;
    const float lf = a.llf[n * 2 + 1];
    if (t < Tn && u <= Un && lf > NEG_TEST) {
        const int li = a.lli[n * 2 + 1];
        const float *row = a.G + nt * 3 * U1p;
        const float *tab = a.TAB + nt * 4 * U1p;
        const int *off = a.OFF + nt * 2 * a.NL;
        const float aL = tab[u], aB = tab[U1p + u];
        const float bL = tab[2 * U1p + u], bB = tab[3 * U1p + u];
        const float p0 = to_log2(row[u]), p1 = to_log2(row[U1p + u]), p2 = to_log2(row[2 * U1p + u]);
        const int la = u / a.C;
        const int oA = off[la];
        const float c_same = static_cast<float>(oA + off[a.NL + la] - li) - lf;
        // arcs leaving the blank state 2u: stay (blank), or emit label u
        float occ0 = ex2(aB + bB + p0 + c_same);
        float occ1 = 0.0f, occ2 = 0.0f;
        if (u >= 1) {
            // arcs leaving the label state 2u-1: to blank 2u, stay (repeat label u-1)
            occ0 += ex2(aL + bB + p0 + c_same);
            occ1 = ex2(aL + bL + p1 + c_same);
        }
        if (u < Un) {
            const int lb = (u + 1) / a.C;
            const float bLn = tab[2 * U1p + u + 1];
            const float c_next = static_cast<float>(oA + off[a.NL + lb] - li) - lf;
            occ2 = ex2(aB + bLn + p2 + c_next);
            if (u >= 1) {
                const int *y = a.ys + static_cast<int64_t>(n) * U;
                if (y[u] != y[u - 1]) occ2 += ex2(aL + bLn + p2 + c_next);
            }
        }
        g0 = -occ0;
        g1 = -occ1;
        g2 = -occ2;
    }
    if (a.ref_layout) {
        float *o = a.out + (nt * a.U1 + u) * 3;
        o[0] = g0;
        o[1] = g1;
        o[2] = g2;
    } else {
        float *o = a.out + nt * 3 * U1p + u;
        o[0] = g0;
        o[U1p] = g1;
        o[2 * U1p] = g2;
    }
}

// ---------------------------------------------------------------------------------------
// dense gradient streamer

template <typename OutT>
struct OutOps;
template <>
struct OutOps<float> {
    static constexpr int E = 4;  // elements per 16-byte store
    __device__ static float cvt(float x) { return x; }
    __device__ static float add(float a, float b) { return a + b; }
    __device__ static unsigned bits(float x) { return __float_as_uint(x); }
};
template <>
struct OutOps<__half> {
    static constexpr int E = 8;
    __device__ static __half cvt(float x) { return __float2half_rn(x); }
    __device__ static __half add(__half a, __half b) { return __hadd(a, b); }
    __device__ static unsigned bits(__half x) { return __half_as_ushort(x); }
};
template <>
struct OutOps<__nv_bfloat16> {
    static constexpr int E = 8;
    __device__ static __nv_bfloat16 cvt(float x) { return __float2bfloat16_rn(x); }
    __device__ static __nv_bfloat16 add(__nv_bfloat16 a, __nv_bfloat16 b) { return __hadd(a, b); }
    __device__ static unsigned bits(__nv_bfloat16 x) { return __bfloat16_as_ushort(x); }
};

struct ScatterArgs {
    const float *GR;        // [N][T][3][U1p] compact gradient
    const float *grad_out;  // [N]
    const int *ys, *lx, *ly;
    void *out;              // [N][T][U1][V]
    int T, U1, U1p, V;
    int64_t rows;           // N*T*U1
};

// value of column `col` of a row whose three patched columns are 0, i1, i2
template <typename OutT>
__device__ __forceinline__ OutT patched(int col, int i1, int i2, OutT v0, OutT v1, OutT v2, bool has1, bool has2) {
    OutT acc = OutOps<OutT>::cvt(0.0f);
    if (col == 0) acc = OutOps<OutT>::add(acc, v0);
    if (has1 && col == i1) acc = OutOps<OutT>::add(acc, v1);
    if (has2 && col == i2) acc = OutOps<OutT>::add(acc, v2);
    return acc;
}

// One warp per vocabulary row, rows dealt round-robin to warps so that at any moment the
// grid writes one contiguous window of the tensor.  VEC = true: V is a multiple of the
// vector width and the base is 16-byte aligned, every lane issues st.global.v4.
template <typename OutT, bool VEC>
__global__ void __launch_bounds__(256) k_scatter_dense(const ScatterArgs a) {
    constexpr int E = OutOps<OutT>::E;
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const int U = a.U1 - 1, V = a.V;
    OutT *out = static_cast<OutT *>(a.out);

    for (int64_t r = warp0; r < a.rows; r += nwarps) {
        const int64_t nt = r / a.U1;
        const int u = static_cast<int>(r - nt * a.U1);
        const int n = static_cast<int>(nt / a.T);
        const int t = static_cast<int>(nt - static_cast<int64_t>(n) * a.T);
        const int Tn = min(a.lx[n], a.T), Un = min(a.ly[n], U);
        OutT v0 = OutOps<OutT>::cvt(0.0f), v1 = v0, v2 = v0;
        int i1 = -1, i2 = -1;
        bool has1 = false, has2 = false;
        const bool valid = t < Tn && u <= Un;
        if (valid) {
            const float go = a.grad_out[n];
            const float *g = a.GR + nt * 3 * a.U1p + u;
            v0 = OutOps<OutT>::cvt(go * g[0]);
            if (u >= 1) {
                has1 = true;
                i1 = min(max(a.ys[static_cast<int64_t>(n) * U + u - 1], 0), V - 1);
                v1 = OutOps<OutT>::cvt(go * g[a.U1p]);
            }
            if (u < Un) {
                has2 = true;
                i2 = min(max(a.ys[static_cast<int64_t>(n) * U + u], 0), V - 1);
                v2 = OutOps<OutT>::cvt(go * g[2 * a.U1p]);
            }
        }
        OutT *dst = out + r * V;
        if (VEC) {
            const int nvec = V / E;
            const int j1 = has1 ? i1 / E : -1, j2 = has2 ? i2 / E : -1;
            uint4 *dv = reinterpret_cast<uint4 *>(dst);
            for (int j = lane; j < nvec; j += 32) {
                uint4 w = make_uint4(0u, 0u, 0u, 0u);
                if (valid && (j == 0 || j == j1 || j == j2)) {
                    unsigned b[E];
#pragma unroll
                    for (int e = 0; e < E; ++e)
                        b[e] = OutOps<OutT>::bits(patched<OutT>(j * E + e, i1, i2, v0, v1, v2, has1, has2));
                    if constexpr (E == 4) {
                        w = make_uint4(b[0], b[1], b[2], b[3]);
                    } else {
                        w = make_uint4(b[0] | (b[1] << 16), b[2] | (b[3] << 16), b[4] | (b[5] << 16),
                                       b[6] | (b[7] << 16));
                    }
                }
                __stcs(dv + j, w);
            }
        } else {
            for (int col = lane; col < V; col += 32)
                dst[col] = valid ? patched<OutT>(col, i1, i2, v0, v1, v2, has1, has2) : OutOps<OutT>::cvt(0.0f);
        }
    }
}

// ---------------------------------------------------------------------------------------
// test hook

struct ExportArgs {
    const float *TAB;
    const int *OFF;
    const float *llf;
    const int *lli;
    const int *lx, *ly;
    double *alpha, *beta_next, *ll_alpha, *ll_beta;
    int T, U1, U1p, NL, C;
};

__global__ void __launch_bounds__(256) k_export_tables(const ExportArgs a) {
    const int n = blockIdx.y;
    const int U = a.U1 - 1, S = 2 * U + 1;
    const int cells = a.T * S;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const double ninf = -__longlong_as_double(0x7ff0000000000000LL);
    if (idx == 0) {
        for (int d = 0; d < 2; ++d) {
            const float f = a.llf[n * 2 + d];
            const double v = f > NEG_TEST ? (static_cast<double>(a.lli[n * 2 + d]) + f) * LN2 : ninf;
            (d ? a.ll_beta : a.ll_alpha)[n] = v;
        }
    }
    if (idx >= cells) return;
    const int t = idx / S, s = idx - t * S;
    const int u = (s + 1) / 2, kind = (s & 1) ? 0 : 1;  // label state 2u-1 -> slot 0, blank 2u -> slot 1
    const int Tn = max(0, min(a.lx[n], a.T)), Un = max(0, min(a.ly[n], U));
    const int64_t nt = static_cast<int64_t>(n) * a.T + t;
    double va = ninf, vb = ninf;
    if (t < Tn && u <= Un) {
        const float *tab = a.TAB + nt * 4 * a.U1p;
        const int *off = a.OFF + nt * 2 * a.NL;
        const int l = u / a.C;
        const float x = tab[kind * a.U1p + u], y = tab[(2 + kind) * a.U1p + u];
        if (x > NEG_TEST) va = (static_cast<double>(off[l]) + x) * LN2;
        if (y > NEG_TEST) vb = (static_cast<double>(off[a.NL + l]) + y) * LN2;
    }
    a.alpha[nt * S + s] = va;
    a.beta_next[nt * S + s] = vb;
}

}  // namespace ctct

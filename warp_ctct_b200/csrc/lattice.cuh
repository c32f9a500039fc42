// Forward (alpha) and backward (beta) lattice recursions of the CTC-Transducer loss.
//
// What is computed is what the reference's k_warp_alphas / k_warp_betas compute
// (csrc/gather.cu:36-291; CPU twins ref_fw_simple / ref_bw_simple, ref_ctct.py:6-74), but
// organised for the hardware instead of ported:
//
//  * The recursion is time-synchronous: the state vector at frame t+1 depends only on the
//    one at frame t.  In the reference's band storage a fixed frame is an anti-diagonal
//    staircase; here a frame is simply one wavefront step.
//  * One CTA per (utterance, direction), no waits between CTAs.  The 2U+1 lattice states
//    live in REGISTERS, grouped by context u: lane l owns contexts [l*C, l*C+C) and for each
//    the pair (label state 2u-1, blank state 2u).  One step needs a single neighbour value
//    (one warp shuffle; shared memory + one barrier per frame only when an utterance needs
//    more than one warp).
//  * The three gathered log-probs per (frame, context) are staged through shared memory in
//    chunks of F frames with cp.async, double buffered, so that the T dependent steps never
//    wait on DRAM.
//  * Arithmetic is in log2 units (ex2/lg2 are single MUFU instructions) and every lane keeps
//    its values near zero by subtracting an INTEGER per-lane offset each frame; the offsets
//    are carried exactly in int32.  The stored tables are therefore accurate to ~1e-6
//    regardless of T, where plain fp32 log-domain tables (values ~ -3000) carry ~1e-4.
//
// Table layout (only written when a gradient is wanted), per (n, t):
//   TAB[n][t][0][u] = alpha(t, 2u-1)   TAB[n][t][1][u] = alpha(t, 2u)
//   TAB[n][t][2][u] = beta(t+1, 2u-1)  TAB[n][t][3][u] = beta(t+1, 2u)
//   OFF[n][t][0][l], OFF[n][t][1][l]   = int offset of lane l for alpha / beta of that row
//   true value (log2 units) = stored + offset.
#pragma once

#include "common.cuh"

namespace ctct {

struct LatticeArgs {
    const float *G;      // [N][T][3][U1p] gathered log-probs (natural log), zeros where invalid
    const int *ys;       // [N][U1-1]
    const int *lx;       // [N]
    const int *ly;       // [N]
    float *TAB;          // [N][T][4][U1p]
    int *OFF;            // [N][T][2][NL]
    float *llf;          // [N][2]  fractional part of log2-likelihood from alpha / beta
    int *lli;            // [N][2]  integer part
    float *costs;        // [N]
    int T, U1, U1p, NL, F;
    int beta_only;       // 1: only the backward variable (no gradient wanted), no table stores
};

template <int C, int W>
__global__ void __launch_bounds__(W * 32) k_lattice(const LatticeArgs a) {
    extern __shared__ __align__(16) float smem[];
    constexpr unsigned FULL = 0xffffffffu;
    const int n = blockIdx.x;
    const int dir = a.beta_only ? 1 : static_cast<int>(blockIdx.y);
    const bool store = !a.beta_only;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int U1p = a.U1p, R = 3 * U1p, F = a.F, T = a.T;
    const int U = a.U1 - 1;
    const int Tn = max(0, min(a.lx[n], T));
    const int Un = max(0, min(a.ly[n], U));
    const int u0 = tid * C;
    const bool active = u0 <= Un;

    float *buf0 = smem;
    float *buf1 = smem + static_cast<size_t>(F) * R;
    float *xf = smem + 2 * static_cast<size_t>(F) * R;  // [2][W] exchanged value
    int *xi = reinterpret_cast<int *>(xf + 2 * W);      // [2][W] exchanged offset

    bool dskip[C], labok[C];
    int uidx[C];
    {
        const int *y = a.ys + static_cast<int64_t>(n) * U;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int u = u0 + c;
            uidx[c] = min(u, U1p - 1);
            labok[c] = u < Un;
            dskip[c] = false;
            if (u >= 1 && u < Un) dskip[c] = y[u] != y[u - 1];
        }
    }

    const int64_t rowbase = static_cast<int64_t>(n) * T;
    const float *Gn = a.G + rowbase * R;

    float L[C], Bk[C];
    int off = 0;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        L[c] = NEG;
        Bk[c] = NEG;
    }
    if (dir == 0) {
        if (tid == 0) Bk[0] = 0.0f;
    } else {
#pragma unroll
        for (int c = 0; c < C; ++c)
            if (u0 + c == Un) {
                Bk[c] = 0.0f;
                if (Un >= 1) L[c] = 0.0f;
            }
    }

    const int nchunks = (Tn + F - 1) / F;
    auto chunk_range = [&](int c, int &lo, int &hi) {
        if (dir == 0) {
            lo = c * F;
            hi = min(Tn, lo + F);
        } else {
            hi = Tn - c * F;
            lo = max(0, hi - F);
        }
    };
    auto issue = [&](int c, float *dst) {
        int lo, hi;
        chunk_range(c, lo, hi);
        const float *src = Gn + static_cast<int64_t>(lo) * R;
        const int nvec = (hi - lo) * R / 4;
        for (int v = tid; v < nvec; v += W * 32) cp_async16(dst + 4 * v, src + 4 * v);
        cp_async_commit();
    };
    auto sync = [&]() {
        if (W == 1)
            __syncwarp();
        else
            __syncthreads();
    };

    int parity = 0;
    if (nchunks > 0) issue(0, buf0);
    for (int c = 0; c < nchunks; ++c) {
        float *cur = (c & 1) ? buf1 : buf0;
        if (c + 1 < nchunks) {
            issue(c + 1, (c & 1) ? buf0 : buf1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        sync();
        int lo, hi;
        chunk_range(c, lo, hi);
        const int nf = hi - lo;
        for (int f = 0; f < nf; ++f) {
            const int tl = (dir == 0) ? f : nf - 1 - f;
            const int t = lo + tl;
            const float *row = cur + static_cast<size_t>(tl) * R;

            if (store && active) {
                float *tr = a.TAB + (rowbase + t) * 4 * U1p + (dir ? 2 * U1p : 0);
#pragma unroll
                for (int cc = 0; cc < C; ++cc)
                    if (u0 + cc < U1p) {
                        tr[u0 + cc] = L[cc];
                        tr[U1p + u0 + cc] = Bk[cc];
                    }
                a.OFF[((rowbase + t) * 2 + dir) * a.NL + tid] = off;
            }

            float p0[C], p1[C], p2[C];
#pragma unroll
            for (int cc = 0; cc < C; ++cc) {
                p0[cc] = to_log2(row[uidx[cc]]);
                p1[cc] = to_log2(row[U1p + uidx[cc]]);
                p2[cc] = to_log2(row[2 * U1p + uidx[cc]]);
            }

            float nL[C], nB[C];
            if (dir == 0) {
                // alpha(t+1) from alpha(t).  P[u] = everything that enters label state 2u+1
                // from context u: from the blank state 2u, and from the label state 2u-1 when
                // the two labels differ (gather.cu:131-148 in band coordinates).
                float q[C], P[C];
#pragma unroll
                for (int cc = 0; cc < C; ++cc) {
                    q[cc] = lse2(Bk[cc], L[cc]);
                    P[cc] = labok[cc] ? p2[cc] + (dskip[cc] ? q[cc] : Bk[cc]) : NEG;
                }
                float Pin = __shfl_up_sync(FULL, P[C - 1], 1);
                int oin = __shfl_up_sync(FULL, off, 1);
                if (W > 1) {
                    if (lane == 31) {
                        xf[parity * W + warp] = P[C - 1];
                        xi[parity * W + warp] = off;
                    }
                    __syncthreads();
                    if (lane == 0 && warp > 0) {
                        Pin = xf[parity * W + warp - 1];
                        oin = xi[parity * W + warp - 1];
                    }
                    parity ^= 1;
                }
                if (tid == 0) Pin = NEG;
                Pin = (Pin > NEG_TEST) ? Pin + static_cast<float>(oin - off) : NEG;
#pragma unroll
                for (int cc = 0; cc < C; ++cc) {
                    const float pin = (cc == 0) ? Pin : P[cc == 0 ? 0 : cc - 1];
                    nL[cc] = lse2(L[cc] + p1[cc], pin);
                    nB[cc] = p0[cc] + q[cc];
                }
            } else {
                // beta(t) from beta(t+1) (gather.cu:222-271 in band coordinates).
                float Lin = __shfl_down_sync(FULL, L[0], 1);
                int oin = __shfl_down_sync(FULL, off, 1);
                if (W > 1) {
                    if (lane == 0) {
                        xf[parity * W + warp] = L[0];
                        xi[parity * W + warp] = off;
                    }
                    __syncthreads();
                    if (lane == 31 && warp + 1 < W) {
                        Lin = xf[parity * W + warp + 1];
                        oin = xi[parity * W + warp + 1];
                    }
                    parity ^= 1;
                }
                if (tid == W * 32 - 1) Lin = NEG;
                Lin = (Lin > NEG_TEST) ? Lin + static_cast<float>(oin - off) : NEG;
#pragma unroll
                for (int cc = 0; cc < C; ++cc) {
                    const float ln = (cc == C - 1) ? Lin : L[cc == C - 1 ? cc : cc + 1];
                    const float X = p0[cc] + Bk[cc];                   // emit blank, go to / stay in 2u
                    const float Y = labok[cc] ? p2[cc] + ln : NEG;     // emit label u, go to 2u+1
                    nB[cc] = lse2(X, Y);
                    nL[cc] = lse2(p1[cc] + L[cc], dskip[cc] ? nB[cc] : X);
                }
                if (tid == 0) nL[0] = NEG;  // context 0 has no label state
            }

            // keep this lane's values near zero; the integer offset carries the rest exactly
            float m = NEG;
#pragma unroll
            for (int cc = 0; cc < C; ++cc) m = fmaxf(m, fmaxf(nL[cc], nB[cc]));
            const float k = (m > NEG_TEST) ? rintf(m) : 0.0f;
#pragma unroll
            for (int cc = 0; cc < C; ++cc) {
                L[cc] = nL[cc] - k;
                Bk[cc] = nB[cc] - k;
            }
            off += static_cast<int>(k);
        }
        sync();
    }

    if (dir == 0) {
#pragma unroll
        for (int cc = 0; cc < C; ++cc)
            if (u0 + cc == Un) {
                a.llf[n * 2 + 0] = lse2(Bk[cc], L[cc]);
                a.lli[n * 2 + 0] = off;
            }
    } else if (tid == 0) {
        a.llf[n * 2 + 1] = Bk[0];
        a.lli[n * 2 + 1] = off;
        const float frac = Bk[0];
        float cost = __int_as_float(0x7f800000);  // no alignment exists
        if (frac > NEG_TEST) cost = static_cast<float>(-(static_cast<double>(off) + static_cast<double>(frac)) * LN2);
        a.costs[n] = cost;
    }
}

}  // namespace ctct

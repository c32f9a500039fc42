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
//    live in REGISTERS, grouped by context u: a thread owns C consecutive contexts (C = 1 up
//    to 1024 contexts) and for each the pair (label state 2u-1, blank state 2u).  A single
//    warp is latency-bound on its own instruction stream, so the per-thread work is kept
//    minimal and the contexts are spread over as many lanes as there are contexts; one step
//    needs the neighbour's values through a warp shuffle, and across warps through shared
//    memory and one CTA barrier per frame.
//  * Every new state value is ONE log-sum-exp of values of the previous frame (the two- and
//    three-way sums are taken directly, not chained), and the renormaliser of a frame is
//    derived from the values the frame started with, so neither the neighbour exchange nor
//    the renormalisation lengthens the frame-to-frame dependency chain.
//  * The three gathered log-probs per (frame, context) are one 16-byte record; they are
//    staged through shared memory in chunks of F frames with cp.async, double buffered, so
//    that the T dependent steps never wait on DRAM.
//  * Arithmetic is in log2 units (ex2/lg2 are single MUFU instructions) and every thread keeps
//    its values near zero by subtracting an INTEGER offset each frame; the offsets are carried
//    exactly in int32.  The stored tables are therefore accurate to ~1e-6 regardless of T,
//    where plain fp32 log-domain tables (values ~ -3000) carry ~1e-4.
//
// Table record (only written when a gradient is wanted), one float4 per (n, t, dir, u):
//   dir 0: {alpha(t, 2u-1), alpha(t, 2u), offset, -}    dir 1: {beta(t+1, 2u-1), beta(t+1, 2u), offset, -}
//   true value (log2 units) = stored + offset (offset is an int32 stored bit-for-bit).
#pragma once

#include "common.cuh"

namespace ctct {

struct LatticeArgs {
    const float4 *G;     // [N][T][U1] {blank, repeat-label, next-label, 0} in log2 units, clamped at NEG; 0 where invalid
    const int *ys;       // [N][U1-1]
    const int *lx;       // [N]
    const int *ly;       // [N]
    float4 *TAB;         // [N][T][2][U1]
    float *llf;          // [N][2]  fractional part of log2-likelihood from alpha / beta
    int *lli;            // [N][2]  integer part
    float *costs;        // [N]
    int T, U1, F;
    int beta_only;       // 1: only the backward variable (no gradient wanted), no table stores
};

template <int C>
__global__ void __launch_bounds__(1024) k_lattice(const LatticeArgs a) {
    extern __shared__ __align__(16) float4 smem4[];
    constexpr unsigned FULL = 0xffffffffu;
    const int n = blockIdx.x;
    const int dir = a.beta_only ? 1 : static_cast<int>(blockIdx.y);
    const bool store = !a.beta_only;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NT = blockDim.x, W = NT >> 5;
    const int U1 = a.U1, F = a.F, T = a.T;
    const int U = U1 - 1;
    const int Tn = max(0, min(a.lx[n], T));
    const int Un = max(0, min(a.ly[n], U));
    const int u0 = tid * C;
    const bool active = u0 <= Un;

    float4 *buf0 = smem4;
    float4 *buf1 = smem4 + static_cast<size_t>(F) * U1;
    float4 *xch = smem4 + 2 * static_cast<size_t>(F) * U1;  // [2][W] values handed to the next / previous warp

    bool dskip[C], labok[C];
    int uidx[C];
    {
        const int *y = a.ys + static_cast<int64_t>(n) * U;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int u = u0 + c;
            uidx[c] = min(u, U1 - 1);
            labok[c] = u < Un;
            dskip[c] = false;
            if (u >= 1 && u < Un) dskip[c] = y[u] != y[u - 1];
        }
    }

    const int64_t rowbase = static_cast<int64_t>(n) * T;
    const float4 *Gn = a.G + rowbase * U1;

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
    auto issue = [&](int c, float4 *dst) {
        int lo, hi;
        chunk_range(c, lo, hi);
        const float4 *src = Gn + static_cast<int64_t>(lo) * U1;
        const int nvec = (hi - lo) * U1;
        for (int v = tid; v < nvec; v += NT) cp_async16(dst + v, src + v);
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
        const float4 *cur = (c & 1) ? buf1 : buf0;
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
        const int tstep = (dir == 0) ? 1 : -1;
        int t = (dir == 0) ? lo : hi - 1;
        const float4 *row = cur + static_cast<int64_t>(t - lo) * U1;
        float4 *tr = a.TAB + ((rowbase + t) * 2 + dir) * U1 + u0;
        for (int f = 0; f < nf; ++f, t += tstep, row += tstep * U1, tr += tstep * 2 * U1) {
            if (store && active) {
#pragma unroll
                for (int cc = 0; cc < C; ++cc)
                    if (u0 + cc < U1) tr[cc] = make_float4(L[cc], Bk[cc], __int_as_float(off), 0.0f);
            }

            float4 p[C];
#pragma unroll
            for (int cc = 0; cc < C; ++cc) p[cc] = row[uidx[cc]];

            // Renormaliser of this frame, from the values the frame starts with (off the
            // dependency chain: it is only needed for the final subtraction).
            float m = NEG;
#pragma unroll
            for (int cc = 0; cc < C; ++cc) m = fmaxf(m, fmaxf(L[cc], Bk[cc]));
            const bool untouched = !(m > NEG_TEST);
            const float k = untouched ? 0.0f : rintf(m);

            float nL[C], nB[C];
            if (dir == 0) {
                // alpha(t+1) from alpha(t).  tB / tL: what context u sends into label state 2u+1,
                // from its blank state 2u and, when labels u-1 and u differ, from its label
                // state 2u-1 (gather.cu:131-148 in band coordinates).
                float tB[C], tL[C];
#pragma unroll
                for (int cc = 0; cc < C; ++cc) {
                    tB[cc] = labok[cc] ? p[cc].z + Bk[cc] : NEG;
                    tL[cc] = dskip[cc] ? p[cc].z + L[cc] : NEG;
                }
                float inB = __shfl_up_sync(FULL, tB[C - 1], 1);
                float inL = __shfl_up_sync(FULL, tL[C - 1], 1);
                int oin = __shfl_up_sync(FULL, off, 1);
                if (W > 1) {
                    if (lane == 31) xch[parity * W + warp] = make_float4(tB[C - 1], tL[C - 1], __int_as_float(off), 0.0f);
                    __syncthreads();
                    if (lane == 0 && warp > 0) {
                        const float4 x = xch[parity * W + warp - 1];
                        inB = x.x;
                        inL = x.y;
                        oin = __float_as_int(x.z);
                    }
                    parity ^= 1;
                }
                if (tid == 0) {
                    inB = NEG;
                    inL = NEG;
                }
                // a thread none of whose states has been reached yet adopts its neighbour's
                // scale, so the first value it receives is small in magnitude
                if (untouched && (inB > NEG_TEST || inL > NEG_TEST)) off = oin;
                const float adj = static_cast<float>(oin - off);
                inB = (inB > NEG_TEST) ? inB + adj : NEG;
                inL = (inL > NEG_TEST) ? inL + adj : NEG;
#pragma unroll
                for (int cc = 0; cc < C; ++cc) {
                    const float b1 = (cc == 0) ? inB : tB[cc == 0 ? 0 : cc - 1];
                    const float c1 = (cc == 0) ? inL : tL[cc == 0 ? 0 : cc - 1];
                    nL[cc] = lse3(L[cc] + p[cc].y, b1, c1);
                    nB[cc] = p[cc].x + lse2(Bk[cc], L[cc]);
                }
            } else {
                // beta(t) from beta(t+1) (gather.cu:222-271 in band coordinates).
                float Lin = __shfl_down_sync(FULL, L[0], 1);
                int oin = __shfl_down_sync(FULL, off, 1);
                if (W > 1) {
                    if (lane == 0) xch[parity * W + warp] = make_float4(L[0], 0.0f, __int_as_float(off), 0.0f);
                    __syncthreads();
                    if (lane == 31 && warp + 1 < W) {
                        const float4 x = xch[parity * W + warp + 1];
                        Lin = x.x;
                        oin = __float_as_int(x.z);
                    }
                    parity ^= 1;
                }
                if (tid == NT - 1) Lin = NEG;
                if (untouched && Lin > NEG_TEST) off = oin;
                Lin = (Lin > NEG_TEST) ? Lin + static_cast<float>(oin - off) : NEG;
#pragma unroll
                for (int cc = 0; cc < C; ++cc) {
                    const float ln = (cc == C - 1) ? Lin : L[cc == C - 1 ? cc : cc + 1];
                    const float X = p[cc].x + Bk[cc];                   // emit blank, go to / stay in 2u
                    const float Y = labok[cc] ? p[cc].z + ln : NEG;     // emit label u, go to 2u+1
                    nB[cc] = lse2(X, Y);
                    nL[cc] = lse3(p[cc].y + L[cc], X, dskip[cc] ? Y : NEG);
                }
                if (tid == 0) nL[0] = NEG;  // context 0 has no label state
            }

            // keep this thread's values near zero; the integer offset carries the rest exactly
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

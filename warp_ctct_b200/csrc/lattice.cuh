// Forward (alpha) and backward (beta) lattice recursions of the CTC-Transducer loss.
//
// What is computed is what the reference's k_warp_alphas / k_warp_betas compute
// (csrc/gather.cu:36-291; CPU twins ref_fw_simple / ref_bw_simple, ref_ctct.py:6-74), but
// organised for the hardware instead of ported:
//
//  * The recursion is time-synchronous: the state vector at frame t+1 depends only on the
//    one at frame t.  In the reference's band storage a fixed frame is an anti-diagonal
//    staircase; here a frame is simply one wavefront step.
//  * One CTA per (utterance, direction), no waits between CTAs.  A lone warp issues about one
//    instruction every five cycles, so a frame costs (instructions per frame) x 5 cycles and the
//    design minimises exactly that count: ONE lattice state per thread, held in a register, and
//    the same straight-line code for every state,
//        new = lse3(own + p_stay, left + p_adv, skip ? left2 + p_adv : impossible),
//    with the two neighbours taken by warp shuffles and, across warps, through shared memory
//    and one CTA barrier per frame.  States sit in "slots": slot 2u = label state 2u-1 of
//    context u, slot 2u+1 = blank state 2u; slot 0 is a dummy that stays impossible.
//  * The three gathered log-probs per (frame, context) are one 16-byte record; they are
//    staged through shared memory in chunks of F frames with cp.async, double buffered, so
//    that the T dependent steps never wait on DRAM.
//  * Arithmetic is in log2 units (ex2/lg2 are single MUFU instructions).  Every RENORM frames a
//    warp subtracts the rounded maximum of its 32 values (one redux.sync) and adds it to an
//    exact int32 offset, so stored values stay within a few tens of zero whatever T is; plain
//    fp32 log-domain tables (values ~ -3000, ulp 2.4e-4) cannot hold 1e-4 gradients.
//
// Table record (only written when a gradient is wanted): float2 {value, int32 offset bits} per
// (n, t, dir, slot); dir 0 = alpha(t), dir 1 = beta(t+1); true log2 value = value + offset.
// Read per context as one float4 {label value, offset, blank value, offset}.
#pragma once

#include <type_traits>

#include "common.cuh"

namespace ctct {

struct LatticeArgs {
    const float4 *G;     // [N][T][U1] {blank, repeat-label, next-label, 0} in log2 units, clamped at NEG; 0 where invalid
    const int *ys;       // [N][U1-1]
    const int *lx;       // [N]
    const int *ly;       // [N]
    float2 *TAB;         // [N][T][2][2*U1]
    float *llf;          // [N][2]  fractional part of log2-likelihood from alpha / beta
    int *lli;            // [N][2]  integer part
    float *costs;        // [N]
    int T, U1, F;
    int beta_only;       // 1: only the backward variable (no gradient wanted), no table stores
    int threads;         // threads of one lattice CTA (multiple of 32, <= blockDim.x)
    ClearSlice clear;    // blocks from clear.first_block on zero a slice of the gradient buffer
    PadClear pad;        // or: blocks from pad.first_block on zero the padding rows of a gradient buffer
    unsigned smem_bytes; // dynamic shared memory of the launch
};

// barrier among the first `nthreads` threads of the block (named barrier 1)
__device__ __forceinline__ void cta_sync(int nthreads) { asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory"); }

constexpr int RENORM = 2;  // frames between renormalisations

// C slots per thread (1 up to 480 contexts), DIR 0 = alpha / 1 = beta, MULTI = more than one warp.
//
// With more than one warp, H lanes of every warp are "halo" lanes (H = 2 for C = 1, else 1): they
// hold copies of the neighbouring warp's two boundary slots, reloaded from shared memory at the
// top of every frame, so that the neighbour values of all real lanes come from plain shuffles
// with no per-lane fix-up.  A warp publishes its own two boundary slots after each step; one CTA
// barrier per frame separates publishing from reloading.
template <int C, int DIR, bool MULTI>
__device__ __forceinline__ void lattice_run(const LatticeArgs &a, float4 *smem4) {
    constexpr unsigned FULL = 0xffffffffu;
    constexpr int H = MULTI ? (C == 1 ? 2 : 1) : 0;
    constexpr int REAL_LANES = 32 - H;
    const int n = a.beta_only ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x >> 1);
    const bool store = !a.beta_only;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NT = a.threads, W = NT >> 5;  // threads of the lattice role (the block may be wider)
    const int U1 = a.U1, F = a.F, T = a.T;
    const int U = U1 - 1, S2 = 2 * U1;  // number of slots
    const int Tn = max(0, min(a.lx[n], T));
    const int Un = max(0, min(a.ly[n], U));
    // first slot of this thread; halo lanes mirror the neighbouring warp's numbering
    const int j0 = (DIR == 0) ? (warp * REAL_LANES + lane - H) * C : (warp * REAL_LANES + lane) * C;
    const bool halo = MULTI && ((DIR == 0) ? lane < H : lane >= REAL_LANES);

    float4 *buf0 = smem4;
    float4 *buf1 = smem4 + static_cast<size_t>(F) * U1;
    // exchange area after the two stage buffers: values [2 parities][W + 1][2], offsets [W + 1]
    float *xs = reinterpret_cast<float *>(smem4 + 2 * static_cast<size_t>(F) * U1);
    int *xo = reinterpret_cast<int *>(xs + 4 * (W + 1));
    // alpha: warp w publishes into entry w+1 and reads entry w (entry 0 stays impossible);
    // beta : warp w publishes into entry w and reads entry w+1 (entry W stays impossible)
    const int e_pub = (DIR == 0) ? warp + 1 : warp;
    const int e_in = (DIR == 0) ? warp : warp + 1;

    // per-slot constants: word offsets of the emissions inside a staged row, masks
    int ofs_s[C], ofs_a[C];
    float mask_a[C];
    bool skip[C], real[C];
    {
        const int *y = a.ys + static_cast<int64_t>(n) * U;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int jr = j0 + c;
            const int j = min(max(jr, 0), S2 - 1);
            const int u = j >> 1;
            const bool blank = j & 1;
            real[c] = !halo && jr >= 1 && jr < S2 && u <= Un;
            ofs_s[c] = 4 * u + (blank ? 0 : 1);
            if (DIR == 0) {
                // blank 2u  : stay p0[u], from the label state of u      p0[u]
                // label 2u-1: stay p1[u], from blank / label of u-1      p2[u-1]
                ofs_a[c] = blank ? 4 * u : 4 * max(u - 1, 0) + 2;
                mask_a[c] = real[c] ? 0.0f : NEG;
                skip[c] = real[c] && !blank && u >= 2 && y[u - 1] != y[u - 2];
            } else {
                // blank 2u  : stay p0[u], to the label of u+1 p2[u] (if it exists)
                // label 2u-1: stay p1[u], to the blank of u   p0[u], skip to the label of u+1 p2[u]
                ofs_a[c] = 4 * u + (blank ? 2 : 0);
                mask_a[c] = (real[c] && (!blank || u < Un)) ? 0.0f : NEG;
                skip[c] = real[c] && !blank && u < Un && y[u] != y[u - 1];
            }
        }
    }

    const int64_t rowbase = static_cast<int64_t>(n) * T;
    const float4 *Gn = a.G + rowbase * U1;

    float x[C];
    int off = 0;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int j = j0 + c;
        x[c] = NEG;
        if (!halo) {
            if (DIR == 0) {
                if (j == 1) x[c] = 0.0f;
            } else {
                if (j == 2 * Un + 1 || (j == 2 * Un && Un >= 1)) x[c] = 0.0f;
            }
        }
    }
    if (MULTI) {
        for (int i = tid; i < 4 * (W + 1); i += NT) xs[i] = NEG;
        for (int i = tid; i < W + 1; i += NT) xo[i] = 0;
        cta_sync(NT);
        // publish the starting values so that the first halo load sees them
        if (DIR == 0) {
            if (C == 1) {
                if (lane >= 30) xs[(0 * (W + 1) + e_pub) * 2 + lane - 30] = x[0];
            } else if (lane == 31) {
                xs[(0 * (W + 1) + e_pub) * 2 + 0] = x[C >= 2 ? C - 2 : 0];
                xs[(0 * (W + 1) + e_pub) * 2 + 1] = x[C - 1];
            }
        } else {
            if (C == 1) {
                if (lane < 2) xs[(0 * (W + 1) + e_pub) * 2 + lane] = x[0];
            } else if (lane == 0) {
                xs[(0 * (W + 1) + e_pub) * 2 + 0] = x[0];
                xs[(0 * (W + 1) + e_pub) * 2 + 1] = x[C >= 2 ? 1 : 0];
            }
        }
        cta_sync(NT);
    }
    float adj = 0.0f;        // neighbour warp's offset minus ours
    bool untouched = true;   // no state of this warp reachable yet (as of the last renormalisation)

    const int nchunks = (Tn + F - 1) / F;
    auto chunk_range = [&](int c, int &lo, int &hi) {
        if (DIR == 0) {
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
    // exchange pointers of this thread for the two buffers (parity of the frame number)
    const bool loader = MULTI && ((C == 1) ? halo : (DIR == 0 ? lane == 0 : lane == 31));
    const bool publisher = MULTI && ((DIR == 0) ? (C == 1 ? lane >= 30 : lane == 31) : (C == 1 ? lane < 2 : lane == 0));
    const int lane_in = (C == 1) ? (DIR == 0 ? lane : lane - 30) : 0;
    const int lane_out = (C == 1) ? (DIR == 0 ? lane - 30 : lane) : 0;
    const float *in_p[2] = {xs + (0 * (W + 1) + e_in) * 2 + (loader ? lane_in : 0),
                            xs + (1 * (W + 1) + e_in) * 2 + (loader ? lane_in : 0)};
    float *out_p[2] = {xs + (0 * (W + 1) + e_pub) * 2 + (publisher ? lane_out : 0),
                       xs + (1 * (W + 1) + e_pub) * 2 + (publisher ? lane_out : 0)};
    const bool off_publisher = MULTI && lane == (DIR == 0 ? 31 : 0);

    const float *row = nullptr;
    float2 *tr = nullptr;

    // One frame.  PAR = parity of the frame number: buffer PAR holds what the neighbours published
    // at the end of the previous frame, buffer PAR^1 receives this frame's; even frames renormalise.
    auto frame_step = [&](auto PAR) {
        constexpr int par = decltype(PAR)::value;
        constexpr bool renorm = (par % RENORM) == 0;
        if (MULTI) {
            if (par == 1) {  // offsets changed in the previous (even) frame: re-read the neighbour's
                const int offp = xo[e_in];
                if (untouched) off = offp;  // adopt the neighbour's scale until something arrives
                adj = static_cast<float>(offp - off);
            }
            if (C == 1) {
                if (loader) x[0] = in_p[par][0] + adj;
            } else if (loader) {
                x[DIR == 0 ? (C >= 2 ? C - 2 : 0) : 0] = in_p[par][0] + adj;
                x[DIR == 0 ? C - 1 : (C >= 2 ? 1 : 0)] = in_p[par][1] + adj;
            }
        }
        if (renorm) {  // subtract the rounded warp maximum, keep it in the integer offset
            int ki = __float2int_rn(x[0]);
#pragma unroll
            for (int cc = 1; cc < C; ++cc) ki = max(ki, __float2int_rn(x[cc]));
            ki = __reduce_max_sync(FULL, ki);
            untouched = ki < -(1 << 30);
            if (!untouched) {
                const float k = static_cast<float>(ki);
#pragma unroll
                for (int cc = 0; cc < C; ++cc) x[cc] -= k;
                off += ki;
            }
        }
        if (store) {
#pragma unroll
            for (int cc = 0; cc < C; ++cc)
                if (real[cc]) tr[cc] = make_float2(x[cc], __int_as_float(off));
        }

        // neighbours: slot j-1, j-2 (alpha) or j+1, j+2 (beta)
        float n1, n2;  // for the first (alpha) / last (beta) slot of this thread
        if (DIR == 0) {
            n1 = __shfl_up_sync(FULL, x[C - 1], 1);
            n2 = (C >= 2) ? __shfl_up_sync(FULL, x[C >= 2 ? C - 2 : 0], 1) : __shfl_up_sync(FULL, x[0], 2);
            if (!MULTI) {
                if (lane == 0) n1 = NEG;
                if (lane == 0 || (C == 1 && lane == 1)) n2 = NEG;
            }
        } else {
            n1 = __shfl_down_sync(FULL, x[0], 1);
            n2 = (C >= 2) ? __shfl_down_sync(FULL, x[C >= 2 ? 1 : 0], 1) : __shfl_down_sync(FULL, x[0], 2);
            if (!MULTI) {
                if (lane == 31) n1 = NEG;
                if (lane == 31 || (C == 1 && lane == 30)) n2 = NEG;
            }
        }

        // one step of the recursion for every slot of this thread
        float nx[C];
#pragma unroll
        for (int cc = 0; cc < C; ++cc) {
            float v1, v2;
            if (DIR == 0) {
                v1 = (cc >= 1) ? x[cc >= 1 ? cc - 1 : 0] : n1;
                v2 = (cc >= 2) ? x[cc >= 2 ? cc - 2 : 0] : ((cc == 1) ? n1 : n2);
            } else {
                v1 = (cc + 1 < C) ? x[cc + 1 < C ? cc + 1 : 0] : n1;
                v2 = (cc + 2 < C) ? x[cc + 2 < C ? cc + 2 : 0] : ((cc + 2 == C) ? n1 : n2);
            }
            const float ps = row[ofs_s[cc]];
            const float pa = row[ofs_a[cc]] + mask_a[cc];
            float pk = pa;
            if (DIR == 1) pk = row[(ofs_s[cc] & ~3) + 2];  // next-label emission of the same context
            const float t3 = skip[cc] ? v2 + pk : NEG;
            nx[cc] = lse3(x[cc] + ps, v1 + pa, t3);
        }
#pragma unroll
        for (int cc = 0; cc < C; ++cc) x[cc] = nx[cc];

        // publish this warp's boundary slots into buffer par^1 (and its offset after a
        // renormalisation); the barrier orders them before the neighbour's reload
        if (MULTI) {
            if (publisher) {
                if (C == 1) {
                    out_p[par ^ 1][0] = x[0];
                } else {
                    out_p[par ^ 1][0] = x[DIR == 0 ? (C >= 2 ? C - 2 : 0) : 0];
                    out_p[par ^ 1][1] = x[DIR == 0 ? C - 1 : (C >= 2 ? 1 : 0)];
                }
            }
            if (renorm && off_publisher) xo[e_pub] = off;
            cta_sync(NT);
        }
        constexpr int tstep = (DIR == 0) ? 1 : -1;
        row += tstep * 4 * U1;
        tr += tstep * 2 * S2;
    };
    using Even = std::integral_constant<int, 0>;
    using Odd = std::integral_constant<int, 1>;

    int frame = 0;
    if (nchunks > 0) issue(0, buf0);
    for (int c = 0; c < nchunks; ++c) {
        const float4 *cur = (c & 1) ? buf1 : buf0;
        if (c + 1 < nchunks) {
            issue(c + 1, (c & 1) ? buf0 : buf1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        if (MULTI)
            cta_sync(NT);
        else
            __syncwarp();
        int lo, hi;
        chunk_range(c, lo, hi);
        const int nf = hi - lo;
        const int t0 = (DIR == 0) ? lo : hi - 1;
        row = reinterpret_cast<const float *>(cur + static_cast<int64_t>(t0 - lo) * U1);
        tr = a.TAB + ((rowbase + t0) * 2 + DIR) * S2 + j0;
        int f = 0;
        if ((frame & 1) == 0) {
            for (; f + 1 < nf; f += 2) {
                frame_step(Even{});
                frame_step(Odd{});
            }
        }
        for (; f < nf; ++f) {
            if ((frame + f) & 1)
                frame_step(Odd{});
            else
                frame_step(Even{});
        }
        frame += nf;
        if (MULTI)
            cta_sync(NT);
        else
            __syncwarp();
    }

    // ---- log-likelihood
    if (DIR == 0) {
        // alpha(T, 2U-1) and alpha(T, 2U) live in slots 2Un and 2Un+1: same thread (C even) or
        // adjacent real lanes of one warp (warps start on even slots)
        float left[C];
        const float prev = __shfl_up_sync(FULL, x[C - 1], 1);
#pragma unroll
        for (int cc = 0; cc < C; ++cc) left[cc] = (cc >= 1) ? x[cc >= 1 ? cc - 1 : 0] : prev;
#pragma unroll
        for (int cc = 0; cc < C; ++cc)
            if (!halo && j0 + cc == 2 * Un + 1) {
                a.llf[n * 2 + 0] = lse2(x[cc], (j0 + cc == 1) ? NEG : left[cc]);
                a.lli[n * 2 + 0] = off;
            }
    } else {
#pragma unroll
        for (int cc = 0; cc < C; ++cc)
            if (!halo && j0 + cc == 1) {
                const float frac = x[cc];
                a.llf[n * 2 + 1] = frac;
                a.lli[n * 2 + 1] = off;
                float cost = __int_as_float(0x7f800000);  // no alignment exists
                if (frac > NEG_TEST) cost = static_cast<float>(-(static_cast<double>(off) + static_cast<double>(frac)) * LN2);
                a.costs[n] = cost;
            }
    }
}

// One launch, two roles.  The first blocks are the lattice CTAs (utterance n = block / 2,
// direction = block & 1; they are dispatched first).  The remaining blocks stream zeros over a
// slice of the dense gradient buffer of the backward pass (see ClearSlice), so that the
// HBM-bound clearing runs on the SMs the latency-bound lattice leaves idle instead of costing
// its own 150 us later.
template <int C, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) k_lattice(const LatticeArgs a) {
    extern __shared__ __align__(16) float4 smem4[];
    // clearing blocks need nothing from the gather launch before this one and may run beside it
    if (clear_role(a.clear, smem4, a.smem_bytes)) return;
    if (pad_clear_role(a.pad, smem4)) return;
    if (static_cast<int>(threadIdx.x) >= a.threads) return;
    pdl_wait();  // the gathered log-probs are complete and visible
    const int dir = a.beta_only ? 1 : static_cast<int>(blockIdx.x & 1);
    const bool multi = a.threads > 32;
    if (dir == 0) {
        if (multi)
            lattice_run<C, 0, true>(a, smem4);
        else
            lattice_run<C, 0, false>(a, smem4);
    } else {
        if (multi)
            lattice_run<C, 1, true>(a, smem4);
        else
            lattice_run<C, 1, false>(a, smem4);
    }
}

}  // namespace ctct

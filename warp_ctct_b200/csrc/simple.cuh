// Kernels of the log-add joiner ("simple") loss: log-probs are composed on the fly as
// f[n,t,v] + g[n,u,v] - den[n,t,u] with den = log sum_v exp(f + g)  (csrc/simple.cu:20-26,
// csrc/simple_unnorm.cu:20-25 without den, warp_ctct/__init__.py:195-215).
//
//  k_logmm_exact      : batched log-semiring product with a per-output running maximum, any
//                       strides, any dynamic range (the contract of csrc/logmatmul.cu:44-146).
//  k_simple_compose   : gathers of f and g fused with the f+g-den composition, straight into the
//                       lattice's internal 3-slot layout (replaces the two torch.gather calls of
//                       warp_ctct/__init__.py:204-215 and the LOGPROB macros of simple.cu).
//  k_logmm_bwd_exact  : backward of the log-semiring product in linear space,
//                       grad_lhs = sum_j grad_out * exp(lhs + rhs - res) (csrc/binding.cpp:251-253);
//                       the exponent is <= 0, so no sign split or log-space detour is needed.
//  k_simple_patch_*   : adds the lattice's own sparse gradient (blank / label columns) on top,
//                       the reductions of csrc/binding.cpp:198,209-219 plus the gather backwards.
#pragma once

#include "common.cuh"

namespace ctct {

constexpr float LN2F = 0.6931471805599453f;

struct LogmmArgs {
    const float *lhs, *rhs;
    float *out;  // (B, M, N) contiguous
    int64_t lsb, lsi, lsk, rsb, rsk, rsj;
    int M, K, N;
    int64_t tiles;         // B * ceil(M/32) * ceil(N/32)
    const int *run_flags;  // optional {a, b}: run only if a or b is non-zero (fallback after the tensor-core kernel)
};

// 32x32 output tile per 256-thread block, 4 outputs per thread, K in chunks of 32 through
// shared memory.  Per chunk: chunk maximum first, one rescale of the running sum, then one
// exp per term.  A row/column pair whose terms are all -inf yields -inf.
__global__ void __launch_bounds__(256) k_logmm_exact(const LogmmArgs a) {
    __shared__ float As[32][33];  // [i][k]
    __shared__ float Bs[32][33];  // [k][j]
    pdl_wait();
    if (a.run_flags != nullptr && a.run_flags[0] == 0 && a.run_flags[1] == 0) return;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // ty in [0,8)
    const float NINF = -__int_as_float(0x7f800000);
    const bool rhs_k_fast = (a.rsk == 1) || (a.rsj != 1);
    // tiles are dealt round-robin to the blocks of the grid (one tile per block for a stand-alone call;
    // a small grid when the kernel is only the stand-by behind the tensor-core kernel)
    const int tiles_j = (a.N + 31) / 32, tiles_i = (a.M + 31) / 32;
    for (int64_t tile = blockIdx.x; tile < a.tiles; tile += gridDim.x) {
    const int b = static_cast<int>(tile / (static_cast<int64_t>(tiles_i) * tiles_j));
    const int rest = static_cast<int>(tile - static_cast<int64_t>(b) * tiles_i * tiles_j);
    const int i0 = (rest / tiles_j) * 32, j0 = (rest % tiles_j) * 32;
    const float *lhs = a.lhs + b * a.lsb;
    const float *rhs = a.rhs + b * a.rsb;

    float m[4], s[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        m[r] = NINF;
        s[r] = 0.0f;
    }
    for (int k0 = 0; k0 < a.K; k0 += 32) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int ii = ty + 8 * r;
            const int gi = i0 + ii, gk = k0 + tx;
            As[ii][tx] = (gi < a.M && gk < a.K) ? __ldg(lhs + gi * a.lsi + gk * a.lsk) : NINF;
            if (rhs_k_fast) {  // tx runs along k
                const int gj = j0 + ii;
                Bs[tx][ii] = (gj < a.N && gk < a.K) ? __ldg(rhs + gk * a.rsk + gj * a.rsj) : NINF;
            } else {  // tx runs along j
                const int kk = k0 + ii, gj = j0 + tx;
                Bs[ii][tx] = (gj < a.N && kk < a.K) ? __ldg(rhs + kk * a.rsk + gj * a.rsj) : NINF;
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int ii = ty + 8 * r;
            float cm = NINF;
#pragma unroll 8
            for (int k = 0; k < 32; ++k) cm = fmaxf(cm, As[ii][k] + Bs[k][tx]);
            const float mn = fmaxf(m[r], cm);
            if (mn > NINF && mn < -NINF) {
                float acc = s[r] * ex2((m[r] - mn) * LOG2E);  // m == -inf -> s == 0 stays 0
                if (!(m[r] > NINF)) acc = 0.0f;
#pragma unroll 8
                for (int k = 0; k < 32; ++k) acc += ex2((As[ii][k] + Bs[k][tx] - mn) * LOG2E);
                s[r] = acc;
                m[r] = mn;
            } else if (mn == -NINF) {  // +inf term: result is +inf
                m[r] = mn;
                s[r] = 1.0f;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int gi = i0 + ty + 8 * r, gj = j0 + tx;
        if (gi < a.M && gj < a.N)
            a.out[(static_cast<int64_t>(b) * a.M + gi) * a.N + gj] = (m[r] > NINF) ? m[r] + lg2(s[r]) * LN2F : NINF;
    }
    __syncthreads();  // the shared tiles are reused by the next tile of this block
    }
}

// ---------------------------------------------------------------------------------------

struct ComposeArgs {
    const float *f;    // (N,T,V)
    const float *g;    // (N,U1,V)
    const float *den;  // (N,T,U1) or nullptr
    const int *ys, *lx, *ly;
    float *G;          // [N][T][U1][4] records {blank, repeat-label, next-label, 0}, log2 units
    int T, U1, V;
    int64_t total;     // N*T*U1*4
};

// One block per (utterance, 8 frames), one warp per frame, lanes over the contexts u.
// What a frame needs from f is one value per LABEL, not three per context: f[t, ys[u]] is the "next
// label" pick of context u and the "repeat" pick of context u+1, so each lane makes one isolated read
// and hands it to its neighbour by a shuffle; the picks of g do not depend on the frame at all and are
// staged once per block in shared memory (3 per context).  A third of the isolated reads of a
// thread-per-element gather.
constexpr int COMPOSE_FRAMES = 8;
__global__ void __launch_bounds__(256) k_simple_compose(const ComposeArgs a) {
    extern __shared__ float gp[];  // [U1][3] picks of g for this utterance, natural-log units
    pdl_wait();
    const int n = blockIdx.y;
    const int U1 = a.U1, U = U1 - 1;
    const int Tn = max(0, min(a.lx[n], a.T));
    const int Un = max(0, min(a.ly[n], U));
    const int *y = a.ys + static_cast<int64_t>(n) * U;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * COMPOSE_FRAMES + warp;
    float4 *Gs = reinterpret_cast<float4 *>(a.G) + (static_cast<int64_t>(n) * a.T + t) * U1;
    if (blockIdx.x * COMPOSE_FRAMES >= Tn) {  // nothing but padding frames in this block
        if (t < a.T)
            for (int u = lane; u < U1; u += 32) Gs[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        return;
    }
    for (int i = threadIdx.x; i < 3 * (Un + 1); i += 256) {
        const int u = i / 3, k = i - 3 * u;
        int idx = 0;
        if (k == 1 && u >= 1) idx = y[u - 1];
        if (k == 2 && u < Un) idx = y[u];
        idx = min(max(idx, 0), a.V - 1);
        gp[i] = __ldg(a.g + (static_cast<int64_t>(n) * U1 + u) * a.V + idx);
    }
    __syncthreads();
    if (t >= a.T) return;
    if (t >= Tn) {
        for (int u = lane; u < U1; u += 32) Gs[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        return;
    }
    const float *frow = a.f + (static_cast<int64_t>(n) * a.T + t) * a.V;
    const float *drow = a.den ? a.den + (static_cast<int64_t>(n) * a.T + t) * U1 : nullptr;
    const float fb = __ldg(frow);  // blank
    float carry = fb;              // f[t, ys[u-1]] of the first context of the next group of 32 (context 0: unused)
    for (int u0 = 0; u0 < U1; u0 += 32) {
        const int u = u0 + lane;
        // this lane's label pick: f[t, ys[u]] for u < Un (contexts at and beyond Un emit no next label)
        float fy = fb;
        if (u < Un) fy = load_sparse(frow + min(max(y[u], 0), a.V - 1));
        float fprev = __shfl_up_sync(0xffffffffu, fy, 1);
        if (lane == 0) fprev = carry;
        carry = __shfl_sync(0xffffffffu, fy, 31);
        if (u < U1) {
            float4 rec = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (u <= Un) {
                const float d = drow ? __ldg(drow + u) : 0.0f;
                // same float32 order as csrc/simple.cu:20-26: (f + g) - den
                float x0 = fb + gp[3 * u], x1 = ((u >= 1) ? fprev : fb) + gp[3 * u + 1], x2 = fy + gp[3 * u + 2];
                if (drow) {
                    x0 -= d;
                    x1 -= d;
                    x2 -= d;
                }
                rec = make_float4(to_log2(x0), to_log2(x1), to_log2(x2), 0.0f);
            }
            Gs[u] = rec;
        }
    }
}

// ---------------------------------------------------------------------------------------

struct LogmmBwdArgs {
    const float *lhs;       // (B,M,K) contiguous       [f]
    const float *rhsT;      // (B,Nc,K) contiguous      [g, i.e. rhs transposed]
    const float *res;       // (B,M,Nc) contiguous      [den]
    const float *gout;      // (B,M,Nc) contiguous, any sign; or nullptr with the fields below
    const float4 *grads3;   // [B][M][Nc] records {g0,g1,g2,0}: grad_out = -scale[b] * sum of the three slots
    const float *scale;     // [B]
    const int *lx, *ly;     // valid extents (rows < lx[b], columns <= ly[b]); nullptr = all valid
    float *grad_lhs;        // (B,M,K) or nullptr
    float *grad_rhsT;       // (B,Nc,K) or nullptr
    int M, Nc, K;
    int64_t items;          // B * ceil(K / VT), set by the launcher
    const int *run_flags;   // optional {a, b}: run only if a or b is non-zero (fallback after the tensor-core kernels)
};

// One thread per k (vocabulary entry), VT threads per block; the block walks all (i,j) of one
// batch entry.  grad_rhs is accumulated over i in shared memory ([Nc][VT]), grad_lhs over j
// in a register.  The rhs tile ([Nc][VT]) is cached in shared memory as well.
template <int VT>
__global__ void __launch_bounds__(VT) k_logmm_bwd_exact(const LogmmBwdArgs a) {
    extern __shared__ float sm[];
    pdl_wait();
    if (a.run_flags != nullptr && a.run_flags[0] == 0 && a.run_flags[1] == 0) return;
    // work items (batch entry, block of VT vocabulary entries) are dealt round-robin to the blocks
    const int kblocks = (a.K + VT - 1) / VT;
    for (int64_t work = blockIdx.x; work < a.items; work += gridDim.x) {
    const int b = static_cast<int>(work / kblocks);
    const int k = static_cast<int>(work - static_cast<int64_t>(b) * kblocks) * VT + threadIdx.x;
    const bool kin = k < a.K;
    float *gT = sm;                                   // [Nc][VT]  rhs tile in log2 units
    float *acc = sm + static_cast<size_t>(a.Nc) * VT;  // [Nc][VT]  grad_rhs accumulators
    float *wrow = acc + static_cast<size_t>(a.Nc) * VT;  // [Nc] weight row, [Nc] res row
    float *drow = wrow + a.Nc;
    const int Mv = a.lx ? max(0, min(a.lx[b], a.M)) : a.M;
    const int Nv = a.ly ? max(0, min(a.ly[b] + 1, a.Nc)) : a.Nc;
    for (int j = 0; j < a.Nc; ++j) {
        gT[j * VT + threadIdx.x] = kin ? __ldg(a.rhsT + (static_cast<int64_t>(b) * a.Nc + j) * a.K + k) * LOG2E : 0.0f;
        acc[j * VT + threadIdx.x] = 0.0f;
    }
    for (int i = 0; i < a.M; ++i) {
        const int64_t bi = static_cast<int64_t>(b) * a.M + i;
        float accF = 0.0f;
        if (i < Mv) {
            __syncthreads();
            for (int j = threadIdx.x; j < Nv; j += VT) {
                float w;
                if (a.gout) {
                    w = a.gout[bi * a.Nc + j];
                } else {
                    const float4 g3 = a.grads3[bi * a.Nc + j];
                    w = -a.scale[b] * (g3.x + g3.y + g3.z);
                }
                wrow[j] = w;
                drow[j] = a.res[bi * a.Nc + j] * LOG2E;
            }
            __syncthreads();
            const float fv = kin ? __ldg(a.lhs + bi * a.K + k) * LOG2E : 0.0f;
            for (int j = 0; j < Nv; ++j) {
                const float w = wrow[j];
                if (w != 0.0f) {
                    const float p = w * ex2(fv + gT[j * VT + threadIdx.x] - drow[j]);
                    accF += p;
                    acc[j * VT + threadIdx.x] += p;
                }
            }
        }
        if (a.grad_lhs && kin) a.grad_lhs[bi * a.K + k] = accF;
    }
    if (a.grad_rhsT && kin)
        for (int j = 0; j < a.Nc; ++j)
            a.grad_rhsT[(static_cast<int64_t>(b) * a.Nc + j) * a.K + k] = acc[j * VT + threadIdx.x];
    __syncthreads();  // the weight rows in shared memory are reused by the next work item
    }
}

// ---------------------------------------------------------------------------------------

struct PatchArgs {
    const float4 *grads3; // [N][T][U1] records {g0,g1,g2,0}
    const float *scale;   // [N]
    const int *ys, *lx, *ly;
    float *grad_f;        // (N,T,V) or nullptr
    float *grad_g;        // (N,U1,V) or nullptr
    int T, U1, V;
};

// grad_f[n,t,0] += sum_u g0;  grad_f[n,t,ys[j]] += g2[t,j] + g1[t,j+1].  One warp per (n,t): the
// blank column gets the warp's sum in one add instead of one atomic per context on the same
// address; labels may repeat inside an utterance, hence atomics for the label columns.
__device__ __forceinline__ void simple_patch_f_block(const PatchArgs &a, const int bx) {
    const int n = blockIdx.y;
    const int U = a.U1 - 1;
    const int t = bx * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int Tn = max(0, min(a.lx[n], a.T)), Un = max(0, min(a.ly[n], U));
    if (t >= Tn) return;
    const int64_t nt = static_cast<int64_t>(n) * a.T + t;
    const float4 *g3 = a.grads3 + nt * a.U1;
    const float sc = a.scale[n];
    float *row = a.grad_f + nt * a.V;
    const int *y = a.ys + static_cast<int64_t>(n) * U;
    float blank = 0.0f;
    for (int j = lane; j <= Un; j += 32) {
        const float4 cur = g3[j];
        blank += cur.x;
        if (j < Un) {
            const int v = min(max(y[j], 0), a.V - 1);
            atomicAdd(row + v, sc * (cur.z + g3[j + 1].y));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) blank += __shfl_xor_sync(0xffffffffu, blank, o);
    if (lane == 0) atomicAdd(row, sc * blank);  // a label equal to the blank index lands here too
}

__global__ void __launch_bounds__(256) k_simple_patch_f(const PatchArgs a) {
    pdl_wait();
    simple_patch_f_block(a, blockIdx.x);
}

// grad_g[n,u,{0, ys[u-1], ys[u]}] += sum_t of the three slots.  One block per (utterance, 32 contexts):
// lanes run along u, so that a warp reads 512 contiguous bytes of records per frame, the 8 warps
// take the frames round-robin, and their partial sums meet in shared memory (fixed order).
__device__ __forceinline__ void simple_patch_g_block(const PatchArgs &a, const int bx) {
    __shared__ float part[8][32][3];
    const int n = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int u = bx * 32 + lane;
    const int U = a.U1 - 1;
    const int Tn = max(0, min(a.lx[n], a.T)), Un = max(0, min(a.ly[n], U));
    if (bx * 32 > Un) return;
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f;
    if (u <= Un) {
        const float4 *g3 = a.grads3 + static_cast<int64_t>(n) * a.T * a.U1 + u;
        int t = warp;
        for (; t + 56 < Tn; t += 64) {  // eight independent loads in flight per lane
            float4 v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = g3[static_cast<int64_t>(t + 8 * k) * a.U1];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                s0 += v[k].x;
                s1 += v[k].y;
                s2 += v[k].z;
            }
        }
        for (; t < Tn; t += 8) {
            const float4 v = g3[static_cast<int64_t>(t) * a.U1];
            s0 += v.x;
            s1 += v.y;
            s2 += v.z;
        }
    }
    part[warp][lane][0] = s0;
    part[warp][lane][1] = s1;
    part[warp][lane][2] = s2;
    __syncthreads();
    if (warp == 0 && u <= Un) {
#pragma unroll
        for (int w = 1; w < 8; ++w) {
            s0 += part[w][lane][0];
            s1 += part[w][lane][1];
            s2 += part[w][lane][2];
        }
        const float sc = a.scale[n];
        float *row = a.grad_g + (static_cast<int64_t>(n) * a.U1 + u) * a.V;
        row[0] += sc * s0;
        if (u >= 1) row[min(max(a.ys[static_cast<int64_t>(n) * U + u - 1], 0), a.V - 1)] += sc * s1;
        if (u < Un) row[min(max(a.ys[static_cast<int64_t>(n) * U + u], 0), a.V - 1)] += sc * s2;
    }
}

__global__ void __launch_bounds__(256) k_simple_patch_g(const PatchArgs a, int N) {
    pdl_wait();
    simple_patch_g_block(a, blockIdx.x);
    (void)N;
}

// Both label patches in one launch: they write different tensors and need nothing of each other.  The first
// `g_blocks` blocks of a row of the grid take the (longer) sums over the frames for grad_g, the others the frames of
// grad_f, so that the two run side by side instead of one behind the other.
__global__ void __launch_bounds__(256) k_simple_patch_fg(const PatchArgs a, int g_blocks) {
    pdl_wait();
    if (static_cast<int>(blockIdx.x) < g_blocks)
        simple_patch_g_block(a, blockIdx.x);
    else
        simple_patch_f_block(a, blockIdx.x - g_blocks);
}

// ---------------------------------------------------------------------------------------
// Pre-gathered form, the reference's extension entry point ctct_loss_simple_fwd (csrc/binding.cpp:103-222):
// f (N,T,U1) already holds f[n,t,{0, ys[0], ..., ys[U-1]}], g (N,U1,3) the three picks per context.

struct GatheredArgs {
    const float *f;    // (N,T,U1)
    const float *g;    // (N,U1,3)
    const float *den;  // (N,T,U1) or nullptr
    const int *lx, *ly;
    float4 *G;         // [N][T][U1] records out (log2 units), 0 outside the valid region
    int T, U1;
    int64_t rows;      // N*T*U1
};

// log-prob of slot k at (n,t,u), csrc/simple.cu:20-26 (LOGPROBB, LOGPROBY): blank f[n,t,0] + g[n,u,0];
// repeat f[n,t,u] + g[n,u,1]; next f[n,t,u+1] + g[n,u,2]; each minus den[n,t,u] when normalised.
__global__ void __launch_bounds__(256) k_gathered_compose(const GatheredArgs a) {
    pdl_wait();
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < a.rows;
         r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t nt = r / a.U1;
        const int u = static_cast<int>(r - nt * a.U1);
        const int n = static_cast<int>(nt / a.T);
        const int t = static_cast<int>(nt - static_cast<int64_t>(n) * a.T);
        float4 rec = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (t < a.lx[n] && u <= a.ly[n]) {
            const float *fr = a.f + nt * a.U1;
            const float *gr = a.g + (static_cast<int64_t>(n) * a.U1 + u) * 3;
            const float d = a.den ? a.den[r] : 0.0f;
            float x0 = fr[0] + gr[0], x1 = fr[u] + gr[1], x2 = (u + 1 < a.U1) ? fr[u + 1] + gr[2] : 0.0f;
            if (a.den) {
                x0 -= d;
                x1 -= d;
                x2 -= d;
            }
            rec = make_float4(to_log2(x0), to_log2(x1), to_log2(x2), 0.0f);
        }
        a.G[r] = rec;
    }
}

struct GatheredReduceArgs {
    const float4 *grads3;  // [N][T][U1] {g0,g1,g2,0}
    const int *lx, *ly;
    float *grad_f;         // (N,T,U1)
    float *grad_g;         // (N,U1,3)
    float *grad_den;       // (N,T,U1) or nullptr
    int N, T, U1;
};

// The reductions of csrc/binding.cpp:198,209-219 for one frame per warp: grad_den = -(g0+g1+g2);
// grad_f[...,0] = sum_u g0; grad_f[...,k] = g1[k] + g2[k-1].  Fixed summation order.
__global__ void __launch_bounds__(256) k_gathered_reduce_t(const GatheredReduceArgs a) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t nt = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (nt >= static_cast<int64_t>(a.N) * a.T) return;
    const float4 *g3 = a.grads3 + nt * a.U1;
    float *gf = a.grad_f + nt * a.U1;
    float blank = 0.0f;
    for (int u = lane; u < a.U1; u += 32) {
        const float4 cur = g3[u];
        blank += cur.x;
        if (a.grad_den) a.grad_den[nt * a.U1 + u] = -(cur.x + cur.y + cur.z);
        if (u >= 1) gf[u] = cur.y + g3[u - 1].z;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) blank += __shfl_xor_sync(0xffffffffu, blank, o);
    if (lane == 0) gf[0] = blank;
}

// grad_g[n,u,k] = sum_t grads[n,t,u,k]: one warp per (n,u), fixed summation order.
__global__ void __launch_bounds__(256) k_gathered_reduce_u(const GatheredReduceArgs a) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (w >= static_cast<int64_t>(a.N) * a.U1) return;
    const int n = static_cast<int>(w / a.U1), u = static_cast<int>(w - static_cast<int64_t>(n) * a.U1);
    const int Tn = max(0, min(a.lx[n], a.T));
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f;
    if (u <= a.ly[n]) {
        for (int t = lane; t < Tn; t += 32) {
            const float4 g3 = a.grads3[(static_cast<int64_t>(n) * a.T + t) * a.U1 + u];
            s0 += g3.x;
            s1 += g3.y;
            s2 += g3.z;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane == 0) {
        float *o = a.grad_g + w * 3;
        o[0] = s0;
        o[1] = s1;
        o[2] = s2;
    }
}

}  // namespace ctct

// CTC-Transducer loss on RAW joint logits: log-softmax fused into both ends of the loss.
//
// The reference takes log-probabilities (warp_ctct/__init__.py:97-100), so its callers run
// log_softmax over the (N,T,U+1,V) joint tensor before the loss and log_softmax's backward after
// it: one more full read + write going in, two full reads + one write coming out, all around
// a gradient that is zero but for <= 3 columns per row.  Here
//
//  k_lse_gather  : ONE streaming read of the valid rows (t < lx, u <= ly) gives the row's
//                  log-sum-exp and the three log-probs the lattice needs (replaces log_softmax
//                  forward + the gather of warp_ctct/__init__.py:124-131);
//  k_logits_grad : ONE pass writes d loss / d logits = G - softmax(logits) * sum(G), where G is
//                  the <= 3-entry sparse row of the occupancy gradient: valid rows are read once
//                  and written once, padding rows are only written (zeros).  Replaces
//                  CTCTLoss.backward + the gather's scatter + log_softmax's backward.
//
// The log-sum-exp of a row travels from the first kernel to the second in the spare fourth word of
// the 16-byte records ({blank, repeat, next, lse} in G, {g0, g1, g2, lse} in the compact gradient),
// in log2 units, so the fused path needs no buffer the plain path does not have.
#pragma once

#include "common.cuh"
#include "grad.cuh"

namespace ctct {

// 16 bytes of the joint tensor <-> E floats
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
    static constexpr int E = 4;
    __device__ static void unpack(const uint4 &v, float (&x)[4]) {
        x[0] = __uint_as_float(v.x);
        x[1] = __uint_as_float(v.y);
        x[2] = __uint_as_float(v.z);
        x[3] = __uint_as_float(v.w);
    }
    __device__ static uint4 pack(const float (&x)[4]) {
        return make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3]));
    }
};
template <>
struct Vec16<__half> {
    static constexpr int E = 8;
    __device__ static void unpack(const uint4 &v, float (&x)[8]) {
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            x[2 * i] = f.x;
            x[2 * i + 1] = f.y;
        }
    }
    __device__ static uint4 pack(const float (&x)[8]) {
        unsigned w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
            w[i] = *reinterpret_cast<const unsigned *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <>
struct Vec16<__nv_bfloat16> {
    static constexpr int E = 8;
    __device__ static void unpack(const uint4 &v, float (&x)[8]) {
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // a bfloat16 is the upper half of a float32
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static uint4 pack(const float (&x)[8]) {
        unsigned w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            w[i] = *reinterpret_cast<const unsigned *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// streaming 16-byte read: the tensor is far larger than L2 and every row is read once per pass
__device__ __forceinline__ uint4 load_stream16(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

constexpr int LOGITS_BLOCKS_PER_SM = 4;  // resident blocks of 8 warps the two streaming kernels are built for
constexpr float LSE_FLOOR = -3.0e38f;  // finite start of a running maximum: no inf - inf anywhere

// running (maximum, sum of 2^(x - maximum)) of a set of log2-domain values; merging two such pairs
struct MaxSum {
    float m, s;
};
__device__ __forceinline__ MaxSum merge(const MaxSum a, const MaxSum b) {
    const float m = fmaxf(a.m, b.m);
    return MaxSum{m, a.s * ex2(a.m - m) + b.s * ex2(b.m - m)};
}

struct LseArgs {
    const void *logits;  // (N,T,U1,V)
    const int *ys, *lx, *ly;
    float4 *G;           // [N][T][U1] out: {blank, repeat-label, next-label, row lse}, log2 units; 0 outside the valid region
    int T, U1, V;
    int64_t rows;        // N*T*U1
    int vec;             // V is a multiple of the 16-byte vector width and the base is 16-byte aligned
};

// One warp per vocabulary row, rows dealt round-robin to the warps of a grid that fills the GPU
// once.  A lane has four independent 16-byte loads in flight (a whole 2 KB row per warp at
// the benchmark shapes) and keeps an online (max, sum) pair, so any V is one pass.
template <typename InT>
__global__ void __launch_bounds__(256, LOGITS_BLOCKS_PER_SM) k_lse_gather(const LseArgs a) {
    pdl_wait();
    pdl_trigger();
    constexpr int E = Vec16<InT>::E;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
    const int U = a.U1 - 1;
    const InT *base = static_cast<const InT *>(a.logits);
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); r < a.rows; r += nwarps) {
        const int64_t nt = r / a.U1;
        const int u = static_cast<int>(r - nt * a.U1);
        const int n = static_cast<int>(nt / a.T);
        const int t = static_cast<int>(nt - static_cast<int64_t>(n) * a.T);
        const int Un = min(a.ly[n], U);
        if (t >= a.lx[n] || u > Un) {
            if (lane == 0) a.G[r] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            continue;
        }
        const InT *row = base + r * a.V;
        // the three picked logits: lane 0 blank, lane 1 label u-1 (repeat), lane 2 label u (next)
        float pick = 0.0f;
        if (lane < 3) {
            int idx = 0;
            if (lane == 1 && u >= 1) idx = a.ys[static_cast<int64_t>(n) * U + (u - 1)];
            if (lane == 2 && u < Un) idx = a.ys[static_cast<int64_t>(n) * U + u];
            idx = min(max(idx, 0), a.V - 1);
            pick = load_as_float(row + idx);
        }
        MaxSum acc{LSE_FLOOR, 0.0f};
        if (a.vec) {
            const uint4 *rv = reinterpret_cast<const uint4 *>(row);
            const int nv = a.V / E;
            for (int j0 = lane; j0 < nv; j0 += 128) {
                uint4 v[4];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (j0 + 32 * k < nv) v[k] = load_stream16(rv + j0 + 32 * k);
                float x[4][E];
                float m = acc.m;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (j0 + 32 * k < nv) {
                        Vec16<InT>::unpack(v[k], x[k]);
#pragma unroll
                        for (int e = 0; e < E; ++e) {
                            x[k][e] *= LOG2E;
                            m = fmaxf(m, x[k][e]);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < E; ++e) x[k][e] = -__int_as_float(0x7f800000);  // contributes 2^-inf = 0
                    }
                }
                float s = acc.s * ex2(acc.m - m);
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                    for (int e = 0; e < E; ++e) s += ex2(x[k][e] - m);
                acc = MaxSum{m, s};
            }
        } else {
            for (int c = lane; c < a.V; c += 32) {
                const float x = load_as_float(row + c) * LOG2E;
                const float m = fmaxf(acc.m, x);
                acc = MaxSum{m, acc.s * ex2(acc.m - m) + ex2(x - m)};
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            MaxSum other;
            other.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
            other.s = __shfl_xor_sync(0xffffffffu, acc.s, o);
            acc = merge(acc, other);
        }
        // a row without a single finite logit has no softmax: every arc through it is forbidden
        const bool dead = !(acc.s > 0.0f);
        const float lse2 = dead ? 0.0f : acc.m + lg2(acc.s);
        const float val = dead ? NEG : fmaxf(pick * LOG2E - lse2, NEG);
        const float v1 = __shfl_sync(0xffffffffu, val, 1), v2 = __shfl_sync(0xffffffffu, val, 2);
        if (lane == 0) a.G[r] = make_float4(val, v1, v2, lse2);
    }
}

struct LogitsGradArgs {
    const void *logits;     // (N,T,U1,V)
    const float4 *GR;       // [N][T][U1] {g0, g1, g2, row lse in log2 units}
    const float *grad_out;  // [N], or one float when scalar_grad
    const int *ys, *lx, *ly;
    void *out;              // (N,T,U1,V), same element type as logits
    int T, U1, V;
    int vec;
    int scalar_grad;
    ReduceSpec red;
    int64_t rows;
};

// One warp per row again.  Padding rows are streamed out as zeros; a valid row is read once
// (four 16-byte loads per lane in flight), turned into -softmax * sum(G) in registers, gets its
// <= 3 sparse entries added by the lanes that own those columns, and is written once.
template <typename T>
__global__ void __launch_bounds__(256, LOGITS_BLOCKS_PER_SM) k_logits_grad(const LogitsGradArgs a) {
    pdl_wait();
    constexpr int E = Vec16<T>::E;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
    const int U = a.U1 - 1, V = a.V;
    const T *in = static_cast<const T *>(a.logits);
    T *outp = static_cast<T *>(a.out);
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); r < a.rows; r += nwarps) {
        const int64_t nt = r / a.U1;
        const int u = static_cast<int>(r - nt * a.U1);
        const int n = static_cast<int>(nt / a.T);
        const int t = static_cast<int>(nt - static_cast<int64_t>(n) * a.T);
        const int lx_n = a.lx[n];
        const int Un = min(a.ly[n], U);
        T *orow = outp + r * V;
        if (t >= lx_n || u > Un) {
            if (a.vec) {
                uint4 *dv = reinterpret_cast<uint4 *>(orow);
                for (int j = lane; j < V / E; j += 32) dv[j] = z;
            } else {
                const T zt = OutOps<T>::cvt(0.0f);
                for (int c = lane; c < V; c += 32) orow[c] = zt;
            }
            continue;
        }
        const float4 gr = a.GR[r];
        const float go = a.scalar_grad ? a.grad_out[0] * utterance_weight(a.red, lx_n) : a.grad_out[n];
        // sparse part: column 0 and the two label columns; coinciding columns add up
        float c0 = go * gr.x, c1 = 0.0f, c2 = 0.0f;
        int i1 = -1, i2 = -1;
        const int *y = a.ys + static_cast<int64_t>(n) * U;
        if (u >= 1) {
            i1 = min(max(y[u - 1], 0), V - 1);
            c1 = go * gr.y;
        }
        if (u < Un) {
            i2 = min(max(y[u], 0), V - 1);
            c2 = go * gr.z;
        }
        const float nsum = -(c0 + c1 + c2);  // minus the sum of the sparse row: weight of the softmax
        if (i1 == 0) {
            c0 += c1;
            i1 = -1;
        }
        if (i2 == 0) {
            c0 += c2;
            i2 = -1;
        }
        if (i1 >= 0 && i1 == i2) {
            c1 += c2;
            i2 = -1;
        }
        const float lse2 = gr.w;
        const T *row = in + r * V;
        if (a.vec) {
            const uint4 *rv = reinterpret_cast<const uint4 *>(row);
            uint4 *dv = reinterpret_cast<uint4 *>(orow);
            const int nv = V / E;
            const int j1 = i1 >= 0 ? i1 / E : -1, j2 = i2 >= 0 ? i2 / E : -1;
            for (int j0 = lane; j0 < nv; j0 += 128) {
                uint4 v[4];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (j0 + 32 * k < nv) v[k] = load_stream16(rv + j0 + 32 * k);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int j = j0 + 32 * k;
                    if (j < nv) {
                        float x[E];
                        Vec16<T>::unpack(v[k], x);
#pragma unroll
                        for (int e = 0; e < E; ++e) x[e] = ex2(fmaf(x[e], LOG2E, -lse2)) * nsum;
                        if (j == 0 || j == j1 || j == j2) {
#pragma unroll
                            for (int e = 0; e < E; ++e) {
                                const int col = j * E + e;
                                if (col == 0) x[e] += c0;
                                if (col == i1) x[e] += c1;
                                if (col == i2) x[e] += c2;
                            }
                        }
                        dv[j] = Vec16<T>::pack(x);
                    }
                }
            }
        } else {
            for (int c = lane; c < V; c += 32) {
                float x = ex2(fmaf(load_as_float(row + c), LOG2E, -lse2)) * nsum;
                if (c == 0) x += c0;
                if (c == i1) x += c1;
                if (c == i2) x += c2;
                orow[c] = OutOps<T>::cvt(x);
            }
        }
    }
}

}  // namespace ctct

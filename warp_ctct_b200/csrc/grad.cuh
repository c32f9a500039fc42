// Gradient kernels.
//
//  k_fill_grad    : occupancy gradient w.r.t. the three gathered log-probs of every (n,t,u),
//                   the quantity the reference's k_fill_grad produces (csrc/gather.cu:311-374),
//                   evaluated from the normalised tables of lattice.cuh.
//  k_dense_grad   : the dense (N,T,U+1,V) gradient in ONE pass, every byte written once with
//                   16-byte stores: zeros everywhere except <= 3 columns per row, which are
//                   patched in registers before the store.
//                   Replaces what autograd does for the reference after CTCTLoss.backward
//                   (warp_ctct/__init__.py:31-33): a multiply, a cast, a memset of the full tensor
//                   and a scatter_add.
//  k_export_tables: test hook, tables in natural-log units and unshifted coordinates.
#pragma once

#include "common.cuh"

namespace ctct {

// occupancies of the arcs leaving context u at frame t: {blank, repeat label, next label}
__device__ __forceinline__ float3 occupancies(const float4 *__restrict__ G, const float4 *__restrict__ TAB,
                                              const int *__restrict__ y, int64_t nt, int u, int U1, int Un, float lf,
                                              int li) {
    // table record of a context: {label-state value, offset, blank-state value, offset}
    const float4 p = G[nt * U1 + u];
    const float4 av = TAB[(nt * 2 + 0) * U1 + u];
    const float4 bv = TAB[(nt * 2 + 1) * U1 + u];
    const float aL = av.x, aB = av.z, bL = bv.x, bB = bv.z;
    // the blank slot of a live context is always written; a label slot shares its warp (and so
    // its offset) whenever it exists
    const int oA = __float_as_int(av.w);
    const float c_same = static_cast<float>(oA + __float_as_int(bv.w) - li) - lf;
    // arcs leaving the blank state 2u: stay (blank), or emit label u
    float occ0 = ex2(aB + bB + p.x + c_same);
    float occ1 = 0.0f, occ2 = 0.0f;
    if (u >= 1) {
        // arcs leaving the label state 2u-1: to blank 2u, stay (repeat label u-1)
        occ0 += ex2(aL + bB + p.x + c_same);
        occ1 = ex2(aL + bL + p.y + c_same);
    }
    if (u < Un) {
        const float4 bn = TAB[(nt * 2 + 1) * U1 + u + 1];
        const float c_next = static_cast<float>(oA + __float_as_int(bn.y) - li) - lf;
        occ2 = ex2(aB + bn.x + p.z + c_next);
        if (u >= 1 && y[u] != y[u - 1]) occ2 += ex2(aL + bn.x + p.z + c_next);
    }
    return make_float3(occ0, occ1, occ2);
}

// How per-utterance costs are folded into one scalar (warp_ctct/__init__.py:138-147):
// loss = sum_n costs[n] * w[n], w[n] = (average_frames ? 1/lx[n] : 1) * (mean ? 1/norm : 1).
struct ReduceSpec {
    int reduction;       // 0 none, 1 sum, 2 mean
    int average_frames;  // divide each cost by its number of frames first
    float norm;          // divisor of 'mean' (the global batch size)
};

__device__ __forceinline__ float utterance_weight(const ReduceSpec &r, int lx_n) {
    float w = 1.0f;
    if (r.average_frames) w = 1.0f / static_cast<float>(lx_n);
    if (r.reduction == 2) w = w / r.norm;
    return w;
}

// Deterministic block-wide reduction of the costs (fixed order: strided partial sums, shuffle
// tree, then the warps in order).  Called by one whole block of 256 threads.
__device__ __forceinline__ void reduce_costs_block(const float *__restrict__ costs, const int *__restrict__ lx, int N,
                                                   const ReduceSpec r, float *__restrict__ loss_out) {
    __shared__ float part[8];
    float acc = 0.0f;
    for (int n = threadIdx.x; n < N; n += 256) {
        float c = costs[n];
        if (r.average_frames) c = c / static_cast<float>(lx[n]);
        acc += c;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.0f;
        for (int w = 0; w < 8; ++w) tot += part[w];
        if (r.reduction == 2) tot = tot / r.norm;
        *loss_out = tot;
    }
}

__global__ void __launch_bounds__(256) k_reduce_costs(const float *costs, const int *lx, int N, const ReduceSpec r,
                                                      float *loss_out) {
    reduce_costs_block(costs, lx, N, r, loss_out);
}

struct GradArgs {
    const float4 *G;    // [N][T][U1], log2 units
    const float4 *TAB;  // [N][T][2][U1]
    const float *llf;   // [N][2]
    const int *lli;     // [N][2]
    const int *ys, *lx, *ly;
    float *out;         // internal [N][T][U1] float4 {g0,g1,g2,w} or reference [N][T][U1][3]
    int T, U1;
    int ref_layout;
    int keep_w;         // internal layout: copy the fourth word of the G record (a row's log-sum-exp) into w, else w = 0
    // optional fused reduction of the costs (done by block 0); loss_out == nullptr: none
    const float *costs;
    float *loss_out;
    int N;
    ReduceSpec red;
    int64_t frames;     // N * T: own blocks = ceil(frames / 8), one warp per frame
    ClearSlice clear;
};

// One warp per frame (n,t); lanes stride over the contexts u.  Every arc (state at t) -> (state at
// t+1) contributes exp2(alpha + logp + beta - loglik); arcs outside the band contribute an exact 0
// because one of the two variables is "impossible" there, so the reference's band guards
// (gather.cu:335-337,355-359) need no restating.
//
// Exactly one arc leaves every frame on every alignment, so the occupancies of a frame sum to one.
// The warp divides by the sum it actually gets: what alpha, beta and the log-likelihood have each
// accumulated in approximation error over up to T recursion steps is common to all arcs of the frame
// and cancels, which leaves the relative error of single terms (~1e-6) instead of ~1e-7 per step
// times T.  The first FG_KEEP * 32 contexts stay in registers between the two passes; beyond that
// (U+1 > 128) the occupancies are evaluated a second time from L1/L2.
constexpr int FG_KEEP = 4;
__global__ void __launch_bounds__(256) k_fill_grad(const GradArgs a) {
    pdl_wait();
    if (clear_role(a.clear, nullptr, 0)) return;
    if (a.loss_out != nullptr && blockIdx.x == 0) reduce_costs_block(a.costs, a.lx, a.N, a.red, a.loss_out);
    const int lane = threadIdx.x & 31;
    const int64_t nt = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (nt >= a.frames) return;
    const int n = static_cast<int>(nt / a.T);
    const int t = static_cast<int>(nt - static_cast<int64_t>(n) * a.T);
    const int U1 = a.U1, U = U1 - 1;
    const int Tn = max(0, min(a.lx[n], a.T));
    const int Un = max(0, min(a.ly[n], U));
    const float lf = a.llf[n * 2 + 1];
    const bool live = t < Tn && lf > NEG_TEST;
    const int li = a.lli[n * 2 + 1];
    const int *y = a.ys + static_cast<int64_t>(n) * U;

    float3 keep[FG_KEEP];
    float z = 0.0f;
    if (live) {
#pragma unroll
        for (int i = 0; i < FG_KEEP; ++i) {
            const int u = lane + 32 * i;
            keep[i] = make_float3(0.0f, 0.0f, 0.0f);
            if (u <= Un) {
                keep[i] = occupancies(a.G, a.TAB, y, nt, u, U1, Un, lf, li);
                z += keep[i].x + keep[i].y + keep[i].z;
            }
        }
        for (int u = lane + 32 * FG_KEEP; u <= Un; u += 32) {
            const float3 o = occupancies(a.G, a.TAB, y, nt, u, U1, Un, lf, li);
            z += o.x + o.y + o.z;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    }
    const float inv = (z > 0.0f) ? -1.0f / z : -1.0f;  // gradient of the cost: minus the occupancy

    auto put = [&](int u, float3 o) {
        const float3 g = make_float3(o.x * inv, o.y * inv, o.z * inv);
        if (a.ref_layout) {
            float *p = a.out + (nt * U1 + u) * 3;
            p[0] = g.x;
            p[1] = g.y;
            p[2] = g.z;
        } else {
            const float w = (a.keep_w && live && u <= Un) ? a.G[nt * U1 + u].w : 0.0f;
            reinterpret_cast<float4 *>(a.out)[nt * U1 + u] = make_float4(g.x, g.y, g.z, w);
        }
    };
#pragma unroll
    for (int i = 0; i < FG_KEEP; ++i) {
        const int u = lane + 32 * i;
        if (u < U1) put(u, (live && u <= Un) ? keep[i] : make_float3(0.0f, 0.0f, 0.0f));
    }
    for (int u = lane + 32 * FG_KEEP; u < U1; u += 32)
        put(u, (live && u <= Un) ? occupancies(a.G, a.TAB, y, nt, u, U1, Un, lf, li) : make_float3(0.0f, 0.0f, 0.0f));
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
};
template <>
struct OutOps<__half> {
    static constexpr int E = 8;
    __device__ static __half cvt(float x) { return __float2half_rn(x); }
    __device__ static __half add(__half a, __half b) { return __hadd(a, b); }
};
template <>
struct OutOps<__nv_bfloat16> {
    static constexpr int E = 8;
    __device__ static __nv_bfloat16 cvt(float x) { return __float2bfloat16_rn(x); }
    __device__ static __nv_bfloat16 add(__nv_bfloat16 a, __nv_bfloat16 b) { return __hadd(a, b); }
};

struct DenseArgs {
    const float4 *GR;       // [N][T][U1] compact gradient {g0,g1,g2,0}
    const float *grad_out;  // [N]
    const int *ys, *lx, *ly;
    void *out;              // [N][T][U1][V]
    int T, U1, V;
    int vec;                // 1: V is a multiple of the 16-byte vector width and the base is 16-byte aligned
    // scalar_grad != 0: grad_out is ONE float (gradient of the reduced loss) and the per-utterance
    // scale is grad_out[0] * utterance_weight(red, lx[n]); otherwise grad_out holds N floats
    int scalar_grad;
    ReduceSpec red;
    const int64_t *cu;      // packed output: row offsets per utterance (N+1), nullptr = padded (N,T,U1,V)
    int64_t packed_rows;    // rows of the packed output (rows beyond it are never written)
};

// Row offsets of the packed layout: cu[n] = sum_{m<n} lx[m] * (ly[m] + 1), cu[N] = total rows.
// One block; N <= 65535.  Every thread sums a run of utterances, the 1024 run totals are scanned with
// shuffles (inside the warps, then over the 32 warp totals), and every thread writes its run.
__global__ void __launch_bounds__(1024) k_packed_offsets(const int *__restrict__ lx, const int *__restrict__ ly, int N, int T,
                                                         int U1, int64_t *__restrict__ cu) {
    __shared__ long long warp_total[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = (N + 1023) / 1024;
    const int lo = threadIdx.x * per, hi = min(N, lo + per);
    auto rows_of = [&](int n) {
        return static_cast<long long>(max(0, min(lx[n], T))) * (max(0, min(ly[n], U1 - 1)) + 1);
    };
    long long s = 0;
    for (int n = lo; n < hi; ++n) s += rows_of(n);
    long long incl = s;  // inclusive scan of the run totals inside the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const long long v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) warp_total[warp] = incl;
    __syncthreads();
    if (warp == 0) {  // exclusive scan of the warp totals; lane 31 ends up with the grand total
        const long long w = warp_total[lane];
        long long wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long v = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += v;
        }
        warp_total[lane] = wi - w;
        if (lane == 31) cu[N] = wi;
    }
    __syncthreads();
    long long run = warp_total[warp] + incl - s;
    for (int n = lo; n < hi; ++n) {
        cu[n] = run;
        run += rows_of(n);
    }
}

// What one row of the dense gradient holds besides zeros: column 0 and up to two label columns.
template <typename OutT>
struct RowPatch {
    OutT c0, c1, c2;
    int i1, i2;  // label columns, -1 when absent (or merged into an earlier column)
};

// Columns that coincide add up in slot order, each product rounded to OutT first -- what a
// cast followed by scatter_add onto zeros produces.
template <typename OutT>
__device__ __forceinline__ RowPatch<OutT> make_patch(const float4 g, float go, int y_prev, int y_next, int u, int Un,
                                                     int V) {
    using O = OutOps<OutT>;
    RowPatch<OutT> p;
    const OutT zero = O::cvt(0.0f);
    p.c0 = O::add(zero, O::cvt(go * g.x));
    p.c1 = zero;
    p.c2 = zero;
    p.i1 = -1;
    p.i2 = -1;
    if (u >= 1) {
        p.i1 = min(max(y_prev, 0), V - 1);
        p.c1 = O::add(zero, O::cvt(go * g.y));
    }
    if (u < Un) {
        p.i2 = min(max(y_next, 0), V - 1);
        p.c2 = O::add(zero, O::cvt(go * g.z));
    }
    if (p.i1 == 0) {
        p.c0 = O::add(p.c0, p.c1);
        p.i1 = -1;
    }
    if (p.i2 == 0) {
        p.c0 = O::add(p.c0, p.c2);
        p.i2 = -1;
    }
    if (p.i1 >= 0 && p.i1 == p.i2) {
        p.c1 = O::add(p.c1, p.c2);
        p.i2 = -1;
    }
    return p;
}

template <typename OutT>
__device__ __forceinline__ unsigned out_bits(OutT x);
template <>
__device__ __forceinline__ unsigned out_bits<float>(float x) { return __float_as_uint(x); }
template <>
__device__ __forceinline__ unsigned out_bits<__half>(__half x) { return __half_as_ushort(x); }
template <>
__device__ __forceinline__ unsigned out_bits<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat16_as_ushort(x); }

// One CTA per (n,t) slab of U1 rows; inside, one warp per row (rows dealt round-robin to the 8
// warps), lanes stride over the row in 16-byte vectors.  A lane patches the non-zero columns
// in its own registers before the store, so every byte is written exactly once and nothing
// waits on anything: the only loads are one 16-byte record and two labels per row, issued one
// row ahead.  Many short CTAs (not a persistent grid) is what reaches the HBM write peak here.
template <typename OutT>
__global__ void __launch_bounds__(256) k_dense_grad(const DenseArgs a) {
    constexpr int E = OutOps<OutT>::E;
    const int64_t slab = blockIdx.x;  // = n*T + t
    const int n = static_cast<int>(slab / a.T);
    const int t = static_cast<int>(slab - static_cast<int64_t>(n) * a.T);
    const int U = a.U1 - 1, V = a.V;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    OutT *base = static_cast<OutT *>(a.out) + slab * static_cast<int64_t>(a.U1) * V;
    const int *y = a.ys + static_cast<int64_t>(n) * U;
    const float4 *gr = a.GR + slab * a.U1;
    // Everything the first row needs is requested at once, whether or not it turns out to be
    // needed (all addresses are inside the buffers), so that the CTA pays one memory latency
    // before its first store, not a chain of them.
    const int lx_n = a.lx[n], ly_n = a.ly[n];
    const float go_raw = a.scalar_grad ? a.grad_out[0] : a.grad_out[n];
    float4 g_next = gr[min(warp, U)];
    int yp_next = (U > 0) ? y[min(max(warp - 1, 0), U - 1)] : 0;
    int yn_next = (U > 0) ? y[min(warp, U - 1)] : 0;
    const int Tn = min(lx_n, a.T);
    const int Un = (t < Tn) ? min(ly_n, U) : -1;  // rows u <= Un carry values
    const float go = a.scalar_grad ? go_raw * utterance_weight(a.red, lx_n) : go_raw;

    for (int u = warp; u < a.U1; u += 8) {
        const float4 g = g_next;
        const int y_prev = yp_next, y_nxt = yn_next;
        if (u + 8 <= Un) {  // one row ahead
            g_next = gr[u + 8];
            yp_next = y[u + 7];
            if (u + 8 < Un) yn_next = y[u + 8];
        }
        OutT *row = base + static_cast<int64_t>(u) * V;
        if (u > Un) {  // padding row
            if (a.vec) {
                uint4 *dv = reinterpret_cast<uint4 *>(row);
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                for (int j = lane; j < V / E; j += 32) dv[j] = z;
            } else {
                const OutT z = OutOps<OutT>::cvt(0.0f);
                for (int c = lane; c < V; c += 32) row[c] = z;
            }
            continue;
        }
        const RowPatch<OutT> p = make_patch<OutT>(g, go, y_prev, y_nxt, u, Un, V);
        if (a.vec) {
            uint4 *dv = reinterpret_cast<uint4 *>(row);
            const int j1 = p.i1 >= 0 ? p.i1 / E : -1, j2 = p.i2 >= 0 ? p.i2 / E : -1;
            for (int j = lane; j < V / E; j += 32) {
                uint4 w = make_uint4(0u, 0u, 0u, 0u);
                if (j == 0 || j == j1 || j == j2) {
                    unsigned b[E];
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        const int col = j * E + e;
                        OutT x = OutOps<OutT>::cvt(0.0f);
                        if (col == 0) x = p.c0;
                        if (col == p.i1) x = p.c1;
                        if (col == p.i2) x = p.c2;
                        b[e] = out_bits<OutT>(x);
                    }
                    if constexpr (E == 4) {
                        w = make_uint4(b[0], b[1], b[2], b[3]);
                    } else {
                        w = make_uint4(b[0] | (b[1] << 16), b[2] | (b[3] << 16), b[4] | (b[5] << 16), b[6] | (b[7] << 16));
                    }
                }
                dv[j] = w;
            }
        } else {
            for (int c = lane; c < V; c += 32) {
                OutT x = OutOps<OutT>::cvt(0.0f);
                if (c == 0) x = p.c0;
                if (c == p.i1) x = p.c1;
                if (c == p.i2) x = p.c2;
                row[c] = x;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Two-step alternative to k_dense_grad, for callers that can start clearing the gradient buffer
// before the gradient scale is known (e.g. on a second stream while the lattice runs):
// k_zero_fill streams zeros, k_dense_patch later writes the <= 3 non-zero columns of every live row.

// Each block clears one contiguous chunk of 1024 16-byte vectors (4 per thread, strided by the
// block): many short blocks reach the HBM write peak, a persistent grid does not.
__global__ void __launch_bounds__(256) k_zero_fill(uint4 *__restrict__ out, size_t nvec, unsigned char *__restrict__ tail,
                                                   int tail_bytes) {
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    const size_t base = static_cast<size_t>(blockIdx.x) * 1024;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const size_t v = base + i * 256 + threadIdx.x;
        if (v < nvec) out[v] = z;
    }
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < tail_bytes) tail[threadIdx.x] = 0;
}

// One whole 32-byte sector of a row in registers: zeros except the patched columns that fall into it.
// Whole-sector writes need no read of the old contents, so patching costs DRAM writes only.
// A sector is built from zeros by dropping each value into its position (one compare and one
// predicated move per position), not by comparing every column with every patch.
template <typename OutT>
struct SectorWords {
    static constexpr int ES = 2 * OutOps<OutT>::E;                    // elements per sector
    static constexpr int PER_WORD = 4 / static_cast<int>(sizeof(OutT));  // elements per 32-bit word
    unsigned w[8];
    __device__ __forceinline__ void clear() {
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = 0u;
    }
    // element `pos` (0 <= pos < ES) of the sector becomes x; an earlier value at the same position is replaced
    __device__ __forceinline__ void put(int pos, OutT x) {
        const unsigned bits = out_bits<OutT>(x);
        if constexpr (PER_WORD == 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (pos == i) w[i] = bits;
        } else {
            const int word = pos >> 1;
            const unsigned shift = (pos & 1) * 16u;
            const unsigned keep = ~(0xffffu << shift), val = bits << shift;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (word == i) w[i] = (w[i] & keep) | val;
        }
    }
    __device__ __forceinline__ void store(OutT *row, int sector) const {
        uint4 *dst = reinterpret_cast<uint4 *>(row) + sector * 2;
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
};

// The <= 3 sectors of a row that hold non-zero columns: sector 0 (column 0, plus a label column below
// the sector width) and the sectors of the two label columns.
template <typename OutT>
__device__ __forceinline__ void write_row_sectors(OutT *row, const RowPatch<OutT> &p) {
    constexpr int ES = SectorWords<OutT>::ES;
    const int s1 = p.i1 >= 0 ? p.i1 / ES : 0, s2 = p.i2 >= 0 ? p.i2 / ES : 0;
    SectorWords<OutT> sec;
    sec.clear();
    sec.put(0, p.c0);
    if (p.i1 >= 0 && s1 == 0) sec.put(p.i1, p.c1);
    if (p.i2 >= 0 && s2 == 0) sec.put(p.i2, p.c2);
    sec.store(row, 0);
    if (s1 != 0) {
        sec.clear();
        sec.put(p.i1 - s1 * ES, p.c1);
        if (s2 == s1) sec.put(p.i2 - s2 * ES, p.c2);
        sec.store(row, s1);
    }
    if (s2 != 0 && s2 != s1) {
        sec.clear();
        sec.put(p.i2 - s2 * ES, p.c2);
        sec.store(row, s2);
    }
}

// One thread per (n,t,u) row; rows outside t < lx, u <= ly stay zero.  SECTORS: rows start on
// 32-byte boundaries and V is a multiple of the sector width.
template <typename OutT, bool SECTORS>
__global__ void __launch_bounds__(256) k_dense_patch(const DenseArgs a, int64_t rows) {
    pdl_wait();
    const int U = a.U1 - 1, V = a.V;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < rows;
         r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t nt = r / a.U1;
        const int u = static_cast<int>(r - nt * a.U1);
        const int n = static_cast<int>(nt / a.T);
        const int t = static_cast<int>(nt - static_cast<int64_t>(n) * a.T);
        const int lx_n = a.lx[n];
        const int Un = min(a.ly[n], U);
        if (t >= min(lx_n, a.T) || u > Un) continue;
        const float go = a.scalar_grad ? a.grad_out[0] * utterance_weight(a.red, lx_n) : a.grad_out[n];
        const int *y = a.ys + static_cast<int64_t>(n) * U;
        const int y_prev = (u >= 1) ? y[u - 1] : 0;
        const int y_next = (u < Un) ? y[u] : 0;
        const RowPatch<OutT> p = make_patch<OutT>(a.GR[r], go, y_prev, y_next, u, Un, V);
        const int64_t r_out = a.cu ? a.cu[n] + static_cast<int64_t>(t) * (Un + 1) + u : r;
        if (a.cu && r_out >= a.packed_rows) continue;
        OutT *row = static_cast<OutT *>(a.out) + r_out * V;
        if (SECTORS) {
            write_row_sectors<OutT>(row, p);
        } else {
            row[0] = p.c0;
            if (p.i1 >= 0) row[p.i1] = p.c1;
            if (p.i2 >= 0) row[p.i2] = p.c2;
        }
    }
}

// ---------------------------------------------------------------------------------------
// test hook

struct ExportArgs {
    const float4 *TAB;
    const float *llf;
    const int *lli;
    const int *lx, *ly;
    double *alpha, *beta_next, *ll_alpha, *ll_beta;
    int T, U1;
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
    const int u = (s + 1) / 2;
    const bool blank = (s & 1) == 0;
    const int Tn = max(0, min(a.lx[n], a.T)), Un = max(0, min(a.ly[n], U));
    const int64_t nt = static_cast<int64_t>(n) * a.T + t;
    double va = ninf, vb = ninf;
    if (t < Tn && u <= Un) {
        const float4 av = a.TAB[(nt * 2 + 0) * a.U1 + u], bv = a.TAB[(nt * 2 + 1) * a.U1 + u];
        const float x = blank ? av.z : av.x, y = blank ? bv.z : bv.x;
        if (x > NEG_TEST) va = (static_cast<double>(__float_as_int(blank ? av.w : av.y)) + x) * LN2;
        if (y > NEG_TEST) vb = (static_cast<double>(__float_as_int(blank ? bv.w : bv.y)) + y) * LN2;
    }
    a.alpha[nt * S + s] = va;
    a.beta_next[nt * S + s] = vb;
}

}  // namespace ctct

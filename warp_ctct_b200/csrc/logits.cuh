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
constexpr float LSE_FLOOR = -1.0e30f;  // finite start of a running maximum (and finite when scaled by log2 e): no inf - inf anywhere

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
    const int64_t *cu;   // packed logits (total valid rows, V): row offsets per utterance; nullptr = padded
    int64_t packed_rows; // rows of the packed tensor (slabs reaching beyond it are treated as padding)
};

// One CTA per (n,t) slab of U1 rows (a contiguous U1*V block of the tensor), one warp per row, rows
// dealt round-robin to the 8 warps: the only division is one per CTA.  Slabs t >= lx[n] only write
// their (zero) records.
//
// A row reaches its warp through a warp-private ring of LSE_DEPTH 2 KB slots in shared memory filled
// with cp.async (16 bytes per lane and copy, no registers held while the data is on its way): a
// warp has LSE_DEPTH - 1 chunks (4 KB) in flight while it reduces the chunk before them, 128 KB per
// SM with four CTAs resident.  Every lane reads back exactly the 16-byte pieces it copied itself, so the
// ring needs no barrier, only cp.async.wait_group.  A lane keeps an online (max, sum) pair, so a
// row of any length is one pass over its chunks.
constexpr int LSE_DEPTH = 3;
constexpr int LSE_CHUNK_VECS = 128;                                        // 16-byte vectors per ring slot (4 per lane)
constexpr int LSE_SMEM_BYTES = 8 * LSE_DEPTH * LSE_CHUNK_VECS * 16;        // 48 KB per CTA

template <typename InT>
__global__ void __launch_bounds__(256, LOGITS_BLOCKS_PER_SM) k_lse_gather(const LseArgs a) {
    extern __shared__ __align__(16) uint4 lse_ring[];
    pdl_wait();
    pdl_trigger();
    constexpr int E = Vec16<InT>::E;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t nt = blockIdx.x;
    const int n = static_cast<int>(nt / a.T);
    const int t = static_cast<int>(nt - static_cast<int64_t>(n) * a.T);
    const int U1 = a.U1, U = U1 - 1;
    int Un = (t < a.lx[n]) ? min(a.ly[n], U) : -1;  // rows u <= Un are read
    if (a.cu && Un >= 0 && a.cu[n] + static_cast<int64_t>(t + 1) * (Un + 1) > a.packed_rows) Un = -1;
    float4 *Gs = a.G + nt * U1;
    // records of the padding rows
    for (int u = Un + 1 + static_cast<int>(threadIdx.x); u < U1; u += 256) Gs[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const int64_t slab_row = a.cu ? a.cu[n] + static_cast<int64_t>(t) * (Un + 1) : nt * U1;
    const InT *slab = static_cast<const InT *>(a.logits) + slab_row * a.V;
    const int *y = a.ys + static_cast<int64_t>(n) * U;
    const float NINF = -__int_as_float(0x7f800000);

    auto finish_row = [&](int u, MaxSum acc, float pick) {
        // warp-wide maximum first, then one rescale per lane and a plain sum
        float m_all = acc.m;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
        float s_all = acc.s * ex2(acc.m - m_all);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s_all += __shfl_xor_sync(0xffffffffu, s_all, o);
        // a row without a single finite logit has no softmax: every arc through it is forbidden
        const bool dead = !(s_all > 0.0f);
        const float lse2 = dead ? 0.0f : m_all + lg2(s_all);
        const float val = dead ? NEG : fmaxf(pick * LOG2E - lse2, NEG);
        const float v1 = __shfl_sync(0xffffffffu, val, 1), v2 = __shfl_sync(0xffffffffu, val, 2);
        if (lane == 0) Gs[u] = make_float4(val, v1, v2, lse2);
    };
    // the three picked logits of row u: lane 0 blank, lane 1 label u-1 (repeat), lane 2 label u (next)
    auto load_pick = [&](int u) {
        float pick = 0.0f;
        if (lane < 3) {
            int idx = 0;
            if (lane == 1 && u >= 1) idx = y[u - 1];
            if (lane == 2 && u < Un) idx = y[u];
            idx = min(max(idx, 0), a.V - 1);
            pick = load_as_float(slab + static_cast<int64_t>(u) * a.V + idx);
        }
        return pick;
    };

    if (!a.vec) {  // rows that are not whole 16-byte vectors: plain loads
        for (int u = warp; u <= Un; u += 8) {
            const InT *row = slab + static_cast<int64_t>(u) * a.V;
            const float pick = load_pick(u);
            MaxSum acc{LSE_FLOOR, 0.0f};
            for (int c = lane; c < a.V; c += 32) {
                const float x = load_as_float(row + c) * LOG2E;
                const float m = fmaxf(acc.m, x);
                acc = MaxSum{m, acc.s * ex2(acc.m - m) + ex2(x - m)};
            }
            finish_row(u, acc, pick);
        }
        return;
    }

    // The kernel is held back by instruction issue as soon as the per-row bookkeeping costs as much as
    // the 3 instructions per element the sum itself needs (multiply-add, ex2, add), so both sides of the
    // ring keep running pointers and counters instead of dividing, and whole chunks skip the bounds checks.
    uint4 *ring = lse_ring + warp * (LSE_DEPTH * LSE_CHUNK_VECS) + lane;
    const int nv = a.V / E;                                         // vectors per row
    const int nch = (nv + LSE_CHUNK_VECS - 1) / LSE_CHUNK_VECS;     // chunks per row
    const int rows_w = (Un >= warp) ? (Un - warp) / 8 + 1 : 0;      // rows of this warp
    const int units = rows_w * nch;
    const int64_t next_row = static_cast<int64_t>(8) * nv - static_cast<int64_t>(nch - 1) * LSE_CHUNK_VECS;
    // producer side
    const uint4 *src = reinterpret_cast<const uint4 *>(slab + static_cast<int64_t>(warp) * a.V) + lane;
    int p_unit = 0, p_c = 0, p_slot = 0;
    auto issue = [&]() {
        if (p_unit < units) {
            uint4 *dst = ring + p_slot * LSE_CHUNK_VECS;
            const int left = nv - p_c * LSE_CHUNK_VECS - lane;   // vectors of this chunk from this lane's first on
            if (left > 96) {
#pragma unroll
                for (int k = 0; k < 4; ++k) cp_async16(dst + 32 * k, src + 32 * k);
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (32 * k < left) cp_async16(dst + 32 * k, src + 32 * k);
            }
            ++p_unit;
            if (++p_c == nch) {
                p_c = 0;
                src += next_row;
            } else {
                src += LSE_CHUNK_VECS;
            }
        }
        cp_async_commit();  // an empty group keeps the group count in step
        p_slot = (p_slot + 1 == LSE_DEPTH) ? 0 : p_slot + 1;
    };
#pragma unroll
    for (int d = 0; d < LSE_DEPTH - 1; ++d) issue();
    // consumer side: raw maximum m_raw of the row so far and s = sum of 2^((x - m_raw) * log2 e)
    float m_raw = LSE_FLOOR, ssum = 0.0f, pick = 0.0f;
    int c = 0, u = warp, c_slot = 0;
    for (int unit = 0; unit < units; ++unit) {
        issue();
        if (c == 0) pick = load_pick(u);
        cp_async_wait<LSE_DEPTH - 1>();  // this unit's copies have landed
        const uint4 *slot = ring + c_slot * LSE_CHUNK_VECS;
        c_slot = (c_slot + 1 == LSE_DEPTH) ? 0 : c_slot + 1;
        const int left = nv - c * LSE_CHUNK_VECS - lane;
        float x[4][E];
        if (left > 96) {
#pragma unroll
            for (int k = 0; k < 4; ++k) Vec16<InT>::unpack(slot[32 * k], x[k]);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (32 * k < left) {
                    Vec16<InT>::unpack(slot[32 * k], x[k]);
                } else {
#pragma unroll
                    for (int e = 0; e < E; ++e) x[k][e] = NINF;   // contributes 2^-inf = 0
                }
            }
        }
        float m = m_raw;
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int e = 0; e < E; ++e) m = fmaxf(m, x[k][e]);
        const float m2 = m * LOG2E;
        float s = ssum * ex2((m_raw - m) * LOG2E);
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int e = 0; e < E; ++e) s += ex2(fmaf(x[k][e], LOG2E, -m2));
        m_raw = m;
        ssum = s;
        if (++c == nch) {
            finish_row(u, MaxSum{m_raw * LOG2E, ssum}, pick);
            m_raw = LSE_FLOOR;
            ssum = 0.0f;
            c = 0;
            u += 8;
        }
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
    int padding_cleared;    // the padding rows of `out` are zero already (cleared during the forward pass)
    const int64_t *cu;      // packed logits and gradient: row offsets per utterance; nullptr = padded
    int64_t packed_rows;
};

// One CTA per (n,t) slab again, one warp per row.  Padding rows are streamed out as zeros; a valid
// row is read once (four 16-byte loads per lane in flight), turned into -softmax * sum(G) in
// registers, gets its <= 3 sparse entries added by the lanes that own those columns, and is written once.
template <typename T>
__global__ void __launch_bounds__(256, LOGITS_BLOCKS_PER_SM) k_logits_grad(const LogitsGradArgs a) {
    pdl_wait();
    constexpr int E = Vec16<T>::E;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t nt = blockIdx.x;
    const int n = static_cast<int>(nt / a.T);
    const int t = static_cast<int>(nt - static_cast<int64_t>(n) * a.T);
    const int U1 = a.U1, U = U1 - 1, V = a.V;
    const int lx_n = a.lx[n];
    int Un = (t < lx_n) ? min(a.ly[n], U) : -1;
    if (a.cu && Un >= 0 && a.cu[n] + static_cast<int64_t>(t + 1) * (Un + 1) > a.packed_rows) Un = -1;
    const int64_t slab_row = a.cu ? a.cu[n] + static_cast<int64_t>(t) * (Un + 1) : nt * U1;
    const T *slab_in = static_cast<const T *>(a.logits) + slab_row * V;
    T *slab_out = static_cast<T *>(a.out) + slab_row * V;
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    const int *y = a.ys + static_cast<int64_t>(n) * U;
    const float4 *grs = a.GR + nt * U1;
    float go = 0.0f;
    if (Un >= 0) go = a.scalar_grad ? a.grad_out[0] * utterance_weight(a.red, lx_n) : a.grad_out[n];

    // padding rows of the slab form one contiguous block: all 256 threads stream zeros over it
    if (!a.padding_cleared && a.cu == nullptr) {  // a packed tensor has no padding rows
        T *pad = slab_out + static_cast<int64_t>(Un + 1) * V;
        const int64_t count = static_cast<int64_t>(U1 - (Un + 1)) * V;
        if (a.vec) {
            uint4 *dv = reinterpret_cast<uint4 *>(pad);
            for (int64_t j = threadIdx.x; j < count / E; j += 256) dv[j] = z;
        } else {
            const T zt = OutOps<T>::cvt(0.0f);
            for (int64_t c = threadIdx.x; c < count; c += 256) pad[c] = zt;
        }
    }
    for (int u = warp; u <= Un; u += 8) {
        const float4 gr = grs[u];
        // sparse part: column 0 and the two label columns; coinciding columns add up
        float c0 = go * gr.x, c1 = 0.0f, c2 = 0.0f;
        int i1 = -1, i2 = -1;
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
        const T *row = slab_in + static_cast<int64_t>(u) * V;
        T *orow = slab_out + static_cast<int64_t>(u) * V;
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

// Gradient of the log-add joiner's denominator on the tensor cores (tcgen05 + TMEM + TMA).
//
// With den[t,u] = log sum_v exp(f[t,v] + g[u,v]) and w[t,u] = dLoss/d den[t,u]
// (warp_ctct/__init__.py:47-52, csrc/binding.cpp:247-324 compute it one (t,u,v) term at a time):
//     grad_f[t,v] = sum_u w[t,u] exp(f[t,v] + g[u,v] - den[t,u]) = Ef[t,v] * sum_u P[t,u] Eg[u,v]
//     grad_g[u,v] = sum_t w[t,u] exp(f[t,v] + g[u,v] - den[t,u]) = Eg[u,v] * sum_t P[t,u] Ef[t,v]
// where Ef = exp(f - mf), Eg = exp(g - mg) are the max-shifted exponentials whose bf16 hi/lo
// planes the forward pass left in its workspace, and
//     P[t,u] = w[t,u] * exp(mf[t] + mg[u] - den[t,u])
// is small (T x U+1 per utterance).  Both sums are ordinary GEMMs with the vocabulary as the wide
// output dimension; the multiplication by Ef / Eg is the epilogue.  T*(U+1)*V exponentials and
// multiply-adds per utterance on the CUDA cores become (T + U+1) * V exponentials plus tensor-core
// work, and the kernels are bound by reading f (g) and writing grad_f (grad_g) once.
//
//  k_den_weights   : P as two bf16 planes (hi + lo), rows padded to a multiple of 8 columns
//  k_logmm_bwd_tc  : one CTA per 128 x 64 output tile; A_MN = false: A = P (K-major, k = u),
//                    A_MN = true: A = P read transposed (MN-major, m = u, k = t).  The B operand
//                    (Eg or Ef planes) is MN-major in both: the vocabulary index is contiguous.
//                    Two CTAs fit one SM (96 KB of stages each), so one tile's epilogue overlaps
//                    the other's loads.  Waits are bounded as in k_logmm_tc.
#pragma once

#include "logmm_tc.cuh"

namespace ctct {

constexpr int BW_BM = 128, BW_BN = 64, BW_BK = 64, BW_STAGES = 2;
constexpr int BW_A_PLANE = BW_BM * BW_BK * 2;  // 16 KB
constexpr int BW_B_PLANE = BW_BN * BW_BK * 2;  //  8 KB
constexpr int BW_STAGE_BYTES = 2 * BW_A_PLANE + 2 * BW_B_PLANE;
constexpr int BW_SMEM_BYTES = BW_STAGES * BW_STAGE_BYTES + 1024 + 128;

struct DenWeightArgs {
    const float4 *grads3;  // [B][T][U1] records {g0,g1,g2,0}; w = -scale[b] * (g0+g1+g2)
    const float *scale;    // [B]
    const float *den;      // (B,T,U1)
    const float *mf;       // (B,T)
    const float *mg;       // (B,U1)
    const int *lx, *ly;
    __nv_bfloat16 *ph, *pl;  // (B,T,U1p)
    int T, U1, U1p;
    const int *flags;
};

// one block per (b,t) row
__global__ void __launch_bounds__(128) k_den_weights(const DenWeightArgs a) {
    if (a.flags[0] | a.flags[1]) return;
    const int64_t bt = blockIdx.x;
    const int b = static_cast<int>(bt / a.T), t = static_cast<int>(bt - static_cast<int64_t>(b) * a.T);
    const bool row_ok = t < a.lx[b];
    const int un = min(a.ly[b] + 1, a.U1);
    const float sc = -a.scale[b];
    const float mfr = a.mf[bt];
    for (int u = threadIdx.x; u < a.U1p; u += blockDim.x) {
        float p = 0.0f;
        if (row_ok && u < un) {
            const float4 g3 = a.grads3[bt * a.U1 + u];
            const float w = sc * (g3.x + g3.y + g3.z);
            if (w != 0.0f) p = w * ex2((mfr + a.mg[static_cast<int64_t>(b) * a.U1 + u] - a.den[bt * a.U1 + u]) * LOG2E);
        }
        const __nv_bfloat16 h = __float2bfloat16_rn(p);
        a.ph[bt * a.U1p + u] = h;
        a.pl[bt * a.U1p + u] = __float2bfloat16_rn(p - __bfloat162float(h));
    }
}

struct LogmmBwdTcArgs {
    const float *src;  // (B, M, N) fp32: f for grad_f, g for grad_g
    const float *mx;   // (B, M) row maxima of src
    float *out;        // (B, M, N)
    int M, N, K;       // output rows per batch entry, vocabulary, contraction length
    int *flags;        // [0] a bounded wait ran out, [1] forward underflow (exact kernel needed)
};

template <bool A_MN>
__global__ void __launch_bounds__(128) k_logmm_bwd_tc(const __grid_constant__ CUtensorMap map_ah,
                                                      const __grid_constant__ CUtensorMap map_al,
                                                      const __grid_constant__ CUtensorMap map_bh,
                                                      const __grid_constant__ CUtensorMap map_bl,
                                                      const LogmmBwdTcArgs a) {
    extern __shared__ unsigned char bw_raw[];
    __shared__ int skip;
    if (threadIdx.x == 0) skip = a.flags[0] | a.flags[1];
    __syncthreads();
    if (skip) return;  // the exact kernel does the work (same decision for the whole CTA)
    const unsigned raw = smem_u32(bw_raw);
    const unsigned tiles = (raw + 1023u) & ~1023u;
    const unsigned bars = tiles + BW_STAGES * BW_STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (BW_STAGES + s); };
    const unsigned accum_bar = bars + 8u * (2 * BW_STAGES);
    const unsigned slot_addr = bars + 8u * (2 * BW_STAGES + 1);
    unsigned *slot_ptr = reinterpret_cast<unsigned *>(bw_raw + (slot_addr - raw));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BW_BM, n0 = blockIdx.y * BW_BN, b = blockIdx.z;
    const int nk = (a.K + BW_BK - 1) / BW_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < BW_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(BW_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *slot_ptr;
    bool ok = true;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer
        for (int kb = 0; kb < nk && ok; ++kb) {
            const int s = kb % BW_STAGES;
            ok = mbar_wait(empty_bar(s), ((kb / BW_STAGES) & 1) ^ 1);
            if (!ok) break;
            const unsigned st = tiles + s * BW_STAGE_BYTES;
            const unsigned bar = full_bar(s);
            mbar_expect_tx(bar, BW_STAGE_BYTES);
            if (A_MN) {  // two 64-wide chunks of m per plane, each 64 k-rows of 128 bytes
                tma_load_3d(st, &map_ah, bar, m0, kb * BW_BK, b);
                tma_load_3d(st + BW_A_PLANE / 2, &map_ah, bar, m0 + 64, kb * BW_BK, b);
                tma_load_3d(st + BW_A_PLANE, &map_al, bar, m0, kb * BW_BK, b);
                tma_load_3d(st + BW_A_PLANE + BW_A_PLANE / 2, &map_al, bar, m0 + 64, kb * BW_BK, b);
            } else {     // 128 m-rows of 64 k (128 bytes)
                tma_load_3d(st, &map_ah, bar, kb * BW_BK, m0, b);
                tma_load_3d(st + BW_A_PLANE, &map_al, bar, kb * BW_BK, m0, b);
            }
            tma_load_3d(st + 2 * BW_A_PLANE, &map_bh, bar, n0, kb * BW_BK, b);
            tma_load_3d(st + 2 * BW_A_PLANE + BW_B_PLANE, &map_bl, bar, n0, kb * BW_BK, b);
        }
        if (!ok) atomicExch(a.flags, 1);
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: D[128 x 64] += A[128 x 16] * B[16 x 64]; B is MN-major, A as templated
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | (A_MN ? (1u << 15) : 0u) | (1u << 16) |
                               (static_cast<unsigned>(BW_BN >> 3) << 17) | (static_cast<unsigned>(BW_BM >> 4) << 24);
        for (int kb = 0; kb < nk && ok; ++kb) {
            const int s = kb % BW_STAGES;
            ok = mbar_wait(full_bar(s), (kb / BW_STAGES) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned st = tiles + s * BW_STAGE_BYTES;
#pragma unroll
            for (int k4 = 0; k4 < BW_BK / 16; ++k4) {
                uint64_t ah, al;
                if (A_MN) {
                    ah = umma_desc_mn(st + k4 * 2048, BW_A_PLANE / 2);
                    al = umma_desc_mn(st + BW_A_PLANE + k4 * 2048, BW_A_PLANE / 2);
                } else {
                    ah = umma_desc(st + k4 * 32);
                    al = umma_desc(st + BW_A_PLANE + k4 * 32);
                }
                const uint64_t bh = umma_desc_mn(st + 2 * BW_A_PLANE + k4 * 2048, BW_B_PLANE);
                const uint64_t bl = umma_desc_mn(st + 2 * BW_A_PLANE + BW_B_PLANE + k4 * 2048, BW_B_PLANE);
                umma_bf16(tmem_base, ah, bh, idesc, (kb | k4) ? 1u : 0u);
                umma_bf16(tmem_base, ah, bl, idesc, 1u);
                umma_bf16(tmem_base, al, bh, idesc, 1u);
            }
            umma_commit(empty_bar(s));
        }
        if (ok) umma_commit(accum_bar);
        else atomicExch(a.flags, 1);
    }
    __syncwarp();

    // ---- epilogue: out = exp(src - mx) * D; warp w owns TMEM lanes (= output rows) [32w, 32w+32)
    const int row = m0 + warp * 32 + lane;
    const int64_t base = (static_cast<int64_t>(b) * a.M + row) * a.N + n0;
    float mxl = 0.0f;
    if (row < a.M) mxl = a.mx[static_cast<int64_t>(b) * a.M + row];
    const bool done = __all_sync(0xffffffffu, mbar_wait(accum_bar, 0));
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (done) {
#pragma unroll 1
        for (int c = 0; c < BW_BN / 32; ++c) {
            unsigned v[32];
            tmem_ld_32x32(tmem_base + (static_cast<unsigned>(warp * 32) << 16) + c * 32, v);
            if (row < a.M) {
                const float4 *src = reinterpret_cast<const float4 *>(a.src + base + c * 32);
                float4 *dst = reinterpret_cast<float4 *>(a.out + base + c * 32);
                float4 x[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    x[j] = (n0 + c * 32 + 4 * j < a.N) ? __ldg(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (n0 + c * 32 + 4 * j < a.N) {
                        float4 r;
                        // a zero sum stays zero even where exp() would overflow or src is -inf
                        const float d0 = __uint_as_float(v[4 * j]), d1 = __uint_as_float(v[4 * j + 1]);
                        const float d2 = __uint_as_float(v[4 * j + 2]), d3 = __uint_as_float(v[4 * j + 3]);
                        r.x = d0 != 0.0f ? d0 * ex2((x[j].x - mxl) * LOG2E) : 0.0f;
                        r.y = d1 != 0.0f ? d1 * ex2((x[j].y - mxl) * LOG2E) : 0.0f;
                        r.z = d2 != 0.0f ? d2 * ex2((x[j].z - mxl) * LOG2E) : 0.0f;
                        r.w = d3 != 0.0f ? d3 * ex2((x[j].w - mxl) * LOG2E) : 0.0f;
                        dst[j] = r;
                    }
                }
            }
        }
    } else if (threadIdx.x == 0) {
        atomicExch(a.flags, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BW_BN) : "memory");
    }
}

}  // namespace ctct

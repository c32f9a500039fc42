// Log-semiring matrix product on the 5th-generation tensor cores (tcgen05 + TMEM + TMA):
//     den[b,i,j] = log sum_k exp(f[b,i,k] + g[b,j,k])
// the denominator of the log-add joiner (warp_ctct/__init__.py:195-200; the reference computes it
// with one thread block per output element, csrc/logmatmul.cu:44-146).
//
// Factorisation.  With row maxima mf[b,i] = max_k f, mg[b,j] = max_k g,
//     den = mf + mg + log( sum_k exp(f - mf) * exp(g - mg) ),
// so the only dense contraction on the path is an ordinary GEMM on max-shifted exponentials; the
// log / max rescaling is the epilogue.  Only (M + N) * K exponentials are taken instead of
// M * N * K.
//
// Precision.  A single bf16 (or tf32) operand rounding would leave ~1e-5 of error in den, which
// the lattice accumulates over T frames; each operand is therefore split into two bf16 numbers
// (hi = round(x), lo = round(x - hi), 16 significant bits together) and three MMAs are issued
// per k-step (hi*hi, hi*lo, lo*hi) into the same fp32 TMEM accumulator.
//
//  k_exp_split  : row maxima and the two bf16 operand planes of exp(x - max)  (one block per row)
//  k_logmm_tc   : one CTA per 128 x 128 output tile of one batch entry; warp 0 = TMA producer
//                 (4 operand planes per stage, 128-byte swizzle), warp 1 = MMA issuer
//                 (tcgen05.mma.cta_group::1.kind::f16, bf16 x bf16 -> fp32 in TMEM), all four
//                 warps = epilogue (tcgen05.ld, log, + mf + mg, store).  3-stage mbarrier ring.
//                 Every wait is bounded; on a time-out the CTA raises a flag in global memory,
//                 skips the rest and still releases its TMEM.
//  An output whose shifted sum underflows (rows whose maxima sit at different k and whose
//  dynamic range exceeds ~80 nats) raises the same kind of flag; the caller then runs the exact
//  kernel (k_logmm_exact), which looks at that flag and otherwise returns immediately.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace ctct {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64;  // BK bf16 = one 128-byte swizzle row
constexpr int TC_STAGES = 3;
constexpr int TC_TMEM_COLS = 4 * TC_BN;  // three main accumulators + one for the cross terms
constexpr int TC_PLANE_BYTES = TC_BM * TC_BK * 2;                 // 16 KB per operand plane
constexpr int TC_STAGE_BYTES = 4 * TC_PLANE_BYTES;                // A_hi, A_lo, B_hi, B_lo
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr unsigned TC_SPIN_LIMIT = 1u << 23;                      // polls per wait (a fraction of a second)
// The limit the kernels actually use: a constant-memory word, so that a test can set it to 0 (every wait
// gives up before anything was issued) and exercise the give-up paths without hanging anything.
__constant__ unsigned c_tc_spin_limit = TC_SPIN_LIMIT;

// ---- prologue: row maximum, exp(x - max) split into two bf16 planes -------------------------
__global__ void __launch_bounds__(256) k_exp_split(const float *__restrict__ x, int K, __nv_bfloat16 *__restrict__ hi,
                                                   __nv_bfloat16 *__restrict__ lo, float *__restrict__ mx) {
    __shared__ float red[8];
    pdl_wait();
    pdl_trigger();  // the next launch (the other operand, or the GEMM's one CTA per SM) may move in
    const int64_t r = blockIdx.x;
    const float *row = x + r * K;
    const float NINF = -__int_as_float(0x7f800000);
    float m = NINF;
    for (int k = threadIdx.x * 4; k < K; k += 1024) {
        const float4 v = *reinterpret_cast<const float4 *>(row + k);
        m = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    if (threadIdx.x == 0) mx[r] = m;
    const bool dead = !(m > NINF) || !(m < -NINF);  // all -inf (or a +inf / NaN row): contributes nothing here
    for (int k = threadIdx.x * 4; k < K; k += 1024) {
        const float4 v = *reinterpret_cast<const float4 *>(row + k);
        float e[4] = {v.x, v.y, v.z, v.w};
        __nv_bfloat16 h[4], l[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float t = dead ? 0.0f : ex2((e[q] - m) * LOG2E);
            h[q] = __float2bfloat16_rn(t);
            l[q] = __float2bfloat16_rn(t - __bfloat162float(h[q]));
        }
        uint2 ph, pl;
        ph.x = __bfloat16_as_ushort(h[0]) | (static_cast<unsigned>(__bfloat16_as_ushort(h[1])) << 16);
        ph.y = __bfloat16_as_ushort(h[2]) | (static_cast<unsigned>(__bfloat16_as_ushort(h[3])) << 16);
        pl.x = __bfloat16_as_ushort(l[0]) | (static_cast<unsigned>(__bfloat16_as_ushort(l[1])) << 16);
        pl.y = __bfloat16_as_ushort(l[2]) | (static_cast<unsigned>(__bfloat16_as_ushort(l[3])) << 16);
        *reinterpret_cast<uint2 *>(hi + r * K + k) = ph;
        *reinterpret_cast<uint2 *>(lo + r * K + k) = pl;
    }
}

// ---- PTX helpers -----------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void *p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// bounded wait on a phase parity (non-blocking polls); false = gave up
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    const unsigned limit = c_tc_spin_limit;
    for (unsigned spin = 0; spin < limit; ++spin) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap *map, unsigned bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// K-major operand tile, 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO = 64 in 16-byte
// units), leading-dimension offset 1, descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t umma_desc(unsigned smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(64) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// MN-major operand tile (the M or N index is the contiguous one), 128-byte swizzle: rows are k,
// 128 bytes (64 elements of M/N) each; groups of 8 k-rows are 1024 bytes apart (SBO = 64) and
// successive 64-element chunks of M/N are lbo_bytes apart
__device__ __forceinline__ uint64_t umma_desc_mn(unsigned smem_addr, unsigned lbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= static_cast<uint64_t>(64) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// The issuing thread is alone in its warp, so every instruction between two MMAs costs several
// cycles: descriptors are kept as a 32-bit low word (start address and leading offset) that is
// advanced with plain adds (+1 per 16 bytes) next to a constant high word.
constexpr unsigned UMMA_DESC_HI = 64u | (1u << 14) | (2u << 29);  // SBO 1024 B, version 1, SWIZZLE_128B
__device__ __forceinline__ unsigned umma_lo(unsigned smem_addr) { return ((smem_addr >> 4) & 0x3fffu) | (1u << 16); }
__device__ __forceinline__ unsigned umma_lo_mn(unsigned smem_addr, unsigned lbo_bytes) {
    return ((smem_addr >> 4) & 0x3fffu) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
__device__ __forceinline__ uint64_t umma_pack(unsigned lo) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(UMMA_DESC_HI));
    return d;
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct LogmmTcArgs {
    float *den;       // (B, M, N)
    const float *mf;  // (B, M) row maxima of f
    const float *mg;  // (B, N) row maxima of g
    int M, N, K;
    int *flags;       // [0] a bounded wait ran out, [1] a shifted sum underflowed (exact kernel needed)
};

__global__ void __launch_bounds__(128) k_logmm_tc(const __grid_constant__ CUtensorMap map_ah,
                                                  const __grid_constant__ CUtensorMap map_al,
                                                  const __grid_constant__ CUtensorMap map_bh,
                                                  const __grid_constant__ CUtensorMap map_bl, const LogmmTcArgs a) {
    extern __shared__ unsigned char tc_raw[];
    const unsigned raw = smem_u32(tc_raw);
    const unsigned tiles = (raw + 1023u) & ~1023u;  // 128-byte swizzle atoms are 1024-byte aligned
    const unsigned bars = tiles + TC_STAGES * TC_STAGE_BYTES;
    // barrier layout (8 bytes each): full[STAGES], empty[STAGES], accum; then the TMEM base slot
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (TC_STAGES + s); };
    const unsigned accum_bar = bars + 8u * (2 * TC_STAGES);
    const unsigned slot_addr = bars + 8u * (2 * TC_STAGES + 1);
    unsigned *slot_ptr = reinterpret_cast<unsigned *>(tc_raw + (slot_addr - raw));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * TC_BN, b = blockIdx.z;
    const int nk = (a.K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *slot_ptr;
    bool ok = true;
    pdl_wait();  // barriers and TMEM were set up while the kernel before this one drained

    if (warp == 0 && lane == 0) {
        // ---- TMA producer
        int issued = 0;
        for (int kb = 0; kb < nk && ok; ++kb) {
            const int s = kb % TC_STAGES;
            ok = mbar_wait(empty_bar(s), ((kb / TC_STAGES) & 1) ^ 1);
            if (!ok) break;
            const unsigned st = tiles + s * TC_STAGE_BYTES;
            issued = kb + 1;
            mbar_expect_tx(full_bar(s), TC_STAGE_BYTES);
            tma_load_3d(st + 0 * TC_PLANE_BYTES, &map_ah, full_bar(s), kb * TC_BK, m0, b);
            tma_load_3d(st + 1 * TC_PLANE_BYTES, &map_al, full_bar(s), kb * TC_BK, m0, b);
            tma_load_3d(st + 2 * TC_PLANE_BYTES, &map_bh, full_bar(s), kb * TC_BK, n0, b);
            tma_load_3d(st + 3 * TC_PLANE_BYTES, &map_bl, full_bar(s), kb * TC_BK, n0, b);
        }
        if (!ok) {
            atomicExch(a.flags, 1);
            // loads still in flight must land before this CTA's shared memory goes to the next one:
            // wait (bounded, like every wait) for the last load of every stage that was armed
            for (int kb = max(0, issued - TC_STAGES); kb < issued; ++kb) mbar_wait(full_bar(kb % TC_STAGES), (kb / TC_STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: D[128x128, fp32 in TMEM] += A[128x16] * B[128x16]^T, both K-major bf16
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<unsigned>(TC_BN >> 3) << 17) |
                               (static_cast<unsigned>(TC_BM >> 4) << 24);
        for (int kb = 0; kb < nk && ok; ++kb) {
            const int s = kb % TC_STAGES;
            ok = mbar_wait(full_bar(s), (kb / TC_STAGES) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned st = tiles + s * TC_STAGE_BYTES;
            // The tensor core truncates when it adds into the fp32 accumulator, a bias that grows
            // with the number of accumulation steps (3e-5 relative after 768 steps).  So the main
            // products hi*hi go round-robin into three accumulators (a third of the steps each)
            // and the small cross terms into a fourth; the epilogue adds the four in fp32.
            const unsigned acc_main = tmem_base + static_cast<unsigned>(kb % 3) * TC_BN;
            const unsigned acc_cross = tmem_base + 3u * TC_BN;
            const unsigned d0 = umma_lo(st);  // A_hi; the other planes follow at TC_PLANE_BYTES each
#pragma unroll
            for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
                const uint64_t ah = umma_pack(d0 + (0 * TC_PLANE_BYTES + k4 * 32) / 16);
                const uint64_t al = umma_pack(d0 + (1 * TC_PLANE_BYTES + k4 * 32) / 16);
                const uint64_t bh = umma_pack(d0 + (2 * TC_PLANE_BYTES + k4 * 32) / 16);
                const uint64_t bl = umma_pack(d0 + (3 * TC_PLANE_BYTES + k4 * 32) / 16);
                umma_bf16(acc_main, ah, bh, idesc, (kb >= 3 || k4 > 0) ? 1u : 0u);
                umma_bf16(acc_cross, ah, bl, idesc, (kb | k4) ? 1u : 0u);
                umma_bf16(acc_cross, al, bh, idesc, 1u);
            }
            umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(accum_bar);
        else atomicExch(a.flags, 1);
    }
    __syncwarp();

    // ---- epilogue: all four warps, warp w owns TMEM lanes (= output rows) [32w, 32w+32)
    const bool done = __all_sync(0xffffffffu, mbar_wait(accum_bar, 0));  // warp-uniform: tcgen05.ld is .aligned
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (done) {
        const float NINF = -__int_as_float(0x7f800000);
        const int row = m0 + warp * 32 + lane;
        const float mfr = (row < a.M) ? a.mf[static_cast<int64_t>(b) * a.M + row] : NINF;
        bool underflow = false;
#pragma unroll 1
        for (int c = 0; c < TC_BN / 32; ++c) {
            unsigned v[32];
            const unsigned lane_base = tmem_base + (static_cast<unsigned>(warp * 32) << 16) + c * 32;
            tmem_ld_32x32(lane_base + 3u * TC_BN, v);  // cross terms first (smallest), then the main parts
            const int nmain = nk < 3 ? nk : 3;
            for (int q = 0; q < nmain; ++q) {
                unsigned w[32];
                tmem_ld_32x32(lane_base + static_cast<unsigned>(q) * TC_BN, w);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
            }
            if (row < a.M) {
                float *out = a.den + (static_cast<int64_t>(b) * a.M + row) * a.N;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int col = n0 + c * 32 + j;
                    if (col < a.N) {
                        const float mgc = __ldg(a.mg + static_cast<int64_t>(b) * a.N + col);
                        const float sum = __uint_as_float(v[j]);
                        float r = NINF;
                        if (mfr > NINF && mgc > NINF) {
                            r = mfr + mgc + lg2(sum) * 0.6931471805599453f;
                            if (!(sum > 1e-30f) || !(mfr < -NINF) || !(mgc < -NINF)) underflow = true;
                        }
                        out[col] = r;
                    }
                }
            }
        }
        if (underflow) atomicExch(a.flags + 1, 1);
    } else if (threadIdx.x == 0) {
        atomicExch(a.flags, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

}  // namespace ctct

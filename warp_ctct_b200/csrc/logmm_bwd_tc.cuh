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
//  k_logmm_bwd_tc  : persistent, one CTA per SM walking 128 x 64 output tiles.  A_MN = false:
//                    A = P (K-major, k = u); A_MN = true: A = P read transposed (MN-major, m = u,
//                    k = t).  The B operand (Eg or Ef planes) is MN-major in both: the vocabulary
//                    index is contiguous.  Warp 0 = TMA producer (operand ring + the fp32 src tile
//                    of the epilogue), warp 1 = MMA issuer, warps 2-9 = epilogue.  Two TMEM
//                    accumulators and two epilogue tiles, so tile i's epilogue (tcgen05.ld,
//                    exp, TMA store) overlaps tile i+1's loads and MMAs.  All global traffic is
//                    TMA.  Waits are bounded as in k_logmm_tc.
#pragma once

#include "logmm_tc.cuh"

namespace ctct {

constexpr int BW_BM = 128, BW_BN = 64, BW_BK = 64;
constexpr int BW_A_PLANE = BW_BM * BW_BK * 2;  // 16 KB
constexpr int BW_B_PLANE = BW_BN * BW_BK * 2;  //  8 KB
constexpr int BW_STAGE_BYTES = 2 * BW_A_PLANE + 2 * BW_B_PLANE;
constexpr int BW_EPI_HALF = BW_BM * 128;       // 128 rows x 32 floats, 128-byte swizzle
constexpr int BW_EPI_BYTES = 2 * BW_EPI_HALF;  // one 128 x 64 fp32 tile
constexpr int BW_EPI_WARPS = 8;                // two per TMEM lane quarter: 32 of the 64 columns each
constexpr int BW_THREADS = 64 + 32 * BW_EPI_WARPS;
constexpr int BW_ARES_KB = 2;                  // k-blocks of A that the resident variant keeps in shared memory
__host__ __device__ constexpr int bw_stage_bytes(bool a_res) { return a_res ? 2 * BW_B_PLANE : BW_STAGE_BYTES; }
constexpr int bw_smem_bytes(int stages, int ebufs, bool a_res) {
    return stages * bw_stage_bytes(a_res) + (a_res ? BW_ARES_KB * 2 * BW_A_PLANE : 0) + ebufs * BW_EPI_BYTES + 1024 + 256;
}

struct DenWeightArgs {
    const float4 *grads3;  // [B][T][U1] records {g0,g1,g2,0}; w = -scale[b] * (g0+g1+g2)
    const float *scale;    // [B]
    const float *gout;     // or: w given directly, (B,T,U1), any sign, every entry valid (then lx, ly unused)
    const float *den;      // (B,T,U1)
    const float *mf;       // (B,T)
    const float *mg;       // (B,U1)
    const int *lx, *ly;
    __nv_bfloat16 *ph, *pl;  // (B,T,U1p)
    int T, U1, U1p;
    const int *flags;
};

// one block per (b,t) row.  Every load is issued before any of them is needed (all addresses are in
// bounds for u < U1), so a block pays one round of memory latency, not two.
__global__ void __launch_bounds__(128) k_den_weights(const DenWeightArgs a) {
    pdl_wait();
    const int64_t bt = blockIdx.x;
    const int b = static_cast<int>(bt / a.T), t = static_cast<int>(bt - static_cast<int64_t>(b) * a.T);
    const int u = threadIdx.x;  // U1p <= 128 columns per pass
    const int f0 = a.flags[0], f1 = a.flags[1];
    const int lxb = a.gout ? a.T : a.lx[b];
    const int lyb = a.gout ? a.U1 : a.ly[b];
    const float scl = a.gout ? 0.0f : a.scale[b];
    const float mfr = a.mf[bt];
    for (int u0 = 0; u0 < a.U1p; u0 += blockDim.x) {
        const int uu = u0 + u;
        float w = 0.0f, mgv = 0.0f, dv = 0.0f;
        if (uu < a.U1) {
            if (a.gout) {
                w = a.gout[bt * a.U1 + uu];
            } else {
                const float4 g3 = a.grads3[bt * a.U1 + uu];
                w = -(g3.x + g3.y + g3.z);
            }
            mgv = a.mg[static_cast<int64_t>(b) * a.U1 + uu];
            dv = a.den[bt * a.U1 + uu];
        }
        if (f0 | f1) return;  // the exact kernel does the work
        if (uu >= a.U1p) continue;
        float p = 0.0f;
        if (!a.gout) w *= scl;
        const bool live = t < lxb && uu < (a.gout ? a.U1 : min(lyb + 1, a.U1));
        if (live && w != 0.0f) p = w * ex2((mfr + mgv - dv) * LOG2E);
        const __nv_bfloat16 h = __float2bfloat16_rn(p);
        a.ph[bt * a.U1p + uu] = h;
        a.pl[bt * a.U1p + uu] = __float2bfloat16_rn(p - __bfloat162float(h));
    }
}

struct LogmmBwdTcArgs {
    const float *mx;   // (B, M) row maxima of src
    int M, N, K;       // output rows per batch entry, vocabulary, contraction length
    int tiles_m, tiles_n, total_tiles;  // total = tiles_m * tiles_n * B; m runs fastest
    int *flags;        // [0] a bounded wait ran out, [1] forward underflow (exact kernel needed)
};

__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, unsigned src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

// maps: A planes (hi, lo), B planes (hi, lo), src (fp32, read), out (fp32, written); the last two
// describe (B, M, N) tensors with a 32 x 128 x 1 box and 128-byte swizzle
// STAGES: depth of the operand ring; EBUFS: epilogue tiles in flight (src loaded, result stored in place).
// A_RES (K-major A, K <= 64 * BW_ARES_KB): each CTA takes a contiguous run of tiles with n fastest
// and keeps the A tile of the current (batch entry, m-tile) in shared memory, so that only B
// streams through the ring; otherwise tiles are dealt round-robin with m fastest.
template <bool A_MN, bool A_RES, int STAGES, int EBUFS>
__global__ void __launch_bounds__(BW_THREADS, 1) k_logmm_bwd_tc(const __grid_constant__ CUtensorMap map_ah,
                                                                const __grid_constant__ CUtensorMap map_al,
                                                                const __grid_constant__ CUtensorMap map_bh,
                                                                const __grid_constant__ CUtensorMap map_bl,
                                                                const __grid_constant__ CUtensorMap map_src,
                                                                const __grid_constant__ CUtensorMap map_out,
                                                                const LogmmBwdTcArgs a) {
    extern __shared__ unsigned char bw_raw[];
    __shared__ int skip;
    pdl_wait();
    if (threadIdx.x == 0) skip = a.flags[0] | a.flags[1];
    __syncthreads();
    if (skip) return;  // the exact kernel does the work (same decision for the whole CTA)
    const unsigned raw = smem_u32(bw_raw);
    static_assert(!(A_RES && A_MN), "the resident A tile is K-major");
    constexpr int STAGE_BYTES = bw_stage_bytes(A_RES);
    constexpr int B_OFF = A_RES ? 0 : 2 * BW_A_PLANE;  // B planes inside a ring stage
    const unsigned ring = (raw + 1023u) & ~1023u;
    const unsigned ares = ring + STAGES * STAGE_BYTES;  // resident A: per k-block hi plane, lo plane
    const unsigned epi = ares + (A_RES ? BW_ARES_KB * 2 * BW_A_PLANE : 0);
    const unsigned bars = epi + EBUFS * BW_EPI_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int q) { return bars + 8u * (2 * STAGES + q); };
    auto acc_empty = [&](int q) { return bars + 8u * (2 * STAGES + 2 + q); };
    auto src_full = [&](int e) { return bars + 8u * (2 * STAGES + 4 + e); };
    auto src_empty = [&](int e) { return bars + 8u * (2 * STAGES + 4 + EBUFS + e); };
    const unsigned a_full = bars + 8u * (2 * STAGES + 4 + 2 * EBUFS), a_empty = a_full + 8u;
    constexpr int NBARS = 2 * STAGES + 4 + 2 * EBUFS + 2;
    static_assert(8 * NBARS + 8 <= 256, "barrier area");
    const unsigned slot_addr = bars + 8u * NBARS;
    unsigned *slot_ptr = reinterpret_cast<unsigned *>(bw_raw + (slot_addr - raw));
    unsigned char *epi_ptr = bw_raw + (epi - raw);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nk = (a.K + BW_BK - 1) / BW_BK;
    constexpr unsigned TMEM_COLS = 2 * BW_BN;

    if (threadIdx.x == 0) {
        for (int q = 0; q < NBARS; ++q) mbar_init(bars + 8u * q, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *slot_ptr;
    bool ok = true;

    // this CTA's tiles: first, first + step, ... < last
    const int first = A_RES ? static_cast<int>(static_cast<int64_t>(blockIdx.x) * a.total_tiles / gridDim.x) : blockIdx.x;
    const int last = A_RES ? static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * a.total_tiles / gridDim.x) : a.total_tiles;
    const int step = A_RES ? 1 : gridDim.x;
    auto tile_coords = [&](int tile, int &m0, int &n0, int &b) {
        if (A_RES) {  // n fastest; tile / tiles_n names the (b, m-tile) group that shares A
            n0 = (tile % a.tiles_n) * BW_BN;
            const int rest = tile / a.tiles_n;
            m0 = (rest % a.tiles_m) * BW_BM;
            b = rest / a.tiles_m;
        } else {
            m0 = (tile % a.tiles_m) * BW_BM;
            const int rest = tile / a.tiles_m;
            n0 = (rest % a.tiles_n) * BW_BN;
            b = rest / a.tiles_n;
        }
    };

    if (warp == 0 && lane == 0) {
        // ---- TMA producer: per tile the operand k-blocks, then the fp32 src tile of the epilogue
        unsigned it = 0;
        unsigned armed = 0, armed_parity = 0;  // bit s: full_bar(s) armed / parity of that phase; bits 8..: src_full
        int group = -1;
        unsigned groups = 0;
        for (int tile = first, i = 0; tile < last && ok; tile += step, ++i) {
            int m0, n0, b;
            tile_coords(tile, m0, n0, b);
            if (A_RES && tile / a.tiles_n != group) {
                // new (batch entry, m-tile): reload A once the MMAs on the old one have finished
                group = tile / a.tiles_n;
                ok = mbar_wait(a_empty, (groups & 1) ^ 1);
                if (!ok) break;
                mbar_expect_tx(a_full, nk * 2 * BW_A_PLANE);
                for (int kb = 0; kb < nk; ++kb) {
                    tma_load_3d(ares + kb * 2 * BW_A_PLANE, &map_ah, a_full, kb * BW_BK, m0, b);
                    tma_load_3d(ares + kb * 2 * BW_A_PLANE + BW_A_PLANE, &map_al, a_full, kb * BW_BK, m0, b);
                }
                armed |= 1u << 16;
                armed_parity = (armed_parity & ~(1u << 16)) | ((groups & 1) << 16);
                ++groups;
            }
            for (int kb = 0; kb < nk; ++kb, ++it) {
                const int s = it % STAGES;
                const unsigned ph = (it / STAGES) & 1;
                ok = mbar_wait(empty_bar(s), ph ^ 1);
                if (!ok) break;
                const unsigned st = ring + s * STAGE_BYTES;
                const unsigned bar = full_bar(s);
                mbar_expect_tx(bar, STAGE_BYTES);
                if (A_RES) {
                } else if (A_MN) {  // two 64-wide chunks of m per plane, each 64 k-rows of 128 bytes
                    tma_load_3d(st, &map_ah, bar, m0, kb * BW_BK, b);
                    tma_load_3d(st + BW_A_PLANE / 2, &map_ah, bar, m0 + 64, kb * BW_BK, b);
                    tma_load_3d(st + BW_A_PLANE, &map_al, bar, m0, kb * BW_BK, b);
                    tma_load_3d(st + BW_A_PLANE + BW_A_PLANE / 2, &map_al, bar, m0 + 64, kb * BW_BK, b);
                } else {     // 128 m-rows of 64 k (128 bytes)
                    tma_load_3d(st, &map_ah, bar, kb * BW_BK, m0, b);
                    tma_load_3d(st + BW_A_PLANE, &map_al, bar, kb * BW_BK, m0, b);
                }
                tma_load_3d(st + B_OFF, &map_bh, bar, n0, kb * BW_BK, b);
                tma_load_3d(st + B_OFF + BW_B_PLANE, &map_bl, bar, n0, kb * BW_BK, b);
                armed |= 1u << s;
                armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
            }
            if (!ok) break;
            const int e = i % EBUFS;
            const unsigned eph = (i / EBUFS) & 1;
            ok = mbar_wait(src_empty(e), eph ^ 1);
            if (!ok) break;
            mbar_expect_tx(src_full(e), BW_EPI_BYTES);
            tma_load_3d(epi + e * BW_EPI_BYTES, &map_src, src_full(e), n0, m0, b);
            tma_load_3d(epi + e * BW_EPI_BYTES + BW_EPI_HALF, &map_src, src_full(e), n0 + 32, m0, b);
            armed |= 1u << (8 + e);
            armed_parity = (armed_parity & ~(1u << (8 + e))) | (eph << (8 + e));
        }
        if (!ok) atomicExch(a.flags, 1);
        // no copy of this CTA may still be in flight when it exits (bounded; immediate when all went well)
        for (int s = 0; s < STAGES; ++s)
            if (armed & (1u << s)) mbar_wait(full_bar(s), (armed_parity >> s) & 1);
        for (int e = 0; e < EBUFS; ++e)
            if (armed & (1u << (8 + e))) mbar_wait(src_full(e), (armed_parity >> (8 + e)) & 1);
        if (armed & (1u << 16)) mbar_wait(a_full, (armed_parity >> 16) & 1);
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: D[128 x 64] += A[128 x 16] * B[16 x 64]; B is MN-major, A as templated
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | (A_MN ? (1u << 15) : 0u) | (1u << 16) |
                               (static_cast<unsigned>(BW_BN >> 3) << 17) | (static_cast<unsigned>(BW_BM >> 4) << 24);
        unsigned it = 0;
        int group = -1;
        unsigned groups = 0;
        for (int tile = first, i = 0; tile < last && ok; tile += step, ++i) {
            const int q = i & 1;
            if (A_RES && tile / a.tiles_n != group) {
                group = tile / a.tiles_n;
                ok = mbar_wait(a_full, groups & 1);
                if (!ok) break;
                ++groups;
            }
            ok = mbar_wait(acc_empty(q), ((i >> 1) & 1) ^ 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned acc = tmem_base + static_cast<unsigned>(q) * BW_BN;
            for (int kb = 0; kb < nk; ++kb, ++it) {
                const int s = it % STAGES;
                ok = mbar_wait(full_bar(s), (it / STAGES) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned st = ring + s * STAGE_BYTES;
                // low descriptor words of the hi planes; lo planes and k-steps are constant offsets away
                const unsigned da = A_RES  ? umma_lo(ares + kb * 2 * BW_A_PLANE)
                                    : A_MN ? umma_lo_mn(st, BW_A_PLANE / 2)
                                           : umma_lo(st);
                const unsigned db = umma_lo_mn(st + B_OFF, BW_B_PLANE);
                constexpr unsigned A_KSTEP = (A_MN ? 2048 : 32) / 16, B_KSTEP = 2048 / 16;
#pragma unroll
                for (int k4 = 0; k4 < BW_BK / 16; ++k4) {
                    const uint64_t ah = umma_pack(da + k4 * A_KSTEP);
                    const uint64_t al = umma_pack(da + BW_A_PLANE / 16 + k4 * A_KSTEP);
                    const uint64_t bh = umma_pack(db + k4 * B_KSTEP);
                    const uint64_t bl = umma_pack(db + BW_B_PLANE / 16 + k4 * B_KSTEP);
                    umma_bf16(acc, ah, bh, idesc, (kb | k4) ? 1u : 0u);
                    umma_bf16(acc, ah, bl, idesc, 1u);
                    umma_bf16(acc, al, bh, idesc, 1u);
                }
                umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
            }
            if (ok) umma_commit(acc_full(q));
            // last tile on this A: let the producer overwrite it once these MMAs are done
            if (A_RES && ok && (tile + 1 >= last || (tile + 1) / a.tiles_n != group)) umma_commit(a_empty);
        }
        if (!ok) atomicExch(a.flags, 1);
    } else if (warp >= 2) {
        // ---- epilogue warps: out = exp(src - mx) * D, in place in the src tile, then one TMA store.
        // A warp may read the TMEM lanes [32 * (warp % 4), +32): one tile row per thread; the two
        // warps of a lane quarter take 32 columns each.
        const int part = warp & 3;
        const int c = (warp - 2) >> 2;
        const int r = part * 32 + lane;
        const bool leader = (threadIdx.x == 64);
        constexpr int PENDING = EBUFS >= 2 ? 1 : 0;  // stores that may still be reading their tile
        for (int tile = first, i = 0; tile < last; tile += step, ++i) {
            int m0, n0, b;
            tile_coords(tile, m0, n0, b);
            const int q = i & 1;
            const int e = i % EBUFS;
            float mxr = 0.0f;
            if (m0 + r < a.M) mxr = __ldg(a.mx + static_cast<int64_t>(b) * a.M + m0 + r);
            bool got = mbar_wait(src_full(e), (i / EBUFS) & 1);
            got = got && mbar_wait(acc_full(q), (i >> 1) & 1);
            // same decision in all epilogue warps (they meet again at a barrier below)
            unsigned all_got;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.u32 q, %1, 0;\n\t"
                "bar.red.and.pred p, 1, %2, q;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(all_got)
                : "r"(static_cast<unsigned>(got)), "n"(32 * BW_EPI_WARPS)
                : "memory");
            ok = all_got != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            {
                unsigned v[32];
                tmem_ld_32x32(tmem_base + (static_cast<unsigned>(part * 32) << 16) + q * BW_BN + c * 32, v);
                unsigned char *rowp = epi_ptr + e * BW_EPI_BYTES + c * BW_EPI_HALF + r * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float4 *cell = reinterpret_cast<float4 *>(rowp + ((j ^ (r & 7)) << 4));  // 128-byte swizzle
                    const float4 x = *cell;
                    // a zero sum stays zero even where exp() would overflow or src is -inf
                    const float d0 = __uint_as_float(v[4 * j]), d1 = __uint_as_float(v[4 * j + 1]);
                    const float d2 = __uint_as_float(v[4 * j + 2]), d3 = __uint_as_float(v[4 * j + 3]);
                    float4 o;
                    o.x = d0 != 0.0f ? d0 * ex2((x.x - mxr) * LOG2E) : 0.0f;
                    o.y = d1 != 0.0f ? d1 * ex2((x.y - mxr) * LOG2E) : 0.0f;
                    o.z = d2 != 0.0f ? d2 * ex2((x.z - mxr) * LOG2E) : 0.0f;
                    o.w = d3 != 0.0f ? d3 * ex2((x.w - mxr) * LOG2E) : 0.0f;
                    *cell = o;
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // tile writes -> visible to the TMA store
            asm volatile("bar.sync 1, %0;" ::"n"(32 * BW_EPI_WARPS) : "memory");  // the epilogue warps
            if (leader) {
                mbar_arrive(acc_empty(q));  // every epilogue warp has read this accumulator
                tma_store_3d(&map_out, epi + e * BW_EPI_BYTES, n0, m0, b);
                tma_store_3d(&map_out, epi + e * BW_EPI_BYTES + BW_EPI_HALF, n0 + 32, m0, b);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                if (i >= PENDING) {
                    // the store issued PENDING tiles ago has finished reading its buffer: hand it back
                    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory");
                    mbar_arrive(src_empty((i - PENDING) % EBUFS));
                }
            }
        }
        if (leader) {
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            if (!ok) atomicExch(a.flags, 1);
        }
    }
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace ctct

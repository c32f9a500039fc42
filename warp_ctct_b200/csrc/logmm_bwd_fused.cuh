// Both gradients of the log-add joiner's denominator in ONE pass over the Ef planes
// (see logmm_bwd_tc.cuh for the algebra):
//     grad_f[t,v] = Ef[t,v] * sum_u P[t,u] Eg[u,v]          (GEMM 1, per 128-frame block)
//     grad_g[u,v] = Eg[u,v] * sum_t P[t,u] Ef[t,v]          (GEMM 2, accumulated over the frame blocks)
// A work item is one utterance and one slab of 64 vocabulary entries; the CTA walks the frame blocks
// of that slab.  Per frame block one shared-memory stage holds the P tile (128 t x 128 u, hi + lo)
// and the Ef tile (128 t x 64 v, hi + lo):
//   * the P tile is the K-major A operand of GEMM 1 and, through a second descriptor over the very
//     same bytes, the MN-major (transposed) A operand of GEMM 2;
//   * the Ef tile is the B operand of GEMM 2 and, read back by the epilogue threads as hi + lo, the
//     factor Ef of grad_f, so f is never read; the finished fp32 tile of grad_f is written over the
//     lo planes of the P tile (free once both GEMMs are done, same number of bytes) and leaves
//     through one TMA store.  So the Ef part of a stage goes back to the producer as soon as the
//     epilogue threads have read it and the hi planes of P as soon as the MMAs are done; only the
//     load of the next lo planes of P (32 KB out of L2) has to wait for the store.
// Eg (128 u x 64 v, hi + lo) stays resident for the item as B operand of GEMM 1; grad_g is finished
// by the epilogue threads straight from / to global memory (it is a tenth of the traffic).
// HBM traffic: Ef planes read once, grad_f written once, g and grad_g once.
//
// Warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-9 = epilogue, warp 10 = TMA stores.  Needs
// U+1 <= 128.  Waits are bounded as in k_logmm_tc; any failure raises the flag that makes the exact
// kernel behind this one redo the work.
#pragma once

#include "logmm_bwd_tc.cuh"

namespace ctct {

constexpr int FU_T = 128, FU_V = 64;                 // frame block, vocabulary slab
constexpr int FU_P_BYTES = 4 * BW_A_PLANE;           // P tile: hi u-block 0, hi u-block 1, lo 0, lo 1 (16 KB each)
constexpr int FU_E_BYTES = 2 * BW_A_PLANE;           // Ef tile: hi (128 t-rows x 128 B), lo
constexpr int FU_STAGE_BYTES = FU_P_BYTES + FU_E_BYTES;  // 96 KB
constexpr int FU_STAGES = 2;
constexpr int FU_EG_BYTES = 2 * BW_A_PLANE;          // Eg slab: hi (128 u-rows x 128 B), lo
constexpr int FU_THREADS = 64 + 32 * BW_EPI_WARPS + 32;
constexpr int FU_SMEM_BYTES = FU_STAGES * FU_STAGE_BYTES + FU_EG_BYTES + 1024 + 256;

struct DenBwdFusedArgs {
    const float *g;    // (B, U1, V)
    const float *mg;   // (B, U1)
    float *grad_g;     // (B, U1, V)
    int T, U1, V;
    int slabs, items;  // vocabulary slabs per utterance, slabs * B
    int *flags;        // [0] a bounded wait ran out, [1] forward underflow (exact kernel needed)
};

// maps: P planes as stored (64 u x 128 t box), Ef planes (64 v x 64 t box), Eg planes (64 v x 64 u box),
// grad_f (fp32, 32 v x 128 t box, 128-byte swizzle)
__global__ void __launch_bounds__(FU_THREADS, 1) k_den_bwd_fused(const __grid_constant__ CUtensorMap map_ph,
                                                                 const __grid_constant__ CUtensorMap map_pl,
                                                                 const __grid_constant__ CUtensorMap map_fh,
                                                                 const __grid_constant__ CUtensorMap map_fl,
                                                                 const __grid_constant__ CUtensorMap map_gh,
                                                                 const __grid_constant__ CUtensorMap map_gl,
                                                                 const __grid_constant__ CUtensorMap map_out,
                                                                 const DenBwdFusedArgs a) {
    extern __shared__ unsigned char fu_raw[];
    __shared__ int skip;
    pdl_wait();
    if (threadIdx.x == 0) skip = a.flags[0] | a.flags[1];
    __syncthreads();
    if (skip) return;  // the exact kernel does the work (same decision for the whole CTA)
    const unsigned raw = smem_u32(fu_raw);
    const unsigned ring = (raw + 1023u) & ~1023u;
    const unsigned eg = ring + FU_STAGES * FU_STAGE_BYTES;
    const unsigned bars = eg + FU_EG_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };              // stage loaded
    auto empty_bar = [&](int s) { return bars + 8u * (2 + s); };       // Ef part free again (the epilogue has read it)
    auto p_hi_empty = [&](int s) { return bars + 8u * (14 + s); };     // hi planes of P free again (both GEMMs complete)
    auto p_lo_empty = [&](int s) { return bars + 8u * (16 + s); };     // lo planes of P free again (both GEMMs complete AND
                                                                       // the store of the grad_f tile written over them has read it)
    auto done_bar = [&](int s) { return bars + 8u * (4 + s); };        // both GEMMs of the stage complete
    auto ready_bar = [&](int s) { return bars + 8u * (6 + s); };       // grad_f tile written, store may go
    auto d1_empty = [&](int q) { return bars + 8u * (8 + q); };        // accumulator of GEMM 1 read out
    const unsigned eg_full = bars + 8u * 10, eg_empty = bars + 8u * 11;
    const unsigned d2_full = bars + 8u * 12, d2_empty = bars + 8u * 13;
    constexpr int NBARS = 18;
    const unsigned slot_addr = bars + 8u * NBARS;
    unsigned *slot_ptr = reinterpret_cast<unsigned *>(fu_raw + (slot_addr - raw));
    unsigned char *ring_ptr = fu_raw + (ring - raw);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntb = (a.T + FU_T - 1) / FU_T;
    constexpr unsigned TMEM_COLS = 256;  // D1[0] at 0, D1[1] at 64, D2 at 128

    if (threadIdx.x == 0) {
        // full: three arrivals (Ef loads, P hi loads, P lo loads); p_lo_empty: two (MMA commit, store thread);
        // d2_empty: one per epilogue warp
        for (int q = 0; q < NBARS; ++q) mbar_init(bars + 8u * q, q == 13 ? BW_EPI_WARPS : (q < 2 ? 3 : (q >= 16 ? 2 : 1)));
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

    auto item_coords = [&](int item, int &v0, int &b) {
        v0 = (item % a.slabs) * FU_V;
        b = item / a.slabs;
    };

    if (warp == 0 && lane == 0) {
        // ---- TMA producer
        unsigned tbc = 0;
        unsigned armed = 0, armed_parity = 0;  // bits 0,1: full_bar armed / its parity; bit 8: eg_full
        for (int item = blockIdx.x, i = 0; item < a.items && ok; item += gridDim.x, ++i) {
            int v0, b;
            item_coords(item, v0, b);
            ok = mbar_wait(eg_empty, (i & 1) ^ 1);
            if (!ok) break;
            mbar_expect_tx(eg_full, FU_EG_BYTES);
            tma_load_3d(eg, &map_gh, eg_full, v0, 0, b);
            tma_load_3d(eg + BW_A_PLANE / 2, &map_gh, eg_full, v0, 64, b);
            tma_load_3d(eg + BW_A_PLANE, &map_gl, eg_full, v0, 0, b);
            tma_load_3d(eg + BW_A_PLANE + BW_A_PLANE / 2, &map_gl, eg_full, v0, 64, b);
            armed |= 1u << 8;
            armed_parity = (armed_parity & ~(1u << 8)) | (static_cast<unsigned>(i & 1) << 8);
            for (int tb = 0; tb < ntb; ++tb, ++tbc) {
                const int s = tbc & 1;
                const unsigned ph = (tbc >> 1) & 1;
                // the Ef part comes back as soon as the epilogue threads have read it, the hi planes of P when the
                // MMAs are done, the lo planes (which the grad_f tile is written over) when the store has read them
                const unsigned st = ring + s * FU_STAGE_BYTES;
                const unsigned bar = full_bar(s);
                const int t0 = tb * FU_T;
                ok = mbar_wait(empty_bar(s), ph ^ 1);
                if (!ok) break;
                mbar_expect_tx(bar, FU_E_BYTES);
                const unsigned ef = st + FU_P_BYTES;
                tma_load_3d(ef, &map_fh, bar, v0, t0, b);
                tma_load_3d(ef + BW_A_PLANE / 2, &map_fh, bar, v0, t0 + 64, b);
                tma_load_3d(ef + BW_A_PLANE, &map_fl, bar, v0, t0, b);
                tma_load_3d(ef + BW_A_PLANE + BW_A_PLANE / 2, &map_fl, bar, v0, t0 + 64, b);
                armed |= 1u << s;
                armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
                ok = mbar_wait(p_hi_empty(s), ph ^ 1);
                if (!ok) {
                    mbar_expect_tx(bar, 0);  // the missing arrivals of the phase, so that the Ef loads can be waited for
                    mbar_expect_tx(bar, 0);
                    break;
                }
                mbar_expect_tx(bar, FU_P_BYTES / 2);
                tma_load_3d(st, &map_ph, bar, 0, t0, b);
                tma_load_3d(st + BW_A_PLANE, &map_ph, bar, 64, t0, b);
                ok = mbar_wait(p_lo_empty(s), ph ^ 1);
                if (!ok) {
                    mbar_expect_tx(bar, 0);
                    break;
                }
                mbar_expect_tx(bar, FU_P_BYTES / 2);
                tma_load_3d(st + 2 * BW_A_PLANE, &map_pl, bar, 0, t0, b);
                tma_load_3d(st + 3 * BW_A_PLANE, &map_pl, bar, 64, t0, b);
            }
        }
        if (!ok) atomicExch(a.flags, 1);
        // no copy of this CTA may still be in flight when it exits (bounded; immediate when all went well)
        for (int s = 0; s < FU_STAGES; ++s)
            if (armed & (1u << s)) mbar_wait(full_bar(s), (armed_parity >> s) & 1);
        if (armed & (1u << 8)) mbar_wait(eg_full, (armed_parity >> 8) & 1);
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        const unsigned idesc_common = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |  // fp32 acc, bf16 x bf16, B MN-major
                                      (static_cast<unsigned>(FU_V >> 3) << 17) | (static_cast<unsigned>(128 >> 4) << 24);
        const unsigned idesc1 = idesc_common;               // A = P, K-major
        const unsigned idesc2 = idesc_common | (1u << 15);  // A = P transposed, MN-major
        unsigned tbc = 0;
        for (int item = blockIdx.x, i = 0; item < a.items && ok; item += gridDim.x, ++i) {
            ok = mbar_wait(eg_full, i & 1);
            if (!ok) break;
            for (int tb = 0; tb < ntb; ++tb, ++tbc) {
                const int s = tbc & 1, q = tbc & 1;
                ok = mbar_wait(full_bar(s), (tbc >> 1) & 1) && mbar_wait(d1_empty(q), ((tbc >> 1) & 1) ^ 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned st = ring + s * FU_STAGE_BYTES;
                const unsigned d1 = tmem_base + static_cast<unsigned>(q) * FU_V;
                const unsigned d2 = tmem_base + 2u * FU_V;
                // GEMM 1: D1[t, v] = sum_u P[t, u] Eg[u, v]; two u-blocks of 64
                const unsigned pa = umma_lo(st);                         // P hi, u-block 0 (K-major)
                const unsigned gb = umma_lo_mn(eg, BW_A_PLANE / 2);      // Eg hi, u-rows 0.. (MN-major)
#pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        if (kb * 64 + k4 * 16 >= a.U1) continue;  // columns of P beyond U+1 are zero
                        const uint64_t ah = umma_pack(pa + (kb * BW_A_PLANE + k4 * 32) / 16);
                        const uint64_t al = umma_pack(pa + (2 * BW_A_PLANE + kb * BW_A_PLANE + k4 * 32) / 16);
                        const uint64_t bh = umma_pack(gb + (kb * 8192 + k4 * 2048) / 16);
                        const uint64_t bl = umma_pack(gb + (BW_A_PLANE + kb * 8192 + k4 * 2048) / 16);
                        umma_bf16(d1, ah, bh, idesc1, (kb | k4) ? 1u : 0u);
                        umma_bf16(d1, ah, bl, idesc1, 1u);
                        umma_bf16(d1, al, bh, idesc1, 1u);
                    }
                }
                if (tb == ntb - 1) umma_commit(eg_empty);  // Eg may be replaced once these MMAs are done
                if (tb == 0) {
                    ok = mbar_wait(d2_empty, (i & 1) ^ 1);  // the previous item's grad_g has left TMEM
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                // GEMM 2: D2[u, v] += sum_t P[t, u] Ef[t, v]; the P tile read transposed: rows are t,
                // the two 64-wide chunks of u are the two u-block tiles (BW_A_PLANE apart)
                const unsigned pt = umma_lo_mn(st, BW_A_PLANE);
                const unsigned fb = umma_lo_mn(st + FU_P_BYTES, BW_A_PLANE / 2);
#pragma unroll
                for (int k4 = 0; k4 < FU_T / 16; ++k4) {
                    const uint64_t ah = umma_pack(pt + (k4 * 2048) / 16);
                    const uint64_t al = umma_pack(pt + (2 * BW_A_PLANE + k4 * 2048) / 16);
                    const uint64_t bh = umma_pack(fb + (k4 * 2048) / 16);
                    const uint64_t bl = umma_pack(fb + (BW_A_PLANE + k4 * 2048) / 16);
                    umma_bf16(d2, ah, bh, idesc2, (tb | k4) ? 1u : 0u);
                    umma_bf16(d2, ah, bl, idesc2, 1u);
                    umma_bf16(d2, al, bh, idesc2, 1u);
                }
                umma_commit(done_bar(s));
                umma_commit(p_hi_empty(s));
                umma_commit(p_lo_empty(s));
                if (tb == ntb - 1) umma_commit(d2_full);
            }
        }
        if (!ok) atomicExch(a.flags, 1);
    } else if (warp >= 2 && warp < 2 + BW_EPI_WARPS) {
        // ---- epilogue warps.  A warp may read the TMEM lanes [32 * (warp % 4), +32): one row per
        // thread; the two warps of a lane quarter take 32 of the 64 columns each.
        const int part = warp & 3;
        const int c = (warp - 2) >> 2;
        const int r = part * 32 + lane;
        const bool leader = (threadIdx.x == 64);
        // the same verdict in all epilogue warps (they meet at barriers, so they must leave together)
        auto all_agree = [](bool mine) -> bool {
            unsigned all;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.u32 q, %1, 0;\n\t"
                "bar.red.and.pred p, 1, %2, q;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(all)
                : "r"(static_cast<unsigned>(mine)), "n"(32 * BW_EPI_WARPS)
                : "memory");
            return all != 0;
        };
        unsigned tbc = 0;
        for (int item = blockIdx.x, i = 0; item < a.items; item += gridDim.x, ++i) {
            int v0, b;
            item_coords(item, v0, b);
            // this thread's 32 values of g and its row maximum for the item's grad_g: requested now,
            // needed only after the last frame block
            const int64_t grow = static_cast<int64_t>(b) * a.U1 + r;
            const int gcol = v0 + c * 32;
            float4 gx[8];
            float mgr = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) gx[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < a.U1) {
                mgr = __ldg(a.mg + grow);
                const float4 *src = reinterpret_cast<const float4 *>(a.g + grow * a.V + gcol);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (gcol + 4 * j < a.V) gx[j] = __ldg(src + j);
            }
            for (int tb = 0; tb < ntb; ++tb, ++tbc) {
                const int s = tbc & 1, q = tbc & 1;
                ok = all_agree(mbar_wait(done_bar(s), (tbc >> 1) & 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char *ef = ring_ptr + s * FU_STAGE_BYTES + FU_P_BYTES;
                // Ef[r, 32c .. 32c+32) = hi + lo from the two planes (row r is 128 bytes, 16-byte units swizzled)
                float e[32];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int unit = ((4 * c + j) ^ (r & 7)) << 4;
                    const uint4 h = *reinterpret_cast<const uint4 *>(ef + r * 128 + unit);
                    const uint4 l = *reinterpret_cast<const uint4 *>(ef + BW_A_PLANE + r * 128 + unit);
                    const unsigned hw[4] = {h.x, h.y, h.z, h.w}, lw[4] = {l.x, l.y, l.z, l.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        e[8 * j + 2 * k] = __uint_as_float(hw[k] << 16) + __uint_as_float(lw[k] << 16);
                        e[8 * j + 2 * k + 1] = __uint_as_float(hw[k] & 0xffff0000u) + __uint_as_float(lw[k] & 0xffff0000u);
                    }
                }
                unsigned d[32];
                tmem_ld_32x32(tmem_base + (static_cast<unsigned>(part * 32) << 16) + q * FU_V + c * 32, d);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                // every thread has read its part of the Ef tile: the producer may load the next one into it
                asm volatile("bar.sync 2, %0;" ::"n"(32 * BW_EPI_WARPS) : "memory");
                if (leader) mbar_arrive(empty_bar(s));
                // the grad_f tile goes over the lo planes of the P tile (both GEMMs that read them are complete)
                unsigned char *orow = ring_ptr + s * FU_STAGE_BYTES + (2 + c) * BW_A_PLANE + r * 128;  // column half c of the fp32 tile
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float4 o;
                    o.x = e[4 * j] * __uint_as_float(d[4 * j]);
                    o.y = e[4 * j + 1] * __uint_as_float(d[4 * j + 1]);
                    o.z = e[4 * j + 2] * __uint_as_float(d[4 * j + 2]);
                    o.w = e[4 * j + 3] * __uint_as_float(d[4 * j + 3]);
                    *reinterpret_cast<float4 *>(orow + ((j ^ (r & 7)) << 4)) = o;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // tile writes -> visible to the TMA store
                asm volatile("bar.sync 1, %0;" ::"n"(32 * BW_EPI_WARPS) : "memory");
                if (leader) {
                    mbar_arrive(d1_empty(q));
                    mbar_arrive(ready_bar(s));
                }
            }
            if (!ok) break;
            // grad_g of this item: D2[u, v] * exp(g[u, v] - mg[u]), rows straight from / to global memory
            ok = all_agree(mbar_wait(d2_full, i & 1));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned d[32];
            tmem_ld_32x32(tmem_base + (static_cast<unsigned>(part * 32) << 16) + 2 * FU_V + c * 32, d);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(d2_empty);
            if (r < a.U1) {
                float4 *dst = reinterpret_cast<float4 *>(a.grad_g + grow * a.V + gcol);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (gcol + 4 * j < a.V) {
                        const float d0 = __uint_as_float(d[4 * j]), d1v = __uint_as_float(d[4 * j + 1]);
                        const float d2v = __uint_as_float(d[4 * j + 2]), d3 = __uint_as_float(d[4 * j + 3]);
                        float4 o;
                        // a zero sum stays zero even where exp() would overflow or g is -inf
                        o.x = d0 != 0.0f ? d0 * ex2((gx[j].x - mgr) * LOG2E) : 0.0f;
                        o.y = d1v != 0.0f ? d1v * ex2((gx[j].y - mgr) * LOG2E) : 0.0f;
                        o.z = d2v != 0.0f ? d2v * ex2((gx[j].z - mgr) * LOG2E) : 0.0f;
                        o.w = d3 != 0.0f ? d3 * ex2((gx[j].w - mgr) * LOG2E) : 0.0f;
                        __stcs(dst + j, o);
                    }
                }
            }
        }
        if (!ok && lane == 0) atomicExch(a.flags, 1);
    } else if (warp == 2 + BW_EPI_WARPS && lane == 0) {
        // ---- store thread: one TMA store per finished grad_f tile; the P part of the stage goes back to
        // the producer as soon as the store has read it
        unsigned tbc = 0;
        for (int item = blockIdx.x; item < a.items && ok; item += gridDim.x) {
            int v0, b;
            item_coords(item, v0, b);
            for (int tb = 0; tb < ntb; ++tb, ++tbc) {
                const int s = tbc & 1;
                ok = mbar_wait(ready_bar(s), (tbc >> 1) & 1);
                if (!ok) break;
                const unsigned tile = ring + s * FU_STAGE_BYTES + 2 * BW_A_PLANE;
                tma_store_3d(&map_out, tile, v0, tb * FU_T, b);
                tma_store_3d(&map_out, tile + BW_A_PLANE, v0 + 32, tb * FU_T, b);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                mbar_arrive(p_lo_empty(s));
            }
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (!ok) atomicExch(a.flags, 1);
    }
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace ctct

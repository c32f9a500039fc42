// Shared device helpers of the CTC-Transducer kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ctct {

// Stand-in for log(0).  Finite, so that sums and differences of "impossible" states
// never produce NaN; anything below NEG_TEST counts as impossible.
constexpr float NEG = -1.0e30f;
constexpr float NEG_TEST = -1.0e29f;
constexpr float LOG2E = 1.4426950408889634f;
constexpr double LN2 = 0.6931471805599453;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// log2(2^a + 2^b) for finite a, b.
__device__ __forceinline__ float lse2(float a, float b) {
    const float m = fmaxf(a, b);
    const float n = fminf(a, b);
    return m + lg2(1.0f + ex2(n - m));
}

// log2(2^a + 2^b + 2^c) for finite a, b, c.
__device__ __forceinline__ float lse3(float a, float b, float c) {
    const float m = fmaxf(a, fmaxf(b, c));
    return m + lg2(ex2(a - m) + ex2(b - m) + ex2(c - m));
}

// natural-log input value -> clamped log2 value
__device__ __forceinline__ float to_log2(float lp) { return fmaxf(lp * LOG2E, NEG); }

__device__ __forceinline__ float load_as_float(const float *p) { return __ldg(p); }
__device__ __forceinline__ float load_as_float(const __half *p) {
    return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(p))));
}
__device__ __forceinline__ float load_as_float(const __nv_bfloat16 *p) {
    return __bfloat162float(__ushort_as_bfloat16(__ldg(reinterpret_cast<const unsigned short *>(p))));
}

// Isolated element reads (one element out of a 2-4 KB vocabulary row): non-coherent, no L1
// allocation, and the smallest L2 fetch granule, so that a 4-byte read does not pull a 128-byte
// line out of HBM.
__device__ __forceinline__ float load_sparse(const float *p) {
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::64B.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float load_sparse(const __half *p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::64B.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ float load_sparse(const __nv_bfloat16 *p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::64B.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __bfloat162float(__ushort_as_bfloat16(v));
}

// The same reads without a fill-size hint: for a source in pinned host memory, where every
// byte asked for crosses PCIe.
__device__ __forceinline__ float load_remote(const float *p) {
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float load_remote(const __half *p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ float load_remote(const __nv_bfloat16 *p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __bfloat162float(__ushort_as_bfloat16(v));
}

// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may
// start while the kernel before it in the stream is still running; pdl_wait() returns once that
// kernel has completed and its writes are visible (at once when nothing is pending, or when the
// launch did not carry the attribute).  pdl_trigger() lets the NEXT kernel in the stream start
// launching once every block of this one has called it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__host__ __device__ __forceinline__ int64_t pad4(int64_t x) { return (x + 3) & ~int64_t(3); }

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src) {
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A slice of a buffer that extra thread blocks of a kernel fill with zeros while the kernel's own
// blocks do their work.  The dense gradient of the backward pass is all zeros but for <= 3
// columns per row, and clearing it needs nothing the forward pass computes, so the forward
// kernels carry its clearing: blocks [first_block, gridDim.x) of a launch clear CLEAR_CHUNK 16-byte
// vectors each (many short blocks reach the HBM write peak, a persistent grid does not).
struct ClearSlice {
    uint4 *ptr;                 // nullptr: no clearing in this launch
    unsigned long long vecs;    // 16-byte vectors in this slice
    int tail;                   // extra bytes after the last vector (only on the final slice)
    unsigned first_block;       // blocks below this index do the kernel's own work
};

constexpr unsigned CLEAR_TILE_BYTES = 16384;                       // zeroed shared-memory tile
// Bulk stores per clearing block.  Short blocks win: measured at the benchmark shape (1.09 GB beside 64
// lattice CTAs) 16 / 32 / 48 / 64 / 96 / 256 / 1024 KB per block give 158.5 / 158.7 / 159.9 / 160.1 /
// 161.7 / 168.8 / 174.3 us for the launch (tile sizes of 8, 16 and 32 KB make no difference).
constexpr unsigned CLEAR_TILES_PER_BLOCK = 2;
constexpr unsigned CLEAR_CHUNK = CLEAR_TILE_BYTES / 16 * CLEAR_TILES_PER_BLOCK;  // 16-byte vectors per block

// Returns true if this block is a clearing block (and has done its clearing).
// The block zeroes a 16 KB tile of its shared memory once and one thread then streams it out with
// 1-D bulk (TMA) stores: a handful of instructions per 32 KB, so the clearing hardly touches the
// load/store pipes that the kernel's own blocks on the same SM depend on.  `smem` must offer
// CLEAR_TILE_BYTES (16-byte aligned); with less, plain 16-byte stores are used.
__device__ __forceinline__ bool clear_role(const ClearSlice &c, void *smem, unsigned smem_bytes) {
    if (c.ptr == nullptr || blockIdx.x < c.first_block) return false;
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    const unsigned long long chunk = blockIdx.x - c.first_block;
    const unsigned long long base = chunk * CLEAR_CHUNK;
    uint4 *p = c.ptr + base;
    const unsigned long long left = c.vecs > base ? c.vecs - base : 0;
    const unsigned n = left < CLEAR_CHUNK ? static_cast<unsigned>(left) : CLEAR_CHUNK;
    if (chunk == 0 && static_cast<int>(threadIdx.x) < c.tail) reinterpret_cast<unsigned char *>(c.ptr + c.vecs)[threadIdx.x] = 0;
    if (smem_bytes >= CLEAR_TILE_BYTES) {
        uint4 *tile = static_cast<uint4 *>(smem);
        for (unsigned i = threadIdx.x; i < CLEAR_TILE_BYTES / 16; i += blockDim.x) tile[i] = z;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> async proxy reads
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned src = static_cast<unsigned>(__cvta_generic_to_shared(tile));
            unsigned done = 0;
            while (done < n) {
                const unsigned v = (n - done) < CLEAR_TILE_BYTES / 16 ? (n - done) : CLEAR_TILE_BYTES / 16;
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(p + done), "r"(src),
                             "r"(v * 16u)
                             : "memory");
                done += v;
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the tile must outlive the reads
        }
        return true;
    }
    const unsigned nt = blockDim.x;
    unsigned i = threadIdx.x;
    for (; i + 3 * nt < n; i += 4 * nt) {  // four independent stores in flight per thread
        p[i] = z;
        p[i + nt] = z;
        p[i + 2 * nt] = z;
        p[i + 3 * nt] = z;
    }
    for (; i < n; i += nt) p[i] = z;
    return true;
}

// Ragged variant: extra blocks of a launch zero the PADDING ROWS of an (N,T,U1,V) tensor, i.e. for every
// (n,t) slab the contiguous block of rows u > ly[n] (the whole slab when t >= lx[n]).  Block
// first_block + s handles slab s.  The loss on raw logits uses it to move the zero half of its dense
// gradient under the latency-bound lattice.  row_bytes must be a multiple of 16, `out` 16-byte aligned.
struct PadClear {
    unsigned char *out;        // nullptr: none
    const int *lx, *ly;
    int T, U1;
    unsigned row_bytes;        // V * sizeof(element)
    unsigned first_block;
    unsigned slabs;            // N * T
    unsigned parts;            // blocks per slab: block first_block + slab * parts + p takes bytes [p, p + 1) * PAD_PART_BYTES of the slab
};
constexpr unsigned PAD_PART_BYTES = CLEAR_TILE_BYTES * CLEAR_TILES_PER_BLOCK;  // short blocks, as for the flat clearing

// Returns true if this block is a padding-clearing block (and has done its work).  `smem`: at least
// CLEAR_TILE_BYTES, 16-byte aligned.
__device__ __forceinline__ bool pad_clear_role(const PadClear &c, void *smem) {
    if (c.out == nullptr || blockIdx.x < c.first_block) return false;
    const unsigned idx = blockIdx.x - c.first_block;
    const unsigned slab = idx / c.parts, part = idx - slab * c.parts;
    if (slab >= c.slabs) return true;
    const int n = static_cast<int>(slab / static_cast<unsigned>(c.T));
    const int t = static_cast<int>(slab - static_cast<unsigned>(n) * c.T);
    const int Un = (t < c.lx[n]) ? min(c.ly[n], c.U1 - 1) : -1;
    // this block's window of the slab, cut to the slab's padding rows [(Un + 1) * row_bytes, U1 * row_bytes)
    const unsigned long long slab_bytes = static_cast<unsigned long long>(c.U1) * c.row_bytes;
    const unsigned long long pad_lo = static_cast<unsigned long long>(Un + 1) * c.row_bytes;
    unsigned long long lo = static_cast<unsigned long long>(part) * PAD_PART_BYTES;
    unsigned long long hi = lo + PAD_PART_BYTES;
    lo = lo < pad_lo ? pad_lo : lo;
    hi = hi > slab_bytes ? slab_bytes : hi;
    if (lo >= hi) return true;
    unsigned char *p = c.out + static_cast<unsigned long long>(slab) * slab_bytes + lo;
    const unsigned long long bytes = hi - lo;
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    uint4 *tile = static_cast<uint4 *>(smem);
    for (unsigned i = threadIdx.x; i < CLEAR_TILE_BYTES / 16; i += blockDim.x) tile[i] = z;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> async proxy reads
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned src = static_cast<unsigned>(__cvta_generic_to_shared(tile));
        unsigned long long done = 0;
        while (done < bytes) {
            const unsigned long long left = bytes - done;
            const unsigned v = left < CLEAR_TILE_BYTES ? static_cast<unsigned>(left) : CLEAR_TILE_BYTES;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(p + done), "r"(src), "r"(v)
                         : "memory");
            done += v;
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the tile must outlive the reads
    }
    return true;
}

}  // namespace ctct

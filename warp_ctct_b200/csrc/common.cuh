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

}  // namespace ctct

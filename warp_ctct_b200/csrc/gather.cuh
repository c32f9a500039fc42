// Gather kernels: pick the blank, "repeat current label" and "emit next label" log-probs
// out of every vocabulary row of the joint tensor.
//
// Replaces the index build + torch.gather of the reference (warp_ctct/__init__.py:124-131,
// CPU twin collect_units in ref_ctct.py:223-230).  One thread per OUTPUT element so that
// the stores are coalesced; the loads are one 32-byte sector each by nature, so the kernel
// lives on memory-level parallelism: PER (four) independent elements per thread, all loads
// issued before the first store.
#pragma once

#include "common.cuh"

namespace ctct {

// `cu` != nullptr: the joint tensor is PACKED, (total rows, V) with only the valid rows of every
// utterance (needs valid_only); the output keeps the padded [N][T][U1] record layout either way.
// INTERNAL = true : out[n][t][u] = one 16-byte record {blank, repeat-label, next-label, 0}, values
//                   converted to log2 units and clamped at NEG; everything outside t < lx,
//                   u <= ly is written as 0
// INTERNAL = false: out[n][t][u][slot]    (the reference's (N,T,U+1,3) layout)
template <typename InT, typename IdxT, bool INTERNAL, int PER = 4>
__global__ void __launch_bounds__(256)
k_gather3(const InT *__restrict__ lp, const int *__restrict__ ys, const int *__restrict__ lx,
          const int *__restrict__ ly, float *__restrict__ out, int T, int U1, int V,
          IdxT total, int mode, const ClearSlice clear, const int64_t *__restrict__ cu = nullptr,
          int64_t packed_rows = 0) {
    // everything before this launch is done before anything here runs; from then on the next launch
    // (the lattice with its clearing blocks) may move in beside this one
    pdl_wait();
    pdl_trigger();
    if (clear_role(clear, nullptr, 0)) return;
    const int valid_only = mode & 1;    // read only frames t < lx[n] and contexts u <= ly[n]
    const bool remote = (mode & 2) != 0;  // lp is pinned host memory
    const IdxT stride = static_cast<IdxT>(clear.ptr ? clear.first_block : gridDim.x) * blockDim.x;
    IdxT e0 = static_cast<IdxT>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int U = U1 - 1;

    for (; e0 < total; e0 += stride * PER) {
        float val[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const IdxT e = e0 + stride * j;
            val[j] = 0.0f;
            if (e < total) {
                int u, k;
                IdxT nt;
                if (INTERNAL) {
                    k = static_cast<int>(e & 3);
                    const IdxT r = e >> 2;
                    u = static_cast<int>(r % static_cast<IdxT>(U1));
                    nt = r / static_cast<IdxT>(U1);
                } else {
                    k = static_cast<int>(e % 3);
                    const IdxT r = e / 3;
                    u = static_cast<int>(r % static_cast<IdxT>(U1));
                    nt = r / static_cast<IdxT>(U1);
                }
                const int n = static_cast<int>(nt / static_cast<IdxT>(T));
                const int t = static_cast<int>(nt - static_cast<IdxT>(n) * T);
                bool take = k < 3;
                if (valid_only) take = take && t < lx[n] && u <= ly[n];
                if (take) {
                    int idx = 0;
                    if (k == 1 && u >= 1) idx = ys[static_cast<int64_t>(n) * U + (u - 1)];
                    // with valid_only the label ys[n,u] is a real one only for u < ly[n]
                    if (k == 2 && u < U && (!valid_only || u < ly[n])) idx = ys[static_cast<int64_t>(n) * U + u];
                    idx = min(max(idx, 0), V - 1);
                    // packed input: utterance n owns rows [cu[n], cu[n+1]), frame-major, ly[n]+1 rows per frame
                    const int64_t row = cu ? cu[n] + static_cast<int64_t>(t) * (ly[n] + 1) + u : static_cast<int64_t>(nt) * U1 + u;
                    float x = 0.0f;
                    // lengths that do not agree with the packed tensor must not read past its end
                    if (cu == nullptr || row < packed_rows) x = remote ? load_remote(lp + row * V + idx) : load_sparse(lp + row * V + idx);
                    val[j] = INTERNAL ? to_log2(x) : x;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const IdxT e = e0 + stride * j;
            if (e < total) out[e] = val[j];
        }
    }
}

// (N,T,U1,3) reference layout -> internal layout (log2 units), zeroing everything outside the valid region.
// Used when the caller hands in pre-gathered log-probs (csrc/binding.cpp:31-34 interface).
__global__ void __launch_bounds__(256)
k_repack_gathered(const float *__restrict__ g, const int *__restrict__ lx, const int *__restrict__ ly,
                  float *__restrict__ out, int T, int U1, int64_t total) {
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int k = static_cast<int>(e & 3);
        const int64_t r = e >> 2;
        const int u = static_cast<int>(r % U1);
        const int64_t nt = r / U1;
        const int n = static_cast<int>(nt / T);
        const int t = static_cast<int>(nt - static_cast<int64_t>(n) * T);
        float v = 0.0f;
        if (k < 3 && t < lx[n] && u <= ly[n]) v = to_log2(g[(nt * U1 + u) * 3 + k]);
        out[e] = v;
    }
}

}  // namespace ctct

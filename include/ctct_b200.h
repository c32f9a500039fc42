/*
 * ctct_b200 -- C ABI of the B200 (sm_100a) CTC-Transducer loss kernels.
 *
 * Plain pointers and sizes only; every pointer is DEVICE memory unless a comment
 * says otherwise.  No entry point allocates, frees or synchronises: the caller
 * owns all buffers (outputs and the scratch "workspace") and passes the CUDA
 * stream to launch on (a cudaStream_t cast to void*, NULL = legacy default).
 * Every function returns 0 on success or a negative CTCT_ERR_* code and never
 * terminates the process (the reference's launchers print and exit(-1),
 * csrc/core.h:5-12).
 *
 * Citations name files of the reference project (maxwellzh/warp-ctct) whose
 * interface each entry point replaces.
 */
#ifndef CTCT_B200_H
#define CTCT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CTCT_OK 0
#define CTCT_ERR_ARG (-1)        /* null pointer, negative size, unknown dtype          */
#define CTCT_ERR_WORKSPACE (-2)  /* workspace missing, too small or misaligned          */
#define CTCT_ERR_LAUNCH (-3)     /* CUDA reported a launch / configuration error        */
#define CTCT_ERR_UNSUPPORTED (-4)/* size outside what the kernels were built for        */

/* element type of the joint tensor and of the dense gradient */
#define CTCT_F32 0
#define CTCT_F16 1
#define CTCT_BF16 2

int ctct_b200_abi_version(void);
const char *ctct_b200_strerror(int code);

/* Number of floats per (utterance, frame) row group of the internal 3-slot layout:
 * contexts padded to a multiple of 4 so that every row starts on 16 bytes. */
int64_t ctct_b200_padded_contexts(int64_t U1);

/* Elements (floats) of the compact gradient buffer `grads3` used between
 * ctct_b200_loss_forward and ctct_b200_loss_backward: N*T*3*padded_contexts(U1). */
size_t ctct_b200_grads3_elems(int64_t N, int64_t T, int64_t U1);

/* Bytes of scratch the forward entry points need (256-byte aligned base). */
size_t ctct_b200_workspace_bytes(int64_t N, int64_t T, int64_t U1, int want_grad);

/*
 * Fused forward of ctct_loss on the full joint tensor.
 * Replaces: the index build + torch.gather + .float() of warp_ctct/__init__.py:124-136,
 * ctct_loss_fwd of csrc/binding.cpp:31-100, and the launchers run_warp_ctct /
 * run_fill_grad of csrc/core.h:14-20 (kernels csrc/gather.cu:36-387).
 *   log_probs (N,T,U1,V) of `dtype`, contiguous;  ys (N,U1-1) int32;  lx, ly (N) int32
 *   costs (N) float32 out: -log-likelihood (the reference's -betas[:,0,0]); +inf when
 *         the utterance has no alignment (lx < ly + adjacent repeats)
 *   grads3 out, only if want_grad: occupancy gradient w.r.t. the three gathered
 *         log-probs per (n,t,u) in the internal layout [n][t][slot][padded u]
 * Labels are only dereferenced for u < ly[n]; frames t >= lx[n] and contexts
 * u > ly[n] of log_probs are never read.
 */
int ctct_b200_loss_forward(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                           const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                           int want_grad, float *costs, float *grads3, void *workspace,
                           size_t workspace_bytes, void *stream);

/*
 * Dense gradient: dense[n,t,u,:] = 0 except the blank column and the columns of
 * labels ys[n,u-1], ys[n,u], which receive grad_out[n] * grads3; columns that
 * coincide add up.  One pass, every byte of `dense` written exactly once.
 * Replaces: CTCTLoss.backward (warp_ctct/__init__.py:31-33) plus the autograd
 * backward of .float() and of the gather at :131 (zeros + scatter_add).
 *   dense (N,T,U1,V) of `dtype` out; for 16-bit dtypes each product is rounded
 *   to the dtype before the add, as the reference's cast-then-scatter does.
 */
int ctct_b200_loss_backward(const float *grads3, const float *grad_out, const int32_t *ys,
                            const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1,
                            int64_t V, int dtype, void *dense, void *stream);

/*
 * The gather alone, in the reference's layout: gathered[n,t,u,0..2] =
 * log_probs[n,t,u,{0, ys[n,u-1], ys[n,u]}] converted to float32 (slots without a
 * label read column 0).  Replaces collect_units (ref_ctct.py:223-230) /
 * warp_ctct/__init__.py:124-135.  valid_only != 0 skips t >= lx[n] or u > ly[n]
 * (those outputs are written as 0 and padded labels are not dereferenced);
 * valid_only == 0 copies every row and clamps labels into [0, V).
 */
int ctct_b200_gather(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                     const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int valid_only,
                     float *gathered, void *stream);

/*
 * Forward from pre-gathered log-probs, the reference's extension entry point
 * ctct_loss_fwd(log_probs(N,T,U1,3), ys, lx, ly, requires_grad) of
 * csrc/binding.cpp:31-100 (launchers csrc/core.h:14-20).
 *   gathered (N,T,U1,3) float32;  grads (N,T,U1,3) float32 out (zeros outside
 *   t < lx, u <= ly), written only if want_grad.
 */
int ctct_b200_gathered_forward(const float *gathered, const int32_t *ys, const int32_t *lx,
                               const int32_t *ly, int64_t N, int64_t T, int64_t U1, int want_grad,
                               float *costs, float *grads, void *workspace, size_t workspace_bytes,
                               void *stream);

/*
 * Test hook: after a forward with want_grad on the same workspace, write the
 * forward/backward variables in natural-log units, unshifted coordinates:
 *   alpha[n,t,s] for t in [0,T), beta_next[n,t,s] = beta(t+1, s), s in [0, 2*(U1-1)+1);
 *   unreachable states are -inf, rows t >= lx[n] and states s > 2*ly[n] are -inf.
 * Counterpart of the tables of ref_fw_simple / ref_bw_simple (ref_ctct.py:6-74).
 *   ll_alpha, ll_beta (N) float64 out: log-likelihood from either direction.
 */
int ctct_b200_export_tables(const void *workspace, size_t workspace_bytes, const int32_t *lx,
                            const int32_t *ly, int64_t N, int64_t T, int64_t U1, double *alpha,
                            double *beta_next, double *ll_alpha, double *ll_beta, void *stream);

/*
 * Optional per-kernel timing for benchmarks (no counterpart in the reference).  While
 * enabled, every ctct_b200_loss_forward records CUDA events on its stream before the gather,
 * after the gather, after the lattice and after the occupancy-gradient kernel, and every
 * ctct_b200_loss_backward records one before and one after the dense-gradient kernel.
 * Events are created once by _enable (room for max_calls calls, per calling thread) and
 * destroyed by _disable; nothing is recorded when profiling is off.
 *   ctct_b200_profile_read: waits for the recorded events, writes for call i
 *     kind[i] (0 forward, 1 backward) and ms[4*i .. 4*i+2] = {gather, lattice, fill_grad}
 *     or {dense gradient, 0, 0}; returns the number of calls recorded (<= capacity) or a
 *     negative error code, and rewinds the recorder.
 */
int ctct_b200_profile_enable(int max_calls);
int ctct_b200_profile_read(float *ms, int *kind, int capacity);
int ctct_b200_profile_disable(void);

#ifdef __cplusplus
}
#endif
#endif /* CTCT_B200_H */

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
#define CTCT_ERR_STATIC_SCRATCH (-5) /* problem needs more scratch than the built-in buffer holds */

/* Largest U+1 (label contexts per utterance) any entry point takes: one staged pair of lattice
 * rows (32 bytes per context) must fit the shared memory of a thread block.
 * ctct_b200_workspace_bytes returns 0 beyond it and the forward entry points refuse with
 * CTCT_ERR_UNSUPPORTED before anything is launched. */
#define CTCT_MAX_U1 7019

/* element type of the joint tensor and of the dense gradient */
#define CTCT_F32 0
#define CTCT_F16 1
#define CTCT_BF16 2

int ctct_b200_abi_version(void);
const char *ctct_b200_strerror(int code);

/* Elements (floats) of the compact gradient buffer `grads3` used between
 * ctct_b200_loss_forward and ctct_b200_loss_backward: one 16-byte record
 * {blank, repeat-label, next-label, 0} per (n,t,u), i.e. N*T*U1*4 floats; the buffer
 * must be 16-byte aligned. */
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
 *         log-probs per (n,t,u), one 16-byte record {g0,g1,g2,0} each
 * Labels are only dereferenced for u < ly[n]; frames t >= lx[n] and contexts
 * u > ly[n] of log_probs are never read.
 * A label outside [0, V) is CLAMPED into that range, silently, by every kernel that indexes the
 * vocabulary with it (gather, patches of the dense gradients, the simple-loss composition): the
 * result is then a finite loss for a different label sequence.  The reference's torch.gather
 * raises a device-side assert for such a label instead; validate labels on the host if they
 * may be corrupt.
  *   log_probs may also point to pinned (page-locked, device-accessible) HOST memory: the gather
 *   kernel is the only reader and fetches just the three elements it needs per row over PCIe.
 *   Every other pointer must be device memory.
 */
int ctct_b200_loss_forward(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                           const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                           int want_grad, float *costs, float *grads3, void *workspace,
                           size_t workspace_bytes, void *stream);

/*
 * ctct_b200_loss_forward without a caller-provided workspace.  (No counterpart in the
 * reference: its host layer always allocates with torch.)
 *
 * For callers that are not allowed to allocate device memory at the time of the call: a
 * plug-in inside a host application that hands out all device memory at start-up and forbids
 * cudaMalloc afterwards, or a latency-critical loop in which the implicit device-wide
 * synchronisation of an allocation is not acceptable, and that have no caching allocator of
 * their own to take a workspace from.  Inputs and outputs are still the caller's buffers.
 *
 * The scratch lives in a fixed array inside the library's device image,
 * CTCT_NOALLOC_SCRATCH_BYTES (32 MiB) large; every GPU that loads the library carries that array
 * until the process exits.  A problem whose ctct_b200_workspace_bytes(N,T,U1,want_grad)
 * exceeds it is rejected with CTCT_ERR_STATIC_SCRATCH before anything is launched (the first
 * benchmark shape, N=32,T=256,U1=65 with gradient, needs 24.4 MiB).  The function calls no
 * cudaMalloc/cudaFree and no allocating library routine.
 *
 * The first call on each device looks up the array's device address once (with that device
 * current) and caches it; make that first call outside any stream capture.
 * All calls share the one array and it keeps whatever the previous call left there; the
 * kernels write every scratch location before they read it, so nothing has to be cleared.
 * Two calls that overlap on the same GPU (different streams or host threads) race on the
 * array: serialise them, or give all but one of them the workspace variant.
 * Same arguments and results as ctct_b200_loss_forward otherwise.
 */
#define CTCT_NOALLOC_SCRATCH_BYTES (32u << 20)
int ctct_b200_loss_forward_noalloc(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                                   const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                                   int want_grad, float *costs, float *grads3, void *stream);

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
 * The same pair with the reduction of warp_ctct/__init__.py:138-147 folded in, so that no
 * separate reduction kernels run:  loss = sum_n costs[n] * w[n],
 *   w[n] = (average_frames ? 1/lx[n] : 1) * (reduction == 2 ? 1/norm : 1),
 *   reduction: 1 = 'sum', 2 = 'mean' (norm = batch size; a sharded caller passes the global batch).
 * Forward writes costs (N) as before and the scalar *loss (deterministic summation order).
 * Backward takes the gradient of that scalar, grad_loss (ONE float on the device), and scales
 * utterance n by grad_loss[0] * w[n].
 */
int ctct_b200_loss_forward_reduced(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                                   const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                                   int want_grad, int reduction, int average_frames, float norm,
                                   float *costs, float *loss, float *grads3, void *workspace,
                                   size_t workspace_bytes, void *stream);
int ctct_b200_loss_backward_reduced(const float *grads3, const float *grad_loss, int reduction,
                                    int average_frames, float norm, const int32_t *ys, const int32_t *lx,
                                    const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int dtype,
                                    void *dense, void *stream);

/*
 * Most fused form of the forward pass: reduction 0 (none; `loss` unused), 1 ('sum') or 2 ('mean')
 * as above, plus an optional buffer (`clear`, `clear_bytes`, 16-byte aligned) that is filled with
 * zeros by extra thread blocks of the lattice launch.  Passing the dense gradient buffer here
 * moves its HBM-bound clearing under the latency-bound lattice; the backward pass is then
 * ctct_b200_loss_backward_patch instead of ctct_b200_loss_backward[_reduced].
 */
int ctct_b200_loss_forward_fused(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                                 const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                                 int want_grad, int reduction, int average_frames, float norm,
                                 float *costs, float *loss, float *grads3, void *clear, size_t clear_bytes,
                                 void *workspace, size_t workspace_bytes, void *stream);

/*
 * Two-step form of the dense gradient, for callers that can clear the buffer early (before the
 * gradient scale exists; ctct_b200_loss_forward_fused does the clearing inside the lattice launch):
 *   ctct_b200_zero_fill            streams zeros over `bytes` bytes (16-byte aligned buffer);
 *   ctct_b200_loss_backward_patch  writes the <= 3 non-zero columns of every live row into a
 *                                  buffer that is already zero.
 * Together they produce exactly what ctct_b200_loss_backward (scalar_grad == 0, `grad` = N floats)
 * or ctct_b200_loss_backward_reduced (scalar_grad != 0, `grad` = one float) produce in one pass.
 * Same reference counterpart: warp_ctct/__init__.py:31-33 and the autograd backward of :131.
 */
int ctct_b200_zero_fill(void *buffer, size_t bytes, void *stream);
int ctct_b200_loss_backward_patch(const float *grads3, const float *grad, int scalar_grad, int reduction,
                                  int average_frames, float norm, const int32_t *ys, const int32_t *lx,
                                  const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int dtype,
                                  void *dense, void *stream);

/*
 * The loss on RAW joint logits: ctct_loss(log_softmax(logits, -1), ...) with the log-softmax fused
 * into both passes.  Replaces, for a caller that holds logits, the caller's torch.log_softmax, the
 * gather and .float() of warp_ctct/__init__.py:124-136, ctct_loss_fwd (csrc/binding.cpp:31-100)
 * and, in the backward pass, CTCTLoss.backward (warp_ctct/__init__.py:31-33), the scatter of the
 * gather's autograd and log_softmax's backward.
 *   forward : one streaming read of the valid rows (t < lx[n], u <= ly[n]) yields each row's
 *             log-sum-exp and the three log-probs the lattice needs; then the lattice and the
 *             occupancy gradient as in ctct_b200_loss_forward_fused.  grads3 records carry the row's
 *             log-sum-exp (log2 units) in their fourth word.  Workspace: ctct_b200_workspace_bytes.
 *             logits must be device memory.  reduction 0 / 1 / 2 as above (`loss` unused for 0).
 *             grad_logits (optional, NULL = none; needs V * sizeof(element) % 16 == 0 and a 16-byte
 *             aligned base): the buffer the backward call will write.  Its padding rows (t >= lx[n]
 *             or u > ly[n]; 30-70 % of the tensor for ragged batches) are zero-filled by extra thread
 *             blocks of the latency-bound lattice launch, so that the backward call, given
 *             padding_cleared = 1, only touches the valid rows.
 *   backward: grad_logits[n,t,u,:] = G - softmax(logits[n,t,u,:]) * sum(G), G = the row's <= 3
 *             occupancy-gradient entries scaled by the upstream gradient (`grad`: N floats, or ONE
 *             float with scalar_grad != 0 and the reduction of the forward call); valid rows are
 *             read once and written once, padding rows are written as zeros.  `logits` are the
 *             forward call's, unchanged; grad_logits has their shape and element type.
 */
int ctct_b200_logits_forward(const void *logits, int dtype, const int32_t *ys, const int32_t *lx,
                             const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int want_grad,
                             int reduction, int average_frames, float norm, float *costs, float *loss,
                             float *grads3, void *grad_logits, void *workspace, size_t workspace_bytes,
                             void *stream);
int ctct_b200_logits_backward(const float *grads3, const float *grad, int scalar_grad, int reduction,
                              int average_frames, float norm, const void *logits, const int32_t *ys,
                              const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                              int dtype, void *grad_logits, int padding_cleared, void *stream);

/*
 * PACKED (ragged) layout: the joint tensor holds only the valid rows, (rows, V) with
 * rows = sum_n lx[n] * (ly[n] + 1); utterance n owns rows [cu_rows[n], cu_rows[n+1]), frame-major, ly[n] + 1
 * rows per frame.  The reference pads every utterance to (T, U+1) and only skips the padding inside
 * its kernels (csrc/gather.cu:321) while autograd still zero-fills it (warp_ctct/__init__.py:124-131);
 * here no padding byte is read or written: for ragged batches that is 30-70 % of all traffic.
 *   ctct_b200_packed_offsets   computes cu_rows (N + 1 int64 on the device) from lx, ly, clamped to T, U1-1
 *   *_forward_packed / *_backward_packed   as ctct_b200_loss_forward_fused + ctct_b200_loss_backward_patch,
 *       and as ctct_b200_logits_forward + ctct_b200_logits_backward, on packed tensors.  T and U1 are upper
 *       bounds of lx and ly + 1 (they size the workspace and grads3 exactly as in the padded calls).
 *       packed_rows = number of rows of the packed tensor(s); rows an inconsistent lx / ly would place
 *       beyond it are neither read nor written.  `clear` of the standard-loss forward is the packed
 *       gradient buffer (packed_rows * V elements), zero-filled by the lattice launch; the backward then
 *       patches it (pass a buffer cleared with ctct_b200_zero_fill when the forward did not clear it).
 *       The logits backward writes every row of packed_grad once; nothing needs clearing.
 */
int ctct_b200_packed_offsets(const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1,
                             int64_t *cu_rows, void *stream);
int ctct_b200_loss_forward_packed(const void *packed, int dtype, const int64_t *cu_rows, int64_t packed_rows,
                                  const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N, int64_t T,
                                  int64_t U1, int64_t V, int want_grad, int reduction, int average_frames,
                                  float norm, float *costs, float *loss, float *grads3, void *clear,
                                  size_t clear_bytes, void *workspace, size_t workspace_bytes, void *stream);
int ctct_b200_loss_backward_packed(const float *grads3, const float *grad, int scalar_grad, int reduction,
                                   int average_frames, float norm, const int64_t *cu_rows, int64_t packed_rows,
                                   const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N, int64_t T,
                                   int64_t U1, int64_t V, int dtype, void *packed_grad, void *stream);
int ctct_b200_logits_forward_packed(const void *packed_logits, int dtype, const int64_t *cu_rows,
                                    int64_t packed_rows, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                                    int64_t N, int64_t T, int64_t U1, int64_t V, int want_grad, int reduction,
                                    int average_frames, float norm, float *costs, float *loss, float *grads3,
                                    void *workspace, size_t workspace_bytes, void *stream);
int ctct_b200_logits_backward_packed(const float *grads3, const float *grad, int scalar_grad, int reduction,
                                     int average_frames, float norm, const void *packed_logits,
                                     const int64_t *cu_rows, int64_t packed_rows, const int32_t *ys,
                                     const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1,
                                     int64_t V, int dtype, void *packed_grad, void *stream);

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
 * Benchmark hook (no counterpart in the reference): the forward pass's gather alone on a float32
 * joint tensor, valid rows only, written as 16-byte records {blank, repeat, next, 0} in log2 units
 * (N*T*U1*4 floats), with `per` (1, 2, 4, 8 or 16) independent loads in flight per thread and
 * `blocks_per_sm` blocks of 256 threads per SM (0 = one thread per `per` elements).  Used to measure
 * how many isolated DRAM reads per second the GPU sustains.
 */
int ctct_b200_gather_probe(const float *log_probs, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                           int64_t N, int64_t T, int64_t U1, int64_t V, int per, int blocks_per_sm,
                           float *records, void *stream);

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

/* ------------------------------------------------------------------------- *
 * log-add joiner ("simple" loss)
 * ------------------------------------------------------------------------- */

/*
 * Batched log-semiring matrix product out[b,i,j] = log sum_k exp(lhs[b,i,k] + rhs[b,k,j]),
 * float32, element strides given explicitly (the reference passes rhs as the transposed
 * view g.transpose(1,2), warp_ctct/__init__.py:195-200); out is (B,M,N) contiguous.
 * Replaces log_matmul of csrc/binding.cpp:224-245 / log_matmul_cuda_impl of csrc/core.h:39-41
 * (kernel csrc/logmatmul.cu:44-181).  Exact for any dynamic range; all -inf gives -inf.
 */
int ctct_b200_log_matmul(const float *lhs, int64_t lhs_stride_b, int64_t lhs_stride_i, int64_t lhs_stride_k,
                         const float *rhs, int64_t rhs_stride_b, int64_t rhs_stride_k, int64_t rhs_stride_j,
                         int64_t B, int64_t M, int64_t K, int64_t N, float *out, void *stream);

/*
 * The same product for contiguous f (B,M,K) and g (B,N,K) -- den[b,i,j] = log sum_k exp(f[b,i,k] +
 * g[b,j,k]), the denominator of ctct_simple_loss -- as a tensor-core GEMM on max-shifted
 * exponentials (tcgen05 / TMEM / TMA, bf16 hi+lo operand split, fp32 accumulation) with the
 * log / max rescaling in the epilogue.  Needs K % 8 == 0, K >= 64 and a scratch workspace of
 * ctct_b200_log_matmul_tc_workspace_bytes (0 = shape not supported: use ctct_b200_log_matmul).
 * Outputs whose shifted sum underflows (dynamic range beyond ~80 nats with maxima at different
 * k) are detected on the device and recomputed by the exact kernel in the same call.
 * Replaces log_matmul of csrc/binding.cpp:224-245 on the loss path (warp_ctct/__init__.py:195-200).
 */
size_t ctct_b200_log_matmul_tc_workspace_bytes(int64_t B, int64_t M, int64_t N, int64_t K);
/* Test hook (no counterpart in the reference): byte offset, inside that workspace, of four int32
 * status words the tensor-core kernels raise: [0] a bounded wait ran out, [1] a max-shifted sum
 * underflowed.  Either one non-zero means the exact kernels produced the results of the calls
 * that used the workspace; all zero means the tensor-core results stand. */
size_t ctct_b200_log_matmul_tc_flags_offset(int64_t B, int64_t M, int64_t N, int64_t K);
/* Test hook (no counterpart in the reference): every wait of the tensor-core kernels (on a TMA load, an
 * MMA, an epilogue) polls at most `polls` times and then gives up: the thread block raises status word
 * [0], lets loads it has already issued land, frees its tensor memory and returns, and the exact kernel
 * launched behind produces the result.  0 makes every wait give up before anything was issued; a negative
 * value restores the default (2^23 polls).  Synchronous (a copy into constant memory of the current
 * device); not for use while kernels of this library run. */
int ctct_b200_debug_set_wait_limit(long long polls);
int ctct_b200_log_matmul_tc(const float *f, const float *g, int64_t B, int64_t M, int64_t N, int64_t K, float *den,
                            void *workspace, size_t workspace_bytes, void *stream);

/*
 * Backward of the product above for an arbitrary (signed) grad_out (B,M,N):
 *   grad_lhs[b,i,k]  = sum_j grad_out[b,i,j] * exp(lhs[b,i,k] + rhs[b,k,j] - res[b,i,j])
 *   grad_rhsT[b,j,k] = sum_i (same term)
 * Replaces log_matmul_backward of csrc/binding.cpp:247-324.  lhs (B,M,K), rhsT = rhs transposed
 * (B,N,K), res (B,M,N), all contiguous; either output may be NULL.
 */
int ctct_b200_log_matmul_backward(const float *grad_out, const float *lhs, const float *rhsT, const float *res,
                                  int64_t B, int64_t M, int64_t K, int64_t N, float *grad_lhs, float *grad_rhsT,
                                  void *stream);

/*
 * Fused forward of ctct_simple_loss after the denominator: gathers of f and g, composition of
 * f + g - den, lattice and occupancy gradient.  Replaces the two torch.gather calls of
 * warp_ctct/__init__.py:204-215 and ctct_loss_simple_fwd of csrc/binding.cpp:103-222 (launchers
 * run_warp_ctct_simple / run_fill_grad_simple, csrc/core.h:22-37; kernels csrc/simple.cu,
 * csrc/simple_unnorm.cu).
 *   f (N,T,V), g (N,U1,V) float32 contiguous; den (N,T,U1) or NULL for the un-normalised loss
 *   costs, grads3, workspace: as for ctct_b200_loss_forward (same workspace size).
 */
int ctct_b200_simple_forward(const float *f, const float *g, const float *den, const int32_t *ys,
                             const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                             int want_grad, float *costs, float *grads3, void *workspace,
                             size_t workspace_bytes, void *stream);

/*
 * The reference's extension entry point for the log-add joiner, ctct_loss_simple_fwd(f, g, ys, den,
 * lx, ly, requires_grad) of csrc/binding.cpp:103-222 (launchers run_warp_ctct_simple /
 * run_fill_grad_simple, csrc/core.h:22-37), on PRE-GATHERED operands:
 *   f (N,T,U1): f[n,t,0] blank, f[n,t,k] = score of label ys[n,k-1];  g (N,U1,3): the three picks of
 *   every context;  den (N,T,U1) or NULL for the un-normalised loss.  All float32, contiguous.
 *   costs (N) out; with want_grad also grad_f (N,T,U1), grad_g (N,U1,3) and, when den is given,
 *   grad_den (N,T,U1): the lattice's occupancy gradient reduced as csrc/binding.cpp:198,209-219 does
 *   (grad_den = -sum of the three slots, grad_g = sum over t, grad_f[...,0] = sum over u of the blank
 *   slot, grad_f[...,k] = repeat slot of context k + next slot of context k-1), in fixed order.
 * Workspace: ctct_b200_simple_gathered_workspace_bytes (256-byte aligned base).
 */
size_t ctct_b200_simple_gathered_workspace_bytes(int64_t N, int64_t T, int64_t U1, int want_grad);
int ctct_b200_simple_gathered_forward(const float *f, const float *g, const float *den, const int32_t *ys,
                                      const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1,
                                      int want_grad, float *costs, float *grad_f, float *grad_g,
                                      float *grad_den, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Dense gradients of ctct_simple_loss w.r.t. f (N,T,V) and g (N,U1,V), each written once:
 * the lattice's sparse part (reductions of csrc/binding.cpp:198,209-219 and the backward of the
 * two gathers) plus, when den is given, the part that flows through the denominator
 * (log_matmul_backward, csrc/binding.cpp:247-324), all scaled by grad_out[n]
 * (SimpleCTCTLoss.backward, warp_ctct/__init__.py:76-85).  Either output may be NULL.
 */
int ctct_b200_simple_backward(const float *grads3, const float *grad_out, const float *f, const float *g,
                              const float *den, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                              int64_t N, int64_t T, int64_t U1, int64_t V, float *grad_f, float *grad_g,
                              void *stream);

/*
 * The same gradients with the part through the denominator (log_matmul_backward,
 * csrc/binding.cpp:247-324) computed as two tensor-core GEMMs,
 *     grad_f = Ef * (P  Eg),   grad_g = Eg * (P^T Ef),   P = w * exp(mf + mg - den),
 * on the bf16 planes of Ef = exp(f - max f), Eg = exp(g - max g) that ctct_b200_log_matmul_tc left
 * in its workspace.  tc_workspace must be the buffer passed to ctct_b200_log_matmul_tc for the same
 * f, g (B = N, M = T, N = U1, K = V), not written since; den must be its result.  If that call had
 * to fall back to the exact kernel (a flag in the workspace says so) this one does too, inside the
 * same launches.  den must not be NULL; f, g, grad_f, grad_g 16-byte aligned.
 */
int ctct_b200_simple_backward_tc(const float *grads3, const float *grad_out, const float *f, const float *g,
                                 const float *den, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                                 int64_t N, int64_t T, int64_t U1, int64_t V, float *grad_f, float *grad_g,
                                 void *tc_workspace, size_t tc_workspace_bytes, void *stream);

/*
 * log_matmul_backward (csrc/binding.cpp:247-324) as two tensor-core GEMMs, for a result that
 * ctct_b200_log_matmul_tc computed: lhs (B,M,K), rhsT (B,N,K), res (B,M,N) are that call's f, g and
 * den, tc_workspace its untouched workspace; grad_out (B,M,N) contiguous float32, any sign.
 * grad_lhs (B,M,K) and grad_rhsT (B,N,K) are written once each; either may be NULL.  Falls back to
 * the exact kernel inside the same call when the forward call had to (flag in the workspace).
 */
int ctct_b200_log_matmul_backward_tc(const float *grad_out, const float *lhs, const float *rhsT, const float *res,
                                     int64_t B, int64_t M, int64_t K, int64_t N, float *grad_lhs, float *grad_rhsT,
                                     void *tc_workspace, size_t tc_workspace_bytes, void *stream);

/*
 * Optional per-kernel timing for benchmarks (no counterpart in the reference).  While
 * enabled, every ctct_b200_loss_forward records CUDA events on its stream before the gather,
 * after the gather, after the lattice and after the occupancy-gradient kernel, and every
 * ctct_b200_loss_backward records one before and one after the dense-gradient kernel.
 * Events are created once by _enable (room for max_calls calls, shared by all host threads) and
 * destroyed by _disable; nothing is recorded when profiling is off.
 *   ctct_b200_profile_read: waits for the recorded events, writes for call i
 *     kind[i] (0 forward, 1 backward, 2 zero fill, 3 log_matmul_tc, 4 simple_forward,
 *     5 simple_backward, 6 logits_forward: {log-sum-exp + gather, lattice, fill_grad},
 *     7 logits_backward: {gradient kernel, 0, 0}) and ms[4*i .. 4*i+2] = {gather, lattice, fill_grad} (kind 0),
 *     {dense gradient / patch / zero fill, 0, 0} (kinds 1, 2), {exp + bf16 split of both operands,
 *     tensor-core kernel, exact fix-up} (kind 3), {compose, lattice, fill_grad} (kind 4),
 *     {denominator weights + grad_f GEMM (or the exact kernel), grad_g GEMM + exact fix-up, label
 *     patches} (kind 5); returns the number of calls recorded (<= capacity) or a
 *     negative error code, and rewinds the recorder.
 */
int ctct_b200_profile_enable(int max_calls);
int ctct_b200_profile_read(float *ms, int *kind, int capacity);
int ctct_b200_profile_disable(void);

#ifdef __cplusplus
}
#endif
#endif /* CTCT_B200_H */

/*
 * mhc_b200.h -- C ABI of the B200 (sm_100a) hyper-connection kernels.
 *
 * Every entry point takes raw device pointers, 64-bit sizes and the CUDA stream
 * to launch on; nothing here depends on PyTorch.  The library never allocates
 * or frees device memory: outputs and scratch are caller-owned (scratch sizes
 * come from mhc_scratch_bytes).  The one piece of device memory the library
 * holds itself is the fixed 1 MiB array of mhc_add_residual_bwd_noalloc, which
 * is part of the library image.  Inputs are never written.  All launches go to
 * the stream passed in; no call synchronises the device or the host.
 *
 * Ticket counters.  Entry points with a `tickets` argument can finish their
 * deterministic sums inside the producing kernel instead of in a second launch:
 * the CTA that stores the last partial sum of a batch element (detected with an
 * integer counter) adds all partial sums up in the usual fixed order.  `tickets`
 * points to at least max(B, 1) int32 counters in device memory that are ZERO on
 * entry; every kernel leaves them zero again, so one buffer zeroed once serves
 * all later calls.  Calls that may overlap on the GPU (different streams) need
 * different counters.  NULL selects the separate finish kernels; the results are
 * bit-identical either way.
 *
 * Each declaration names the function of the reference project
 * (WithNucleusAI/mHC-triton, paths relative to its root) that it replaces.
 *
 * Return value: 0 on success, otherwise one of the MHC_ERR_* codes; the text
 * of the last failure on the calling thread is available from
 * mhc_last_error_string().  No entry point aborts the process.
 *
 * Tensor layouts (all contiguous, row-major):
 *   H, H_residual, H_new, dH*      [B, S, 4, D]   activation dtype (mhc_dtype)
 *   branch_input / branch_output   [B, S, D]      activation dtype
 *   H_pre, H_post                  [B, 4]         float32
 *   H_res                          [B, 4, 4]      float32
 *   x (pooled state)               [B, 4*D]       float32
 *   phi                            [4*D, 24]      float32
 *   bias                           [24]           float32   (pre 0..3, post 4..7, res 8..23)
 */
#ifndef MHC_B200_H
#define MHC_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MHC_B200_VERSION 200 /* major*10000 + minor*100 + patch */

typedef enum mhc_dtype { MHC_F32 = 0, MHC_BF16 = 1, MHC_F16 = 2 } mhc_dtype;

typedef enum mhc_status {
  MHC_OK = 0,
  MHC_ERR_NULL_POINTER = 1,
  MHC_ERR_BAD_SHAPE = 2,
  MHC_ERR_BAD_DTYPE = 3,
  MHC_ERR_BAD_ARGUMENT = 4,
  MHC_ERR_SCRATCH_TOO_SMALL = 5,
  MHC_ERR_MISALIGNED = 6,
  MHC_ERR_CUDA = 7
} mhc_status;

/* d|m|/dm at m == 0 in the Sinkhorn backward.  0: zero (what autograd of the
 * reference's PyTorch path gives, src/mhc/_torch_baseline.py:27).  1: +1 (what the
 * reference's device kernel uses, src/mhc/_backward.py:106-121). */
typedef enum mhc_abs_grad_at_zero { MHC_ABS0_ZERO = 0, MHC_ABS0_PLUS_ONE = 1 } mhc_abs_grad_at_zero;

/* Which entry point a scratch-size query is for. */
typedef enum mhc_op {
  MHC_OP_ADD_RESIDUAL_BWD = 0,
  MHC_OP_STREAM_MIX_BWD = 1,
  MHC_OP_MEANPOOL_FWD = 2,
  MHC_OP_DYNAMIC_WEIGHTS_FWD = 3,
  MHC_OP_DYNAMIC_WEIGHTS_BWD = 4,
  MHC_OP_HC_MIX_FWD = 5,
  MHC_OP_HC_MIX_BWD = 6
} mhc_op;

typedef void* mhc_stream_t; /* a cudaStream_t */
typedef void* mhc_event_t;  /* a cudaEvent_t */

int mhc_version(void);
const char* mhc_last_error_string(void);
const char* mhc_status_name(int status);
/* Kernels launched by this library since it was loaded (all threads). */
int64_t mhc_launch_count(void);

/* Per-kernel timing.  While enabled, every kernel launch of this library is bracketed by two CUDA
 * events on the stream it is launched on.  enable(1) drops earlier records and starts; enable(0)
 * stops (pauses); enable(2) resumes and keeps the records, so that a caller can time a sample of its
 * steps.  After the device is synchronised, record i gives the kernel's name and its duration. */
int mhc_profile_enable(int on);
/* Restrict timing to the kernel with this name (NULL or "" = every kernel); the events of a timed
 * kernel sit between it and its neighbours on the stream, so timing one kernel perturbs least. */
int mhc_profile_select(const char* kernel_name);
int64_t mhc_profile_count(void);
int mhc_profile_get(int64_t index, const char** name, float* milliseconds);

/* Bytes of device scratch the given entry point needs for these sizes
 * (for the two dynamic-weights ops S is ignored and D is the per-stream width,
 * i.e. the projection reads K = 4*D values per row).  Returns < 0 on bad arguments. */
int64_t mhc_scratch_bytes(int op, int64_t B, int64_t S, int64_t D, int dtype);

/* ---- Sinkhorn-Knopp on a batch of 4x4 matrices --------------------------------
 * P = Sinkhorn_iters(|M| + eps).  M, P: [batch, 4, 4] of `dtype`.
 * Replaces sinkhorn_forward, src/mhc/_kernels.py:597-614 (kernel :30-130). */
int mhc_sinkhorn_fwd(const void* M, void* P, int64_t batch, int dtype, int iters, float eps,
                     mhc_stream_t stream);

/* dM from dP with no saved state: the state entering each iteration is recomputed from M.  The
 * default kernel keeps four checkpoints of the forward sweep in registers and recomputes from the
 * nearest one, which gives bit-identical results to recomputing from M every time (the plain
 * O(iters^2) sweep of the reference, selectable with MHC_SINKHORN_PLAIN=1 in the environment) for
 * roughly a third of the work at iters = 20.
 * Replaces sinkhorn_backward, src/mhc/_backward.py:503-530 (kernel :29-262). */
int mhc_sinkhorn_bwd(const void* M, const void* dP, void* dM, int64_t batch, int dtype, int iters,
                     float eps, int abs_grad_at_zero, mhc_stream_t stream);

/* ---- Stream mix -----------------------------------------------------------------
 * branch_input[b,s,d] = sum_n H_pre[b,n] H[b,s,n,d];
 * H_residual[b,s,n,d] = sum_m H_res[b,n,m] H[b,s,m,d].
 * H_residual may be NULL (H_res is then unused): only branch_input is written, for callers that
 * add the residual with mhc_add_residual_mix_fwd.
 * Replaces stream_mix_forward, src/mhc/_kernels.py:617-652 (kernel :137-236). */
int mhc_stream_mix_fwd(const void* H, const float* H_pre, const float* H_res, void* branch_input,
                       void* H_residual, int64_t B, int64_t S, int64_t D, int dtype,
                       mhc_stream_t stream);

/* dH, dH_pre [B,4] (fp32), dH_res [B,4,4] (fp32) in one pass over the data.
 * Replaces stream_mix_backward, src/mhc/_backward.py:578-626 (kernel :358-496) including
 * the torch.sum over its partial buffers (:623-624). */
int mhc_stream_mix_bwd(const void* d_branch_input, const void* dH_residual, const void* H,
                       const float* H_pre, const float* H_res, void* dH, float* dH_pre,
                       float* dH_res, void* scratch, int64_t scratch_bytes, int64_t B, int64_t S,
                       int64_t D, int dtype, mhc_stream_t stream);

/* Two-pass form used when the pooled-state gradient has to be folded into dH
 * (the reference leaves that addition to autograd of H.mean(dim=1), src/mhc/module.py:123).
 *   reduce: only dH_pre / dH_res (reads d_branch_input, dH_residual, H).
 *   apply : dH[b,s,m,d] = H_pre[b,m] d_bi[b,s,d] + sum_n H_res[b,n,m] dH_residual[b,s,n,d]
 *                         + inv_S * grad_x[b, m*D + d]      (grad_x fp32, may be NULL). */
int mhc_stream_mix_bwd_reduce(const void* d_branch_input, const void* dH_residual, const void* H,
                              float* dH_pre, float* dH_res, void* scratch, int64_t scratch_bytes,
                              int64_t B, int64_t S, int64_t D, int dtype, mhc_stream_t stream);
int mhc_stream_mix_bwd_apply(const void* d_branch_input, const void* dH_residual,
                             const float* H_pre, const float* H_res, const float* grad_x,
                             float inv_S, void* dH, int64_t B, int64_t S, int64_t D, int dtype,
                             mhc_stream_t stream);

/* ---- Add residual ---------------------------------------------------------------
 * H_new[b,s,n,d] = H_residual[b,s,n,d] + H_post[b,n] branch_output[b,s,d].
 * Replaces add_residual_forward, src/mhc/_kernels.py:655-687 (kernel :244-310). */
int mhc_add_residual_fwd(const void* H_residual, const void* branch_output, const float* H_post,
                         void* H_new, int64_t B, int64_t S, int64_t D, int dtype,
                         mhc_stream_t stream);

/* Add residual with the residual mix recomputed from H instead of read from a materialised
 * H_residual: H_new[b,s,n,d] = (sum_m H_res[b,n,m] H[b,s,m,d]) + H_post[b,n] branch_output[b,s,d].
 * Together with mhc_hc_mix_fwd called with H_residual == NULL (which then writes branch_input
 * only) this removes the write and the read-back of H_residual from a layer step.  pool_partials
 * may be NULL; if given it receives the token sums of H_new as in mhc_add_residual_pool_fwd.
 * Fuses add_residual_forward (src/mhc/_kernels.py:655-687) with the residual half of
 * stream_mix_forward (src/mhc/_kernels.py:617-652, kernel lines :227-230). */
int mhc_add_residual_mix_fwd(const void* H, const float* H_res, const void* branch_output,
                             const float* H_post, void* H_new, float* pool_partials, int64_t B,
                             int64_t S, int64_t D, int dtype, mhc_stream_t stream);

/* Add residual that also leaves, for the next layer, the token sums of the H_new it writes:
 * pool_partials [B, mhc_add_residual_pool_chunks(S, D), 4*D] fp32, to be handed to that layer's
 * mhc_hc_mix_fwd as pooled_partials.  The next layer then reads H once instead of twice
 * (the reference reads it twice: H.mean(dim=1), src/mhc/module.py:123, then the stream-mix
 * kernel, src/mhc/_kernels.py:137-236).  H_new is identical to mhc_add_residual_fwd's. */
int mhc_add_residual_pool_fwd(const void* H_residual, const void* branch_output, const float* H_post,
                              void* H_new, float* pool_partials, int64_t B, int64_t S, int64_t D,
                              int dtype, mhc_stream_t stream);
int64_t mhc_add_residual_pool_chunks(int64_t S, int64_t D);

/* d_branch_output and dH_post [B,4] (fp32).  dH_residual equals dH_new and is not written:
 * the caller aliases it.  `tickets`: see "Ticket counters" above (may be NULL).
 * Replaces add_residual_backward, src/mhc/_backward.py:533-575
 * (kernel :269-351) including its torch.sum (:573). */
int mhc_add_residual_bwd(const void* dH_new, const void* branch_output, const float* H_post,
                         void* d_branch_output, float* dH_post, void* scratch,
                         int64_t scratch_bytes, int32_t* tickets, int64_t B, int64_t S, int64_t D,
                         int dtype, mhc_stream_t stream);

/* Same result as mhc_add_residual_bwd for callers that cannot supply scratch memory because they
 * have no way to allocate on the device (a C/C++ host without a caching allocator whose serving
 * loop must not call cudaMalloc, or a plugin that only receives input and output buffers).  The
 * partial sums go to a fixed 1 MiB array inside the library image, which every GPU that loads the
 * library holds until the process exits; shapes whose partial sums need more than
 * mhc_add_residual_bwd_noalloc_max_bytes() (16 bytes per 3 to 5 tokens per group of 256 16-byte packs
 * along D, per batch element: 256 KiB for bf16 B=8, S=4096, D=4096) are rejected with
 * MHC_ERR_SCRATCH_TOO_SMALL.  The call allocates and frees nothing.  The first
 * call on each device looks up the array's device address (with that device current) and should
 * therefore come before any stream capture.  All calls on a device share the one array: two calls
 * that may overlap on the GPU (different streams) race and must be ordered by the caller.
 * `stream` must belong to the device that is current when the call is made (the array's address
 * is looked up for the current device).
 * This entry point has no counterpart in the reference. */
int mhc_add_residual_bwd_noalloc(const void* dH_new, const void* branch_output, const float* H_post,
                                 void* d_branch_output, float* dH_post, int64_t B, int64_t S,
                                 int64_t D, int dtype, mhc_stream_t stream);
int64_t mhc_add_residual_bwd_noalloc_max_bytes(void);

/* ---- Sequence mean-pool ---------------------------------------------------------
 * x[b, n*D + d] = (1/S) sum_s H[b,s,n,d], fp32 output.
 * Replaces H.mean(dim=1).reshape(B, 4*D), src/mhc/module.py:123. */
int mhc_meanpool_fwd(const void* H, float* x, void* scratch, int64_t scratch_bytes, int64_t B,
                     int64_t S, int64_t D, int dtype, mhc_stream_t stream);

/* ---- Dynamic weights ------------------------------------------------------------
 * raw = x phi; inv_rms = 1/sqrt(sum(x^2)/K + eps); s = inv_rms * alpha_g * raw + bias;
 * H_pre = sigmoid(s[0:4]) / (sum + eps); H_post = 2 sigmoid(s[4:8]);
 * H_res = Sinkhorn_iters(|s[8:24]| + eps).  alpha_* are device pointers to one float each
 * (no host read of the scales).  saved [batch, 32] fp32 receives raw (24 values), sum(x^2),
 * inv_rms and padding for the backward; it may be NULL.
 * Any batch is accepted.  Below 64 rows every row gets its own CTAs (the sequence-pooled use, batch =
 * number of sequences).  From 64 rows on (per-token use, batch = number of tokens), when K % 4 == 0
 * and x is 16-byte aligned, both directions run on the fifth-generation tensor cores: tcgen05.mma
 * kind::tf32 on hi/lo splits of both operands (3xTF32) with fp32 running sums, x tiles by TMA, and in
 * the forward the whole finish of a row as the kernel's epilogue; same results as the fp32 FMA path
 * to within the fp32 parity band, not bit-identical to it.  Other shapes use mma.sync / FMA kernels
 * (also with MHC_ROWS_TC=0 in the environment).  On the tensor-core path scratch must be 16-byte
 * aligned, and its first int is a status word: 0, or the code of an mbarrier wait that ran out
 * (every wait in those kernels is bounded; the affected outputs are then NaN).
 * Replaces fused_dynamic_weights_forward, src/mhc/_kernels.py:690-752 (kernel :318-590). */
int mhc_dynamic_weights_fwd(const float* x, const float* phi, const float* bias,
                            const float* alpha_pre, const float* alpha_post,
                            const float* alpha_res, float* H_pre, float* H_post, float* H_res,
                            float* saved, void* scratch, int64_t scratch_bytes, int64_t batch,
                            int64_t K, int iters, float eps, mhc_stream_t stream);

/* Gradients of the above: grad_x [batch,K], grad_phi [K,24], grad_bias [24], grad_alpha [3]
 * (pre, post, res), all fp32, written (not accumulated) unless `accumulate_params` is non-zero,
 * in which case grad_phi / grad_bias / grad_alpha are added to.  `saved` is the buffer the
 * forward filled.  On the tensor-core path (see above) grad_x and scratch must be 16-byte aligned.
 * Replaces _FusedDynamicWeights.backward, src/mhc/ops.py:109-228, including its
 * call of sinkhorn_backward (:161-166). */
int mhc_dynamic_weights_bwd(const float* x, const float* phi, const float* bias,
                            const float* alpha_pre, const float* alpha_post,
                            const float* alpha_res, const float* saved, const float* dH_pre,
                            const float* dH_post, const float* dH_res, float* grad_x,
                            float* grad_phi, float* grad_bias, float* grad_alpha, void* scratch,
                            int64_t scratch_bytes, int64_t batch, int64_t K, int iters, float eps,
                            int abs_grad_at_zero, int accumulate_params, mhc_stream_t stream);

/* ---- Fused layer entry points ------------------------------------------------------
 * Forward of the module's fused dynamic path in one call: x = mean_s H (fp32 [B,4D], output),
 * the dynamic weights from x (bias given as the three base parameters, pre [4], post [4],
 * res [16]), then the stream mix.  If pooled_partials is not NULL it holds the token sums of H
 * as left by mhc_add_residual_pool_fwd of the previous layer ([B, pooled_chunks, 4*D] fp32) and
 * the pass over H for pooling is skipped.  H_residual may be NULL: only branch_input is then
 * written and the caller uses mhc_add_residual_mix_fwd afterwards.  `tickets`: see "Ticket
 * counters" above (may be NULL); with them the call is three launches (pooling, projection that
 * also finishes the weights, stream mix).  Replaces the chain
 * HyperConnection._compute_weights (fused branch, src/mhc/module.py:119-139) + fused_stream_mix
 * (src/mhc/module.py:177). */
int mhc_hc_mix_fwd(const void* H, const float* phi, const float* H_pre_base, const float* H_post_base,
                   const float* H_res_base, const float* alpha_pre, const float* alpha_post,
                   const float* alpha_res, float* x, float* H_pre, float* H_post, float* H_res,
                   float* saved, void* branch_input, void* H_residual,
                   const float* pooled_partials, int64_t pooled_chunks, void* scratch,
                   int64_t scratch_bytes, int32_t* tickets, int64_t B, int64_t S, int64_t D,
                   int dtype, int iters, float eps, mhc_stream_t stream);

/* Backward of the same chain in one call.  In: gradients of branch_input, H_residual and H_post
 * plus what the forward left (H, x, saved, H_pre, H_res).  Out: dH (including grad_x / S, i.e.
 * the gradient through the mean-pool), grad_phi [4D,24], grad_bias [24] (pre, post, res bases),
 * grad_alpha [3]; grad_x [B,4D], dH_pre [B,4] and dH_res [B,16] are also written (fp32).
 * `tickets`: see "Ticket counters" above (may be NULL); with them the call is three launches
 * (reduction pass, weights backward, apply pass).  `weight_grads_ready` (may be NULL) is a CUDA
 * event that the call records on `stream` after the kernels that write grad_phi / grad_bias /
 * grad_alpha and before the apply pass that writes dH, so that a collective on another stream can
 * reduce the parameter gradients while dH is still being written.
 * Replaces _FusedStreamMix.backward + _FusedDynamicWeights.backward (src/mhc/ops.py:42-49,
 * 109-228) and autograd's backward of H.mean(dim=1) and torch.cat (src/mhc/module.py:123-131). */
int mhc_hc_mix_bwd(const void* d_branch_input, const void* dH_residual, const float* dH_post,
                   const void* H, const float* x, const float* phi, const float* H_pre_base,
                   const float* H_post_base, const float* H_res_base, const float* alpha_pre,
                   const float* alpha_post, const float* alpha_res, const float* saved,
                   const float* H_pre, const float* H_res, void* dH, float* grad_phi, float* grad_bias,
                   float* grad_alpha, float* grad_x, float* dH_pre, float* dH_res, void* scratch,
                   int64_t scratch_bytes, int32_t* tickets, mhc_event_t weight_grads_ready, int64_t B,
                   int64_t S, int64_t D, int dtype, int iters, float eps, int abs_grad_at_zero,
                   int accumulate_params, mhc_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MHC_B200_H */

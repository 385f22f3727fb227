// Fused entry points of the module's hot path: one C call launches the whole chain
//   forward : mean-pool partials -> projection (finishing the pooling) -> weights finish -> stream mix
//   backward: stream-mix reduction pass -> per-row weights backward (summing the reduction's partials)
//             -> grad_x / grad_phi / grad_bias / grad_alpha -> apply pass writing dH once
// so the host pays for one call and the tiny finish kernels of the single-op entry points vanish.
// With the caller's ticket counters the chains shrink to four and three launches: the projection
// finishes its own rows, the reduction pass adds up its own partial sums, and one kernel does the
// whole weights backward.
#include "common.cuh"
#include "launch.h"

using namespace mhc;

extern "C" int mhc_hc_mix_fwd(const void* H, const float* phi, const float* H_pre_base, const float* H_post_base,
                              const float* H_res_base, const float* alpha_pre, const float* alpha_post,
                              const float* alpha_res, float* x, float* H_pre, float* H_post, float* H_res,
                              float* saved, void* branch_input, void* H_residual, const float* pooled_partials,
                              int64_t pooled_chunks, void* scratch, int64_t scratch_bytes, int32_t* tickets,
                              int64_t B, int64_t S, int64_t D, int dtype, int iters, float eps,
                              mhc_stream_t stream) {
  if (int e = check_bsd_pub("hc_mix_fwd", B, S, D, dtype)) return e;
  if (iters < 0) return fail(MHC_ERR_BAD_ARGUMENT, "hc_mix_fwd: iters < 0");
  if (B == 0) return MHC_OK;
  if (S == 0 || D == 0) return fail(MHC_ERR_BAD_SHAPE, "hc_mix_fwd: empty sequence or width");
  if (!H || !phi || !H_pre_base || !H_post_base || !H_res_base || !alpha_pre || !alpha_post || !alpha_res || !x ||
      !H_pre || !H_post || !H_res || !saved || !branch_input || !scratch)
    return fail(MHC_ERR_NULL_POINTER, "hc_mix_fwd: null pointer");
  if (!is_aligned_to(tickets, 4) || !is_aligned_to(scratch, 4))
    return fail(MHC_ERR_MISALIGNED, "hc_mix_fwd: tickets / scratch must be 4-byte aligned");
  const int64_t pool_floats = meanpool_scratch_floats(B, S, D);
  const int64_t need = pool_floats * (int64_t)sizeof(float) + weights_fwd_scratch_bytes(B, 4 * D);
  if (scratch_bytes < need)
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "hc_mix_fwd: scratch %lld < %lld bytes", (long long)scratch_bytes, (long long)need);
  cudaStream_t st = (cudaStream_t)stream;
  float* pool_part = (float*)scratch;
  float* proj_part = pool_part + pool_floats;
  int nchunk = 0;
  const float* pool_src = pool_part;
  if (pooled_partials) {  // token sums of H left by the previous layer's add residual: no pass over H here
    if (pooled_chunks <= 0 || pooled_chunks > (1 << 20)) return fail(MHC_ERR_BAD_ARGUMENT, "hc_mix_fwd: bad pooled_chunks");
    pool_src = pooled_partials;
    nchunk = (int)pooled_chunks;
  } else if (int e = meanpool_partial_impl(H, pool_part, B, S, D, dtype, st, &nchunk)) {
    return e;
  }
  if (int e = weights_fwd_impl(pool_src, nchunk, 1.0 / (double)S, x, phi, BiasPtrs{H_pre_base, H_post_base, H_res_base},
                               alpha_pre, alpha_post, alpha_res, H_pre, H_post, H_res, saved, proj_part, B, 4 * D,
                               iters, eps, (int*)tickets, st))
    return e;
  return stream_mix_fwd_impl(H, H_pre, H_res, branch_input, H_residual, B, S, D, dtype, st);
}

extern "C" int mhc_hc_mix_bwd(const void* d_branch_input, const void* dH_residual, const float* dH_post,
                              const void* H, const float* x, const float* phi, const float* H_pre_base,
                              const float* H_post_base, const float* H_res_base, const float* alpha_pre,
                              const float* alpha_post, const float* alpha_res, const float* saved,
                              const float* H_pre, const float* H_res, void* dH, float* grad_phi, float* grad_bias,
                              float* grad_alpha, float* grad_x, float* dH_pre, float* dH_res, void* scratch,
                              int64_t scratch_bytes, int32_t* tickets, mhc_event_t weight_grads_ready, int64_t B,
                              int64_t S, int64_t D, int dtype, int iters, float eps, int abs_grad_at_zero,
                              int accumulate_params, mhc_stream_t stream) {
  if (int e = check_bsd_pub("hc_mix_bwd", B, S, D, dtype)) return e;
  if (iters < 0) return fail(MHC_ERR_BAD_ARGUMENT, "hc_mix_bwd: iters < 0");
  if (abs_grad_at_zero != MHC_ABS0_ZERO && abs_grad_at_zero != MHC_ABS0_PLUS_ONE)
    return fail(MHC_ERR_BAD_ARGUMENT, "hc_mix_bwd: abs_grad_at_zero must be 0 or 1");
  if (B == 0) return MHC_OK;
  if (S == 0 || D == 0) return fail(MHC_ERR_BAD_SHAPE, "hc_mix_bwd: empty sequence or width");
  if (!d_branch_input || !dH_residual || !dH_post || !H || !x || !phi || !H_pre_base || !H_post_base || !H_res_base ||
      !alpha_pre || !alpha_post || !alpha_res || !saved || !H_pre || !H_res || !dH || !grad_phi || !grad_bias ||
      !grad_alpha || !grad_x || !dH_pre || !dH_res || !scratch)
    return fail(MHC_ERR_NULL_POINTER, "hc_mix_bwd: null pointer");
  if (!is_aligned_to(tickets, 4) || !is_aligned_to(scratch, 4))
    return fail(MHC_ERR_MISALIGNED, "hc_mix_bwd: tickets / scratch must be 4-byte aligned");
  const int64_t part_floats = mix_bwd_scratch_floats(B, S, D);
  const int64_t need = part_floats * (int64_t)sizeof(float) + weights_bwd_scratch_bytes(B, 4 * D);
  if (scratch_bytes < need)
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "hc_mix_bwd: scratch %lld < %lld bytes", (long long)scratch_bytes, (long long)need);
  cudaStream_t st = (cudaStream_t)stream;
  float* part20 = (float*)scratch;
  float* rows = part20 + part_floats;
  int64_t slots = 0;
  if (!ticket_finish_supported()) tickets = nullptr;
  // With ticket counters the reduction pass leaves finished sums in dH_pre / dH_res; without them the
  // weights backward starts by adding up the per-CTA partial sums.
  if (int e = mix_bwd_partials_impl(1, d_branch_input, dH_residual, H, nullptr, nullptr, nullptr, part20, B, S, D, dtype,
                                    st, &slots, (int*)tickets, dH_pre, dH_res))
    return e;
  if (int e = weights_bwd_impl(x, phi, BiasPtrs{H_pre_base, H_post_base, H_res_base}, alpha_pre, alpha_post, alpha_res,
                               saved, tickets ? nullptr : part20, slots, dH_pre, dH_post, dH_res, grad_x, grad_phi,
                               grad_bias, grad_alpha, rows, B, 4 * D, iters, eps, abs_grad_at_zero, accumulate_params,
                               st))
    return e;
  if (weight_grads_ready) {  // grad_phi / grad_bias / grad_alpha are complete from here on in stream order
    const cudaError_t ce = cudaEventRecord((cudaEvent_t)weight_grads_ready, st);
    if (ce != cudaSuccess) {
      (void)cudaGetLastError();
      return fail(MHC_ERR_CUDA, "hc_mix_bwd: cudaEventRecord: %s", cudaGetErrorString(ce));
    }
  }
  return mix_bwd_apply_impl(d_branch_input, dH_residual, H_pre, H_res, grad_x, 1.f / (float)S, dH, B, S, D, dtype, st);
}

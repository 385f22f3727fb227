// Host-side helpers shared by the C-ABI translation units: status reporting, launch checks,
// and the geometry (tokens per chunk, columns per CTA) of the streaming kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <initializer_list>

#include "../../include/mhc_b200.h"
#include "common.cuh"

namespace mhc {

constexpr int64_t kMaxGridItems = 0x7fffffffLL;  // gridDim.x limit

int fail(int status, const char* fmt, ...);  // records the message for mhc_last_error_string
int check_launch(const char* what);          // cudaGetLastError -> status

inline bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool is_aligned_to(const void* p, unsigned n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1u)) == 0; }

// Geometry of a streaming kernel over [B, S, 4, D].
//   vec   : elements per pack (1 = scalar path for odd D or unaligned pointers)
//   kind  : Stream = no partial sums (short chunks), Reduce = leaves per-CTA partial sums,
//           Pool = the mean-pool kernel (long chunks, sub-groups inside the CTA)
enum class GeoKind { Stream, Reduce, Pool };
#ifndef MHC_FIT_COLS
#define MHC_FIT_COLS 1
#endif
Geo make_geo(int64_t S, int64_t D, int vec, GeoKind kind, int tpc, int occ = 0, bool fit_cols = MHC_FIT_COLS != 0,
             int narrow_mult = 1);
int sm_count();
inline int geo_block(const Geo& g) { return g.cols * g.sub; }
inline int64_t geo_slots(const Geo& g) { return (int64_t)g.nchunk * g.CG; }  // partial rows per batch element

// Pack width usable for a row length D of `dtype` given the pointers involved.
int pick_vec(int dtype, int64_t D, std::initializer_list<const void*> ptrs);

// Programmatic dependent launch (on unless MHC_PDL=0 is set in the environment): every kernel of
// this library may be scheduled while the previous kernel on the stream is still draining; each
// kernel starts with griddepcontrol.wait, so it touches memory only after its predecessor has
// completed and flushed.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline void launch_k(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t st,
                     Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  (void)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);  // errors surface in check_launch()
}

// The 24 bias entries as three device arrays (pre-mix base [4], post base [4], residual base [16]).
struct BiasPtrs { const float *pre, *post, *res; };

// Brackets one kernel launch with CUDA events on its stream while profiling is enabled
// (mhc_profile_enable); free when it is not.
struct ProfScope {
  ProfScope(const char* name, cudaStream_t st);
  ~ProfScope();
  int slot;
  cudaStream_t st;
};

// Internal launch sequences shared by the single-op and the fused entry points.
int stream_mix_fwd_impl(const void* H, const float* H_pre, const float* H_res, void* bi, void* Hr, int64_t B, int64_t S,
                        int64_t D, int dtype, cudaStream_t st);
int meanpool_partial_impl(const void* H, float* part, int64_t B, int64_t S, int64_t D, int dtype, cudaStream_t st,
                          int* nchunk);
int mix_bwd_partials_impl(int mode, const void* dbi, const void* dHr, const void* H, const float* H_pre,
                          const float* H_res, void* dH, float* part, int64_t B, int64_t S, int64_t D, int dtype,
                          cudaStream_t st, int64_t* slots, int* tickets, float* dH_pre, float* dH_res);
bool ticket_finish_supported();
int64_t add_residual_bwd_need_bytes(const void* dH_new, const void* bo, const void* dbo, int64_t B, int64_t S,
                                    int64_t D, int dtype);
int check_bsd_pub(const char* what, int64_t B, int64_t S, int64_t D, int dtype);
int mix_bwd_apply_impl(const void* dbi, const void* dHr, const float* H_pre, const float* H_res, const float* gx,
                       float inv_S, void* dH, int64_t B, int64_t S, int64_t D, int dtype, cudaStream_t st);
int64_t meanpool_scratch_floats(int64_t B, int64_t S, int64_t D);
int64_t mix_bwd_scratch_floats(int64_t B, int64_t S, int64_t D);
int weights_fwd_impl(const float* xsrc, int nsrc, double scale, float* x_out, const float* phi, BiasPtrs bias,
                     const float* alpha_pre, const float* alpha_post, const float* alpha_res, float* H_pre,
                     float* H_post, float* H_res, float* saved, float* part, int64_t batch, int64_t K, int iters,
                     float eps, int* tickets, cudaStream_t st);
int weights_bwd_impl(const float* x, const float* phi, BiasPtrs bias, const float* alpha_pre, const float* alpha_post,
                     const float* alpha_res, const float* saved, const float* part20, int64_t slots, float* dH_pre,
                     const float* dH_post, float* dH_res, float* grad_x, float* grad_phi, float* grad_bias,
                     float* grad_alpha, float* buf, int64_t batch, int64_t K, int iters, float eps,
                     int abs_grad_at_zero, int accumulate_params, cudaStream_t st);

// Many-rows variants (weights_rows.cu), used from kManyRows rows on.
constexpr int64_t kManyRows = 64;
int phi_row_tiles(int64_t batch);
int64_t rows_bwd_extra_floats(int64_t batch, int64_t K);
int project_rows_launch(const float* x, const float* phi, float* part, int64_t batch, int64_t K, int ks_max,
                        cudaStream_t st, int* ks_used);
int bwd_rows_launch(const float* x, const float* phi, const float* buf, float* phi_part, float* grad_x, float* grad_phi,
                    float* grad_bias, float* grad_alpha, int64_t batch, int64_t K, int accumulate, cudaStream_t st);

// Tensor-core (tcgen05) kernels for many rows (weights_rows_tc.cu).
int64_t rows_tc_fwd_scratch_bytes(int64_t K);
bool rows_tc_usable(const float* x, int64_t batch, int64_t K);
int rows_fwd_tc_launch(const float* x, const float* phi, BiasPtrs bias, const float* alpha_pre, const float* alpha_post,
                       const float* alpha_res, float* H_pre, float* H_post, float* H_res, float* saved, void* scratch,
                       int64_t batch, int64_t K, int iters, float eps, cudaStream_t st);

int64_t rows_tc_bwd_scratch_floats(int64_t K);
int rows_bwd_tc_launch(const float* x, const float* phi, const float* buf, float* phi_part, float* grad_x,
                       float* scratch, int64_t batch, int64_t K, int max_groups, cudaStream_t st, int* groups_used);

int64_t weights_fwd_scratch_bytes(int64_t batch, int64_t K);
int64_t weights_bwd_scratch_bytes(int64_t batch, int64_t K);

}  // namespace mhc

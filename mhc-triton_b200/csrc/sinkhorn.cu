// Sinkhorn-Knopp projection of batches of 4x4 matrices: one thread owns one matrix, which
// never leaves its registers.  Forward = `iters` row/column normalisations of |M| + eps;
// backward = reverse sweep that re-derives each iteration's state from M (no saved state).
#include <cstdlib>

#include "common.cuh"
#include "launch.h"

namespace mhc {

// MHC_SINKHORN_PLAIN=1 in the environment selects the plain O(iters^2) sweep (for cross-checks).
static bool sinkhorn_plain_sweep() {
  static const bool on = [] {
    const char* e = std::getenv("MHC_SINKHORN_PLAIN");
    return e && e[0] == '1';
  }();
  return on;
}

template <typename T>
__device__ __forceinline__ void load_matrix(const T* __restrict__ p, float (&m)[16], bool aligned) {
  constexpr int V = vec_width<T>::value;
  if (aligned) {
#pragma unroll
    for (int i = 0; i < 16 / V; ++i) {
      float t[V];
      PackIO<T, V>::load(p + i * V, t);
#pragma unroll
      for (int j = 0; j < V; ++j) m[i * V + j] = t[j];
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = to_f32(p[i]);
  }
}

template <typename T>
__device__ __forceinline__ void store_matrix(T* __restrict__ p, const float (&m)[16], bool aligned) {
  constexpr int V = vec_width<T>::value;
  if (aligned) {
#pragma unroll
    for (int i = 0; i < 16 / V; ++i) {
      float t[V];
#pragma unroll
      for (int j = 0; j < V; ++j) t[j] = m[i * V + j];
      PackIO<T, V>::store(p + i * V, t);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) p[i] = from_f32<T>(m[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(128) k_sinkhorn_fwd(const T* __restrict__ M, T* __restrict__ P, int64_t batch,
                                                      int iters, float eps, bool aligned) {
  pdl_prologue();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch) return;
  float m[16];
  load_matrix(M + i * 16, m, aligned);
#pragma unroll
  for (int k = 0; k < 16; ++k) m[k] = fabsf(m[k]) + eps;
  for (int t = 0; t < iters; ++t) sinkhorn_step(m, eps);
  store_matrix(P + i * 16, m, aligned);
}

// Reverse sweep.  For t = iters-1 .. 0 the state entering iteration t is recomputed from M
// by running t forward iterations, so the work is iters*(iters+1)/2 + iters steps and nothing
// but M and dP is ever read.
template <typename T>
__global__ void __launch_bounds__(128) k_sinkhorn_bwd(const T* __restrict__ M, const T* __restrict__ dP,
                                                      T* __restrict__ dM, int64_t batch, int iters, float eps,
                                                      float sign_at_zero, bool aligned) {
  pdl_prologue();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch) return;
  float m0[16], d[16];
  load_matrix(M + i * 16, m0, aligned);
  load_matrix(dP + i * 16, d, aligned);
  for (int t = iters - 1; t >= 0; --t) {
    float m[16], r[4], c[4], mr[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) m[k] = fabsf(m0[k]) + eps;
    for (int f = 0; f < t; ++f) sinkhorn_step(m, eps);
    sinkhorn_step(m, eps, r, mr, c);
    sinkhorn_step_bwd(d, m, r, mr, c);
  }
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const float sg = m0[k] > 0.f ? 1.f : (m0[k] < 0.f ? -1.f : sign_at_zero);
    d[k] *= sg;
  }
  store_matrix(dM + i * 16, d, aligned);
}

// Same reverse sweep with kCk register-resident checkpoints: the iterations are cut into kCk + 1
// segments of L = ceil(iters / (kCk + 1)); one forward sweep stores the state entering each
// segment, and the state entering iteration t is then recomputed from its segment's checkpoint
// (at most L - 1 steps) instead of from M (t steps).  The recomputation runs the same step
// function from the same values, so the result is bit-identical to k_sinkhorn_bwd, for about
// iters * (L + 3) / 2 steps instead of iters * (iters + 1) / 2.  Still nothing but M and dP is read.
template <typename T>
__global__ void __launch_bounds__(128) k_sinkhorn_bwd_ck(const T* __restrict__ M, const T* __restrict__ dP,
                                                         T* __restrict__ dM, int64_t batch, int iters,
                                                         float eps, float sign_at_zero, bool aligned) {
  pdl_prologue();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch) return;
  float m0[16], d[16];
  load_matrix(M + i * 16, m0, aligned);
  load_matrix(dP + i * 16, d, aligned);
  sinkhorn_backward_ck(m0, d, iters, eps);
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const float sg = m0[k] > 0.f ? 1.f : (m0[k] < 0.f ? -1.f : sign_at_zero);
    d[k] *= sg;
  }
  store_matrix(dM + i * 16, d, aligned);
}

template <typename T>
static int launch_fwd(const void* M, void* P, int64_t batch, int iters, float eps, cudaStream_t st) {
  const bool aligned = is_aligned16(M) && is_aligned16(P);
  const int block = 128;
  const int64_t grid = (batch + block - 1) / block;
  {
    ProfScope ps("k_sinkhorn_fwd", st);
    launch_k(k_sinkhorn_fwd<T>, (unsigned)grid, block, 0, st, (const T*)M, (T*)P, batch, iters, eps, aligned);
  }
  return check_launch("sinkhorn_fwd");
}

template <typename T>
static int launch_bwd(const void* M, const void* dP, void* dM, int64_t batch, int iters, float eps, float sz,
                      cudaStream_t st) {
  const bool aligned = is_aligned16(M) && is_aligned16(dP) && is_aligned16(dM);
  const int block = 128;
  const int64_t grid = (batch + block - 1) / block;
  if (sinkhorn_plain_sweep()) {
    ProfScope ps("k_sinkhorn_bwd", st);
    launch_k(k_sinkhorn_bwd<T>, (unsigned)grid, block, 0, st, (const T*)M, (const T*)dP, (T*)dM, batch, iters, eps, sz,
             aligned);
  } else {
    ProfScope ps("k_sinkhorn_bwd_ck", st);
    launch_k(k_sinkhorn_bwd_ck<T>, (unsigned)grid, block, 0, st, (const T*)M, (const T*)dP, (T*)dM, batch, iters, eps,
             sz, aligned);
  }
  return check_launch("sinkhorn_bwd");
}

}  // namespace mhc

using namespace mhc;

extern "C" int mhc_sinkhorn_fwd(const void* M, void* P, int64_t batch, int dtype, int iters, float eps,
                                mhc_stream_t stream) {
  if (batch == 0) return MHC_OK;
  if (!M || !P) return fail(MHC_ERR_NULL_POINTER, "sinkhorn_fwd: null pointer");
  if (batch < 0 || batch > kMaxGridItems * 128) return fail(MHC_ERR_BAD_SHAPE, "sinkhorn_fwd: bad batch");
  if (iters < 0) return fail(MHC_ERR_BAD_ARGUMENT, "sinkhorn_fwd: iters < 0");
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case MHC_F32: return launch_fwd<float>(M, P, batch, iters, eps, st);
    case MHC_BF16: return launch_fwd<__nv_bfloat16>(M, P, batch, iters, eps, st);
    case MHC_F16: return launch_fwd<__half>(M, P, batch, iters, eps, st);
  }
  return fail(MHC_ERR_BAD_DTYPE, "sinkhorn_fwd: unknown dtype");
}

extern "C" int mhc_sinkhorn_bwd(const void* M, const void* dP, void* dM, int64_t batch, int dtype, int iters,
                                float eps, int abs_grad_at_zero, mhc_stream_t stream) {
  if (batch == 0) return MHC_OK;
  // scalar arguments first, pointers last: a call with bad scalars and null pointers reports the scalars
  if (batch < 0 || batch > kMaxGridItems * 128) return fail(MHC_ERR_BAD_SHAPE, "sinkhorn_bwd: bad batch");
  if (iters < 0) return fail(MHC_ERR_BAD_ARGUMENT, "sinkhorn_bwd: iters < 0");
  if (abs_grad_at_zero != MHC_ABS0_ZERO && abs_grad_at_zero != MHC_ABS0_PLUS_ONE)
    return fail(MHC_ERR_BAD_ARGUMENT, "sinkhorn_bwd: abs_grad_at_zero must be 0 or 1");
  if (!M || !dP || !dM) return fail(MHC_ERR_NULL_POINTER, "sinkhorn_bwd: null pointer");
  const float sz = abs_grad_at_zero == MHC_ABS0_PLUS_ONE ? 1.f : 0.f;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case MHC_F32: return launch_bwd<float>(M, dP, dM, batch, iters, eps, sz, st);
    case MHC_BF16: return launch_bwd<__nv_bfloat16>(M, dP, dM, batch, iters, eps, sz, st);
    case MHC_F16: return launch_bwd<__half>(M, dP, dM, batch, iters, eps, sz, st);
  }
  return fail(MHC_ERR_BAD_DTYPE, "sinkhorn_bwd: unknown dtype");
}

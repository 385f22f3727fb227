// Dynamic connection weights: split-K projection x*phi with sum(x^2) in the same pass, then a
// one-warp finish per row (RMS norm, scale + bias, sigmoids, register-resident Sinkhorn), and
// the matching backward (Sinkhorn reverse sweep, activation / norm algebra, grad_x, grad_phi,
// grad_bias, grad_alpha).  phi is read in its parameter layout [K, 24]: one row is 96
// contiguous bytes, so consecutive k read consecutive memory and no transposed copy exists.
#include "common.cuh"
#include "launch.h"

namespace mhc {

constexpr int kProjW = 25;       // 24 dot products + sum of squares
constexpr int kBwdStride = 56;   // per-row buffer of the backward: ds[24] d_raw[24] coef ga[3] pad
constexpr int kMaxStoredIters = 64;

static inline int k_slices(int64_t K) {
  int64_t ks = (K + 255) / 256;
  if (ks > 128) ks = 128;
  if (ks < 1) ks = 1;
  return (int)ks;
}

int64_t weights_fwd_scratch_bytes(int64_t batch, int64_t K) {
  const int64_t n = batch * k_slices(K) * kProjW * (int64_t)sizeof(float);
  if (batch < kManyRows) return n;
  const int64_t tc = rows_tc_fwd_scratch_bytes(K);   // the tensor-core path keeps a split copy of phi instead
  return n > tc ? n : tc;
}
int64_t weights_bwd_scratch_bytes(int64_t batch, int64_t K) {
  int64_t n = batch * kBwdStride;                                   // per-row records
  if (batch >= kManyRows) n += rows_bwd_extra_floats(batch, K);       // grad_phi partial sums, column sums
  return n * (int64_t)sizeof(float);
}

__device__ __forceinline__ void load_phi_row(const float* __restrict__ phi, int64_t k, bool aligned, float (&p)[24]) {
  const float* row = phi + k * 24;
  if (aligned) {
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(row) + i);
      p[4 * i] = v.x; p[4 * i + 1] = v.y; p[4 * i + 2] = v.z; p[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 24; ++i) p[i] = __ldg(row + i);
  }
}

__device__ __forceinline__ float bias_at(const BiasPtrs& b, int j) {
  return j < 4 ? __ldg(b.pre + j) : (j < 8 ? __ldg(b.post + (j - 4)) : __ldg(b.res + (j - 8)));
}

__device__ __forceinline__ float group_alpha(int j, float a_pre, float a_post, float a_res) {
  return j < 4 ? a_pre : (j < 8 ? a_post : a_res);
}

// One warp finishes one row from its [ks, 25] slice sums: lanes 0..24 add the slices (fp64, index
// order); lanes 0..7 do the sigmoids; lane 8 runs the Sinkhorn projection in registers.
// FRESH: the slice sums were written by other CTAs of the same kernel (read through L2).
template <bool FRESH>
__device__ __forceinline__ void dw_finish_row(const float* __restrict__ part_row, const BiasPtrs& bias,
                                              const float* __restrict__ alpha_pre, const float* __restrict__ alpha_post,
                                              const float* __restrict__ alpha_res, float* __restrict__ H_pre,
                                              float* __restrict__ H_post, float* __restrict__ H_res,
                                              float* __restrict__ saved, int64_t row, int64_t K, int ks, int iters,
                                              float eps, float* s_sc) {
  const int lane = threadIdx.x & 31;
  float tot = 0.f;
  if (lane < kProjW) {
    double t[4] = {0.0, 0.0, 0.0, 0.0};   // four interleaved chains so that the loads overlap; fixed order
    const float* p = part_row + lane;
    int s = 0;
    for (; s + 4 <= ks; s += 4) {
#pragma unroll
      for (int u = 0; u < 4; ++u)
        t[u] += (double)(FRESH ? __ldcg(p + (s + u) * kProjW) : __ldg(p + (s + u) * kProjW));
    }
    for (; s < ks; ++s) t[0] += (double)(FRESH ? __ldcg(p + s * kProjW) : __ldg(p + s * kProjW));
    tot = (float)((t[0] + t[1]) + (t[2] + t[3]));
  }
  const float q = __shfl_sync(0xffffffffu, tot, 24);
  const float inv_rms = 1.f / sqrtf(q / (float)K + eps);
  const float a_pre = __ldg(alpha_pre), a_post = __ldg(alpha_post), a_res = __ldg(alpha_res);
  float sc = 0.f;
  if (lane < 24) {
    sc = (inv_rms * group_alpha(lane, a_pre, a_post, a_res)) * tot + bias_at(bias, lane);
    s_sc[lane] = sc;
    if (saved) saved[row * kSavedStride + lane] = tot;
  }
  if (saved && lane == 24) {
    saved[row * kSavedStride + 24] = q;
    saved[row * kSavedStride + 25] = inv_rms;
  }
  __syncwarp();
  const float sg = sigmoidf_(sc);
  // sum of the four pre-mix sigmoids, in index order, visible to lanes 0..3
  const float s0 = __shfl_sync(0xffffffffu, sg, 0), s1 = __shfl_sync(0xffffffffu, sg, 1),
              s2 = __shfl_sync(0xffffffffu, sg, 2), s3 = __shfl_sync(0xffffffffu, sg, 3);
  if (lane < 4) H_pre[row * 4 + lane] = sg / ((((s0 + s1) + s2) + s3) + eps);
  else if (lane < 8) H_post[row * 4 + (lane - 4)] = 2.f * sg;
  else if (lane == 8) {
    float m[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = fabsf(s_sc[8 + i]) + eps;
    for (int t = 0; t < iters; ++t) sinkhorn_step(m, eps);
#pragma unroll
    for (int i = 0; i < 16; ++i) H_res[row * 16 + i] = m[i];
  }
}

// What the finish of a row needs besides the slice sums.
struct FinishArgs {
  BiasPtrs bias;
  const float *alpha_pre, *alpha_post, *alpha_res;
  float *H_pre, *H_post, *H_res, *saved;
  int iters;
  float eps;
  int* tickets;   // one zeroed counter per row, or null: a separate kernel finishes the rows
};

// part[row, slice, 0..23] = sum over the slice's k of x[row,k] phi[k,:];  part[row, slice, 24] = sum x^2.
// x[row,k] = scale * sum_{c < nsrc} xsrc[(row*nsrc + c)*K + k]: with nsrc = 1, scale = 1 this is a plain
// read of x; with the mean-pool partials as xsrc it finishes the pooling (chunks added in index
// order, fp64) and writes the pooled state to x_out for the backward.
// With tickets, the CTA that stores the last slice of a row also finishes that row (dw_finish_row),
// so the weights are ready when this kernel ends and no second launch sits on the critical path.
__global__ void __launch_bounds__(256)
k_dw_project(const float* __restrict__ xsrc, int nsrc, double scale, float* __restrict__ x_out,
             const float* __restrict__ phi, float* __restrict__ part, int64_t K, int ks, bool phi_aligned,
             FinishArgs fin) {
  pdl_prologue();
  __shared__ float red[32 * kProjW];
  __shared__ float s_sc[24];
  const int64_t row = blockIdx.x / ks;
  const int slice = (int)(blockIdx.x % ks);
  const int64_t per = (K + ks - 1) / ks;
  const int64_t k0 = slice * per, k1 = min(k0 + per, K);
  float acc[kProjW];
#pragma unroll
  for (int i = 0; i < kProjW; ++i) acc[i] = 0.f;
  const float* xr = xsrc + row * nsrc * K;
  for (int64_t k = k0 + threadIdx.x; k < k1; k += blockDim.x) {
    float xv;
    if (nsrc == 1) {
      xv = scale == 1.0 ? __ldg(xr + k) : (float)((double)__ldg(xr + k) * scale);
    } else {
      xv = (float)(sum_strided_f64(xr + k, K, nsrc) * scale);
    }
    if (x_out) x_out[row * K + k] = xv;
    float p[24];
    load_phi_row(phi, k, phi_aligned, p);
#pragma unroll
    for (int j = 0; j < 24; ++j) acc[j] = fmaf(xv, p[j], acc[j]);
    acc[24] = fmaf(xv, xv, acc[24]);
  }
  block_reduce_store<kProjW>(acc, part + (row * ks + slice) * kProjW, red);
  if (!fin.tickets) return;
  if (!cta_arrives_last(fin.tickets + row, ks)) return;
  if (threadIdx.x < 32)
    dw_finish_row<true>(part + row * ks * kProjW, fin.bias, fin.alpha_pre, fin.alpha_post, fin.alpha_res, fin.H_pre,
                        fin.H_post, fin.H_res, fin.saved, row, K, ks, fin.iters, fin.eps, s_sc);
}

// One warp per row: the finish as a kernel of its own (rows projected by the many-rows kernels, or
// callers without ticket counters).
__global__ void __launch_bounds__(32)
k_dw_finish(const float* __restrict__ part, BiasPtrs bias, const float* __restrict__ alpha_pre,
            const float* __restrict__ alpha_post, const float* __restrict__ alpha_res, float* __restrict__ H_pre,
            float* __restrict__ H_post, float* __restrict__ H_res, float* __restrict__ saved, int64_t K, int ks,
            int iters, float eps) {
  pdl_prologue();
  __shared__ float s_sc[24];
  const int64_t row = blockIdx.x;
  dw_finish_row<false>(part + row * ks * kProjW, bias, alpha_pre, alpha_post, alpha_res, H_pre, H_post, H_res, saved,
                       row, K, ks, iters, eps, s_sc);
}

// Backward of one row by one warp: gradients of the 24 pre-activation values (ds), of the raw
// projections (d_raw), the coefficient of x in grad_x that comes from the RMS norm (coef), and this
// row's share of grad_alpha (ga: pre, post, res).
//   up     : 20 floats in shared memory, dH_pre[4] then dH_res[16] of this row
//   s_sc, s_ds : 24 floats of shared memory each, private to the warp
//   state  : [min(iters, kMaxStoredIters)][40] floats of shared memory private to the warp, holding
//            every Sinkhorn iteration's r[4] c[4] mr[16] m_out[16]; with more iterations than that
//            the states are recomputed per step instead
// Lanes 0..7 handle the sigmoid outputs, lane 8 runs the Sinkhorn reverse sweep.  On return lanes
// 0..23 hold ds and d_raw of their index; lane 0 holds coef and ga.
__device__ __forceinline__ void dw_bwd_row_warp(const float* __restrict__ saved_row, const BiasPtrs& bias,
                                                float a_pre, float a_post, float a_res, const float* up,
                                                const float* __restrict__ dH_post_row, float* s_sc, float* s_ds,
                                                float (*state)[40], int64_t K, int iters, float eps,
                                                float sign_at_zero, float& ds, float& d_raw, float& coef,
                                                float (&ga)[3]) {
  const int lane = threadIdx.x & 31;
  const float inv_rms = __ldg(saved_row + 25);
  const float alpha = group_alpha(lane, a_pre, a_post, a_res);
  float raw = 0.f, sc = 0.f;
  if (lane < 24) {
    raw = __ldg(saved_row + lane);
    sc = (inv_rms * alpha) * raw + bias_at(bias, lane);
    s_sc[lane] = sc;
  }
  __syncwarp();
  const float sg = sigmoidf_(sc);
  float g = 0.f;
  if (lane < 4) g = up[lane];
  else if (lane < 8) g = __ldg(dH_post_row + lane - 4);
  // pre-mix: H_pre = sg / (sum + eps);  d sg = (g - <g, H_pre>) / (sum + eps)
  const float s0 = __shfl_sync(0xffffffffu, sg, 0), s1 = __shfl_sync(0xffffffffu, sg, 1),
              s2 = __shfl_sync(0xffffffffu, sg, 2), s3 = __shfl_sync(0xffffffffu, sg, 3);
  const float ssum = (((s0 + s1) + s2) + s3) + eps;
  const float gh = lane < 4 ? g * (sg / ssum) : 0.f;
  const float dot = ((__shfl_sync(0xffffffffu, gh, 0) + __shfl_sync(0xffffffffu, gh, 1)) +
                     __shfl_sync(0xffffffffu, gh, 2)) + __shfl_sync(0xffffffffu, gh, 3);
  ds = 0.f;
  if (lane < 4) ds = ((g - dot) / ssum) * sg * (1.f - sg);
  else if (lane < 8) ds = g * 2.f * sg * (1.f - sg);
  if (lane < 8) s_ds[lane] = ds;
  if (lane == 8) {
    float m0[16], d[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      m0[i] = s_sc[8 + i];
      d[i] = up[4 + i];
    }
    if (iters <= kMaxStoredIters) {
      float m[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) m[i] = fabsf(m0[i]) + eps;
      for (int t = 0; t < iters; ++t) {
        float r[4], c[4], mr[16];
        sinkhorn_step(m, eps, r, mr, c);
#pragma unroll
        for (int i = 0; i < 4; ++i) { state[t][i] = r[i]; state[t][4 + i] = c[i]; }
#pragma unroll
        for (int i = 0; i < 16; ++i) { state[t][8 + i] = mr[i]; state[t][24 + i] = m[i]; }
      }
      for (int t = iters - 1; t >= 0; --t) {
        float r[4], c[4], mr[16], mo[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) { r[i] = state[t][i]; c[i] = state[t][4 + i]; }
#pragma unroll
        for (int i = 0; i < 16; ++i) { mr[i] = state[t][8 + i]; mo[i] = state[t][24 + i]; }
        sinkhorn_step_bwd(d, mo, r, mr, c);
      }
    } else {
      for (int t = iters - 1; t >= 0; --t) {
        float m[16], r[4], c[4], mr[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) m[i] = fabsf(m0[i]) + eps;
        for (int f = 0; f < t; ++f) sinkhorn_step(m, eps);
        sinkhorn_step(m, eps, r, mr, c);
        sinkhorn_step_bwd(d, m, r, mr, c);
      }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float sgn = m0[i] > 0.f ? 1.f : (m0[i] < 0.f ? -1.f : sign_at_zero);
      s_ds[8 + i] = d[i] * sgn;
    }
  }
  __syncwarp();
  float t_inv = 0.f, t_alpha = 0.f;
  d_raw = 0.f;
  if (lane < 24) {
    ds = s_ds[lane];
    d_raw = (ds * inv_rms) * alpha;
    t_inv = (ds * alpha) * raw;       // this lane's term of d(inv_rms)
    t_alpha = (ds * inv_rms) * raw;   // this lane's term of d(alpha_group)
  }
  // fixed-order sums over lanes 0..3, 4..7, 8..23 (every lane gathers the same values)
  float inv_g[3] = {0.f, 0.f, 0.f};
  ga[0] = ga[1] = ga[2] = 0.f;
#pragma unroll
  for (int j = 0; j < 24; ++j) {
    const float a = __shfl_sync(0xffffffffu, t_inv, j), b = __shfl_sync(0xffffffffu, t_alpha, j);
    const int gi = j < 4 ? 0 : (j < 8 ? 1 : 2);
    inv_g[gi] += a;
    ga[gi] += b;
  }
  const float d_inv_rms = (inv_g[0] + inv_g[1]) + inv_g[2];
  // inv_rms = 1/rms: d rms = -d_inv_rms * inv_rms^2;  rms = sqrt(sum x^2 / K + eps): d x = d rms * x / (K rms)
  const float d_rms = d_inv_rms * (-(inv_rms * inv_rms));
  coef = d_rms * inv_rms / (float)K;
}

// Per-row records of the backward, one CTA per row:
//   buf[row, 0..23] ds   buf[row, 24..47] d_raw   buf[row, 48] coef   buf[row, 49..51] ga(pre,post,res)
// If part20 is given, dH_pre / dH_res are first summed from the [slots, 20] per-CTA partials of the
// stream-mix reduction pass (fp64, fixed order) and also written to dH_pre / dH_res; otherwise they
// are read from there.  Then warp 0 works alone (dw_bwd_row_warp).
__global__ void __launch_bounds__(256)
k_dw_bwd_rows(const float* __restrict__ saved, BiasPtrs bias, const float* __restrict__ alpha_pre,
              const float* __restrict__ alpha_post, const float* __restrict__ alpha_res,
              const float* __restrict__ part20, int64_t slots, float* __restrict__ dH_pre,
              const float* __restrict__ dH_post, float* __restrict__ dH_res, float* __restrict__ buf, int64_t K,
              int iters, float eps, float sign_at_zero) {
  pdl_prologue();
  __shared__ float s_sc[24], s_ds[24], s_up[20];
  __shared__ double s_red[8][20];
  __shared__ float s_state[kMaxStoredIters][40];
  const int64_t row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (part20) {
    block_column_sums_fast<20, false>(part20 + row * slots * 20, slots, s_red);
    if (threadIdx.x < 20) {
      double t = 0.0;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += s_red[w][threadIdx.x];
      const float v = (float)t;
      s_up[threadIdx.x] = v;
      if (threadIdx.x < 4) dH_pre[row * 4 + threadIdx.x] = v;
      else dH_res[row * 16 + threadIdx.x - 4] = v;
    }
  } else if (threadIdx.x < 20) {
    s_up[threadIdx.x] = threadIdx.x < 4 ? dH_pre[row * 4 + threadIdx.x] : dH_res[row * 16 + threadIdx.x - 4];
  }
  __syncthreads();
  if (warp != 0) return;
  float ds, d_raw, coef, ga[3];
  dw_bwd_row_warp(saved + row * kSavedStride, bias, __ldg(alpha_pre), __ldg(alpha_post), __ldg(alpha_res), s_up,
                  dH_post + row * 4, s_sc, s_ds, s_state, K, iters, eps, sign_at_zero, ds, d_raw, coef, ga);
  if (lane < 24) {
    buf[row * kBwdStride + lane] = ds;
    buf[row * kBwdStride + 24 + lane] = d_raw;
  }
  if (lane == 0) {
    buf[row * kBwdStride + 48] = coef;
    buf[row * kBwdStride + 49] = ga[0];
    buf[row * kBwdStride + 50] = ga[1];
    buf[row * kBwdStride + 51] = ga[2];
  }
}

// The same per-row records for MANY rows (per-token use): one THREAD per row, everything in registers,
// the Sinkhorn reverse sweep with register checkpoints (sinkhorn_backward_ck) instead of states in
// shared memory.  Same formulas and summation orders as dw_bwd_row_warp, so the records are
// bit-identical to k_dw_bwd_rows'.  dH_pre / dH_res hold finished sums.
__global__ void __launch_bounds__(128)
k_dw_bwd_rows_thread(const float* __restrict__ saved, BiasPtrs bias, const float* __restrict__ alpha_pre,
                     const float* __restrict__ alpha_post, const float* __restrict__ alpha_res,
                     const float* __restrict__ dH_pre, const float* __restrict__ dH_post,
                     const float* __restrict__ dH_res, float* __restrict__ buf, int64_t batch, int64_t K, int iters,
                     float eps, float sign_at_zero) {
  pdl_prologue();
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= batch) return;
  const float* sv = saved + row * kSavedStride;
  const float inv_rms = __ldg(sv + 25);
  const float a_pre = __ldg(alpha_pre), a_post = __ldg(alpha_post), a_res = __ldg(alpha_res);
  float raw[24], sc[24], ds[24];
#pragma unroll
  for (int j = 0; j < 24; ++j) {
    raw[j] = __ldg(sv + j);
    sc[j] = (inv_rms * group_alpha(j, a_pre, a_post, a_res)) * raw[j] + bias_at(bias, j);
  }
  float sg[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) sg[j] = sigmoidf_(sc[j]);
  const float ssum = (((sg[0] + sg[1]) + sg[2]) + sg[3]) + eps;
  float g[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    g[j] = __ldg(dH_pre + row * 4 + j);
    g[4 + j] = __ldg(dH_post + row * 4 + j);
  }
  const float dot = ((g[0] * (sg[0] / ssum) + g[1] * (sg[1] / ssum)) + g[2] * (sg[2] / ssum)) + g[3] * (sg[3] / ssum);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    ds[j] = ((g[j] - dot) / ssum) * sg[j] * (1.f - sg[j]);
    ds[4 + j] = g[4 + j] * 2.f * sg[4 + j] * (1.f - sg[4 + j]);
  }
  {
    float m0[16], d[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      m0[i] = sc[8 + i];
      d[i] = __ldg(dH_res + row * 16 + i);
    }
    sinkhorn_backward_ck(m0, d, iters, eps);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float sgn = m0[i] > 0.f ? 1.f : (m0[i] < 0.f ? -1.f : sign_at_zero);
      ds[8 + i] = d[i] * sgn;
    }
  }
  float inv_g[3] = {0.f, 0.f, 0.f}, ga[3] = {0.f, 0.f, 0.f};
  float* o = buf + row * kBwdStride;
#pragma unroll
  for (int j = 0; j < 24; ++j) {
    const float alpha = group_alpha(j, a_pre, a_post, a_res);
    const int gi = j < 4 ? 0 : (j < 8 ? 1 : 2);
    inv_g[gi] += (ds[j] * alpha) * raw[j];
    ga[gi] += (ds[j] * inv_rms) * raw[j];
    o[j] = ds[j];
    o[24 + j] = (ds[j] * inv_rms) * alpha;
  }
  const float d_inv_rms = (inv_g[0] + inv_g[1]) + inv_g[2];
  const float d_rms = d_inv_rms * (-(inv_rms * inv_rms));
  o[48] = d_rms * inv_rms / (float)K;
  o[49] = ga[0];
  o[50] = ga[1];
  o[51] = ga[2];
}

// grad_x[row,k] = sum_j d_raw[row,j] phi[k,j] + coef[row] x[row,k];  grad_phi[k,j] = sum_row x[row,k] d_raw[row,j]
// (rows added in index order, fp64 accumulators).  The last CTA sums grad_bias and grad_alpha over rows.
constexpr int kRowTile = 32;
__global__ void __launch_bounds__(256)
k_dw_bwd_main(const float* __restrict__ x, const float* __restrict__ phi, const float* __restrict__ buf,
              float* __restrict__ grad_x, float* __restrict__ grad_phi, float* __restrict__ grad_bias,
              float* __restrict__ grad_alpha, int64_t batch, int64_t K, bool phi_aligned, bool gphi_aligned,
              int accumulate) {
  pdl_prologue();
  __shared__ float s_draw[kRowTile][25];
  if (blockIdx.x == gridDim.x - 1) {  // parameter sums over rows
    const int j = threadIdx.x;
    if (j < 27) {
      const int col = j < 24 ? j : 49 + (j - 24);
      double a = 0.0;
      for (int64_t r = 0; r < batch; ++r) a += (double)__ldg(buf + r * kBwdStride + col);
      float* dst = j < 24 ? grad_bias + j : grad_alpha + (j - 24);
      *dst = accumulate ? *dst + (float)a : (float)a;
    }
    return;
  }
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = k < K;
  float p[24];
  double acc[24];
#pragma unroll
  for (int j = 0; j < 24; ++j) { p[j] = 0.f; acc[j] = 0.0; }
  if (live) load_phi_row(phi, k, phi_aligned, p);
  for (int64_t r0 = 0; r0 < batch; r0 += kRowTile) {
    const int nr = (int)min((int64_t)kRowTile, batch - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < nr * 25; i += blockDim.x) {
      const int rr = i / 25, jj = i % 25;
      s_draw[rr][jj] = __ldg(buf + (r0 + rr) * kBwdStride + 24 + jj);  // d_raw[24] then coef
    }
    __syncthreads();
    if (live) {
      for (int rr = 0; rr < nr; ++rr) {
        const float xv = __ldg(x + (r0 + rr) * K + k);
        double gx = (double)s_draw[rr][24] * (double)xv;
#pragma unroll
        for (int j = 0; j < 24; ++j) {
          gx += (double)s_draw[rr][j] * (double)p[j];
          acc[j] += (double)xv * (double)s_draw[rr][j];
        }
        grad_x[(r0 + rr) * K + k] = (float)gx;
      }
    }
  }
  if (live) {
    float* o = grad_phi + k * 24;
    if (gphi_aligned) {
#pragma unroll
      for (int i = 0; i < 6; ++i) {
        float4 v = make_float4((float)acc[4 * i], (float)acc[4 * i + 1], (float)acc[4 * i + 2], (float)acc[4 * i + 3]);
        float4* dst = reinterpret_cast<float4*>(o) + i;
        if (accumulate) { const float4 old = *dst; v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w; }
        *dst = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 24; ++j) o[j] = accumulate ? o[j] + (float)acc[j] : (float)acc[j];
    }
  }
}

// The two kernels above in one, for up to kFusedRows rows (the per-GPU batch of the layer path):
// every CTA first works out the records of ALL rows by itself (warp w takes rows w, w + 8, ...; a few
// microseconds of redundant arithmetic on 20 + 32 values per row), keeps them in shared memory, and
// then does its 256 columns of grad_x / grad_phi.  No CTA waits for another one and one launch less
// sits between the reduction pass and the apply pass of the layer's backward.  The results are
// bit-identical to k_dw_bwd_rows + k_dw_bwd_main.  dH_pre / dH_res must hold the finished sums.
// Dynamic shared memory: 8 warps x min(iters, kMaxStoredIters) x 40 floats of Sinkhorn states.
constexpr int kFusedRows = 16;
__global__ void __launch_bounds__(256)
k_dw_bwd_fused(const float* __restrict__ x, const float* __restrict__ phi, const float* __restrict__ saved,
               BiasPtrs bias, const float* __restrict__ alpha_pre, const float* __restrict__ alpha_post,
               const float* __restrict__ alpha_res, const float* __restrict__ dH_pre,
               const float* __restrict__ dH_post, const float* __restrict__ dH_res, float* __restrict__ grad_x,
               float* __restrict__ grad_phi, float* __restrict__ grad_bias, float* __restrict__ grad_alpha,
               int batch, int64_t K, int iters, float eps, float sign_at_zero, bool phi_aligned,
               bool gphi_aligned, int accumulate) {
  pdl_prologue();
  extern __shared__ float s_states[];   // [8][stored][40]
  __shared__ float s_draw[kFusedRows][25];   // d_raw[24], coef
  __shared__ float s_sums[kFusedRows][27];   // ds[24], ga[3]: what grad_bias / grad_alpha add up
  __shared__ float s_sc[8][24], s_ds[8][24], s_up[8][20];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int stored = iters <= kMaxStoredIters ? iters : 0;
  float (*state)[40] = reinterpret_cast<float (*)[40]>(s_states + (size_t)warp * stored * 40);
  const float a_pre = __ldg(alpha_pre), a_post = __ldg(alpha_post), a_res = __ldg(alpha_res);
  for (int row = warp; row < batch; row += 8) {
    if (lane < 20) s_up[warp][lane] = lane < 4 ? __ldg(dH_pre + row * 4 + lane) : __ldg(dH_res + row * 16 + lane - 4);
    __syncwarp();
    float ds, d_raw, coef, ga[3];
    dw_bwd_row_warp(saved + (int64_t)row * kSavedStride, bias, a_pre, a_post, a_res, s_up[warp], dH_post + row * 4,
                    s_sc[warp], s_ds[warp], state, K, iters, eps, sign_at_zero, ds, d_raw, coef, ga);
    if (lane < 24) {
      s_draw[row][lane] = d_raw;
      s_sums[row][lane] = ds;
    }
    if (lane == 0) {
      s_draw[row][24] = coef;
      s_sums[row][24] = ga[0];
      s_sums[row][25] = ga[1];
      s_sums[row][26] = ga[2];
    }
    __syncwarp();
  }
  __syncthreads();
  if (blockIdx.x == gridDim.x - 1) {  // parameter sums over rows
    const int j = threadIdx.x;
    if (j < 27) {
      double a = 0.0;
      for (int r = 0; r < batch; ++r) a += (double)s_sums[r][j];
      float* dst = j < 24 ? grad_bias + j : grad_alpha + (j - 24);
      *dst = accumulate ? *dst + (float)a : (float)a;
    }
    return;
  }
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  float p[24];
  double acc[24];
#pragma unroll
  for (int j = 0; j < 24; ++j) acc[j] = 0.0;
  load_phi_row(phi, k, phi_aligned, p);
  for (int rr = 0; rr < batch; ++rr) {
    const float xv = __ldg(x + (int64_t)rr * K + k);
    double gx = (double)s_draw[rr][24] * (double)xv;
#pragma unroll
    for (int j = 0; j < 24; ++j) {
      gx += (double)s_draw[rr][j] * (double)p[j];
      acc[j] += (double)xv * (double)s_draw[rr][j];
    }
    grad_x[(int64_t)rr * K + k] = (float)gx;
  }
  float* o = grad_phi + k * 24;
  if (gphi_aligned) {
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      float4 v = make_float4((float)acc[4 * i], (float)acc[4 * i + 1], (float)acc[4 * i + 2], (float)acc[4 * i + 3]);
      float4* dst = reinterpret_cast<float4*>(o) + i;
      if (accumulate) { const float4 old = *dst; v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w; }
      *dst = v;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 24; ++j) o[j] = accumulate ? o[j] + (float)acc[j] : (float)acc[j];
  }
}

// ------------------------------------------------------------------------------ host side
int weights_fwd_impl(const float* xsrc, int nsrc, double scale, float* x_out, const float* phi, BiasPtrs bias,
                     const float* alpha_pre, const float* alpha_post, const float* alpha_res, float* H_pre,
                     float* H_post, float* H_res, float* saved, float* part, int64_t batch, int64_t K, int iters,
                     float eps, int* tickets, cudaStream_t st) {
  int ks = k_slices(K);
  const bool many_rows = nsrc == 1 && scale == 1.0 && !x_out && batch >= kManyRows;
  if (many_rows && rows_tc_usable(xsrc, batch, K))   // tcgen05 projection with the finish as its epilogue
    return rows_fwd_tc_launch(xsrc, phi, bias, alpha_pre, alpha_post, alpha_res, H_pre, H_post, H_res, saved, part, batch,
                              K, iters, eps, st);
  if (many_rows) {
    if (int e = project_rows_launch(xsrc, phi, part, batch, K, ks, st, &ks)) return e;
  } else {
    if (batch * ks > kMaxGridItems) return fail(MHC_ERR_BAD_SHAPE, "dynamic_weights_fwd: batch too large");
    const FinishArgs fin{bias, alpha_pre, alpha_post, alpha_res, H_pre, H_post, H_res, saved, iters, eps, tickets};
    {
      ProfScope ps("k_dw_project", st);
      launch_k(k_dw_project, (unsigned)(batch * ks), 256, 0, st, xsrc, nsrc, scale, x_out, phi, part, K, ks,
               is_aligned16(phi), fin);
    }
    if (int e = check_launch("dynamic_weights_fwd(project)")) return e;
    if (tickets) return MHC_OK;   // the CTA that stored a row's last slice has finished the row
  }
  {
    ProfScope ps("k_dw_finish", st);
    launch_k(k_dw_finish, (unsigned)batch, 32, 0, st, part, bias, alpha_pre, alpha_post, alpha_res, H_pre, H_post, H_res,
                                                saved, K, ks, iters, eps);
  }
  return check_launch("dynamic_weights_fwd(finish)");
}

// part20 != null: dH_pre / dH_res are still per-CTA partial sums [batch, slots, 20] (summed by the rows
// kernel); part20 == null: dH_pre / dH_res hold the finished sums.
int weights_bwd_impl(const float* x, const float* phi, BiasPtrs bias, const float* alpha_pre, const float* alpha_post,
                     const float* alpha_res, const float* saved, const float* part20, int64_t slots, float* dH_pre,
                     const float* dH_post, float* dH_res, float* grad_x, float* grad_phi, float* grad_bias,
                     float* grad_alpha, float* buf, int64_t batch, int64_t K, int iters, float eps,
                     int abs_grad_at_zero, int accumulate_params, cudaStream_t st) {
  if (batch > kMaxGridItems) return fail(MHC_ERR_BAD_SHAPE, "dynamic_weights_bwd: batch too large");
  const float sign0 = abs_grad_at_zero == MHC_ABS0_PLUS_ONE ? 1.f : 0.f;
  const int64_t kblocks = (K + 255) / 256;
  if (batch && !part20 && batch <= kFusedRows && iters <= 32) {
    const size_t dyn = (size_t)8 * iters * 40 * sizeof(float);
    {
      ProfScope ps("k_dw_bwd_fused", st);
      launch_k(k_dw_bwd_fused, (unsigned)(kblocks + 1), 256, dyn, st, x, phi, saved, bias, alpha_pre, alpha_post,
               alpha_res, (const float*)dH_pre, dH_post, (const float*)dH_res, grad_x, grad_phi, grad_bias, grad_alpha,
               (int)batch, K, iters, eps, sign0, is_aligned16(phi), is_aligned16(grad_phi), accumulate_params);
    }
    return check_launch("dynamic_weights_bwd(fused)");
  }
  if (batch >= kManyRows && !part20) {
    {
      ProfScope ps("k_dw_bwd_rows_thread", st);
      launch_k(k_dw_bwd_rows_thread, (unsigned)((batch + 127) / 128), 128, 0, st, saved, bias, alpha_pre, alpha_post, alpha_res,
               (const float*)dH_pre, dH_post, (const float*)dH_res, buf, batch, K, iters, eps, sign0);
    }
    if (int e = check_launch("dynamic_weights_bwd(rows)")) return e;
  } else if (batch) {
    {
      ProfScope ps("k_dw_bwd_rows", st);
      launch_k(k_dw_bwd_rows, (unsigned)batch, part20 ? 256 : 32, 0, st, saved, bias, alpha_pre, alpha_post, alpha_res, part20, slots,
                                                     dH_pre, dH_post, dH_res, buf, K, iters, eps, sign0);
    }
    if (int e = check_launch("dynamic_weights_bwd(rows)")) return e;
  }
  if (batch >= kManyRows)
    return bwd_rows_launch(x, phi, buf, buf + batch * kBwdStride, grad_x, grad_phi, grad_bias, grad_alpha, batch, K,
                           accumulate_params, st);
  {
    ProfScope ps("k_dw_bwd_main", st);
    launch_k(k_dw_bwd_main, (unsigned)(kblocks + 1), 256, 0, st, x, phi, buf, grad_x, grad_phi, grad_bias, grad_alpha, batch, K,
                                                           is_aligned16(phi), is_aligned16(grad_phi), accumulate_params);
  }
  return check_launch("dynamic_weights_bwd(main)");
}

}  // namespace mhc

using namespace mhc;

extern "C" int mhc_dynamic_weights_fwd(const float* x, const float* phi, const float* bias, const float* alpha_pre,
                                       const float* alpha_post, const float* alpha_res, float* H_pre, float* H_post,
                                       float* H_res, float* saved, void* scratch, int64_t scratch_bytes,
                                       int64_t batch, int64_t K, int iters, float eps, mhc_stream_t stream) {
  if (batch < 0 || K <= 0) return fail(MHC_ERR_BAD_SHAPE, "dynamic_weights_fwd: bad shape");
  if (iters < 0) return fail(MHC_ERR_BAD_ARGUMENT, "dynamic_weights_fwd: iters < 0");
  if (batch == 0) return MHC_OK;
  if (!x || !phi || !bias || !alpha_pre || !alpha_post || !alpha_res || !H_pre || !H_post || !H_res || !scratch)
    return fail(MHC_ERR_NULL_POINTER, "dynamic_weights_fwd: null pointer");
  if (scratch_bytes < weights_fwd_scratch_bytes(batch, K))
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "dynamic_weights_fwd: scratch %lld < %lld bytes", (long long)scratch_bytes,
                (long long)weights_fwd_scratch_bytes(batch, K));
  return weights_fwd_impl(x, 1, 1.0, nullptr, phi, BiasPtrs{bias, bias + 4, bias + 8}, alpha_pre, alpha_post, alpha_res,
                          H_pre, H_post, H_res, saved, (float*)scratch, batch, K, iters, eps, nullptr,
                          (cudaStream_t)stream);
}

extern "C" int mhc_dynamic_weights_bwd(const float* x, const float* phi, const float* bias, const float* alpha_pre,
                                       const float* alpha_post, const float* alpha_res, const float* saved,
                                       const float* dH_pre, const float* dH_post, const float* dH_res, float* grad_x,
                                       float* grad_phi, float* grad_bias, float* grad_alpha, void* scratch,
                                       int64_t scratch_bytes, int64_t batch, int64_t K, int iters, float eps,
                                       int abs_grad_at_zero, int accumulate_params, mhc_stream_t stream) {
  if (batch < 0 || K <= 0) return fail(MHC_ERR_BAD_SHAPE, "dynamic_weights_bwd: bad shape");
  if (iters < 0) return fail(MHC_ERR_BAD_ARGUMENT, "dynamic_weights_bwd: iters < 0");
  if (abs_grad_at_zero != MHC_ABS0_ZERO && abs_grad_at_zero != MHC_ABS0_PLUS_ONE)
    return fail(MHC_ERR_BAD_ARGUMENT, "dynamic_weights_bwd: abs_grad_at_zero must be 0 or 1");
  if (!x && batch) return fail(MHC_ERR_NULL_POINTER, "dynamic_weights_bwd: null pointer");
  if (!phi || !bias || !alpha_pre || !alpha_post || !alpha_res || !grad_phi || !grad_bias || !grad_alpha)
    return fail(MHC_ERR_NULL_POINTER, "dynamic_weights_bwd: null pointer");
  if (batch && (!saved || !dH_pre || !dH_post || !dH_res || !grad_x || !scratch))
    return fail(MHC_ERR_NULL_POINTER, "dynamic_weights_bwd: null pointer");
  if (scratch_bytes < weights_bwd_scratch_bytes(batch, K))
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "dynamic_weights_bwd: scratch %lld < %lld bytes", (long long)scratch_bytes,
                (long long)weights_bwd_scratch_bytes(batch, K));
  return weights_bwd_impl(x, phi, BiasPtrs{bias, bias + 4, bias + 8}, alpha_pre, alpha_post, alpha_res, saved, nullptr,
                          0, const_cast<float*>(dH_pre), dH_post, const_cast<float*>(dH_res), grad_x, grad_phi,
                          grad_bias, grad_alpha, (float*)scratch, batch, K, iters, eps, abs_grad_at_zero,
                          accumulate_params, (cudaStream_t)stream);
}

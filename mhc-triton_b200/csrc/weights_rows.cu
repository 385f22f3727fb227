// Dynamic weights for MANY rows (per-token use: x [B*S, 4D]).  The few-rows kernels in weights.cu
// give every row its own CTAs, which re-reads phi once per row; from kManyRows rows on, these
// kernels tile over rows instead so that phi (forward) and x (backward) are read once per tile:
//   forward : one thread per row, 128 rows per CTA, x and phi staged through shared memory in
//             32-wide K tiles; same [row, slice, 25] partial layout, so k_dw_finish is shared;
//   backward: grad_x tiled over (32 rows x 256 k); grad_phi as per-tile partial sums over row tiles
//             (fp32 inside a tile, tiles added in index order in fp64); bias / alpha column sums
//             by one CTA in a fixed order.
#include "common.cuh"
#include "launch.h"

namespace mhc {

constexpr int kRowsPerCta = 128;
constexpr int kKT = 32;
constexpr int kBwdRowTile = 32;
constexpr int kBwdStrideRows = 56;  // same per-row record as weights.cu: ds[24] d_raw[24] coef ga[3] pad

int phi_row_tiles(int64_t batch) {
  // at most 32 row tiles for the grad_phi partial sums
  int64_t per = (batch + 31) / 32;
  if (per < 256) per = 256;
  return (int)((batch + per - 1) / per);
}
int64_t phi_rows_per_tile(int64_t batch) { return (batch + phi_row_tiles(batch) - 1) / phi_row_tiles(batch); }

// part[row, slice, 0..23] = sum_{k in slice} x[row,k] phi[k,:];  part[row, slice, 24] = sum x^2.
__global__ void __launch_bounds__(kRowsPerCta)
k_dw_project_rows(const float* __restrict__ x, const float* __restrict__ phi, float* __restrict__ part, int64_t batch,
                  int64_t K, int ks) {
  __shared__ float xs[kRowsPerCta][kKT + 1];
  __shared__ float ps[kKT][24];
  pdl_prologue();
  const int tid = threadIdx.x;
  const int64_t row0 = (int64_t)(blockIdx.x / ks) * kRowsPerCta;
  const int slice = (int)(blockIdx.x % ks);
  int64_t per = (K + ks - 1) / ks;
  per = (per + kKT - 1) / kKT * kKT;
  const int64_t k0 = slice * per, k1 = min(k0 + per, K);
  float acc[25];
#pragma unroll
  for (int j = 0; j < 25; ++j) acc[j] = 0.f;
  for (int64_t kt = k0; kt < k1; kt += kKT) {
#pragma unroll 4
    for (int i = 0; i < kKT; ++i) {
      const int idx = i * kRowsPerCta + tid;
      const int r = idx / kKT, kk = idx % kKT;
      const int64_t row = row0 + r, k = kt + kk;
      xs[r][kk] = (row < batch && k < k1) ? __ldg(x + row * K + k) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < (kKT * 24) / kRowsPerCta; ++i) {
      const int idx = i * kRowsPerCta + tid;
      const int kk = idx / 24, j = idx % 24;
      const int64_t k = kt + kk;
      ps[kk][j] = k < k1 ? __ldg(phi + k * 24 + j) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kKT; ++kk) {
      const float xv = xs[tid][kk];
#pragma unroll
      for (int j = 0; j < 24; ++j) acc[j] = fmaf(xv, ps[kk][j], acc[j]);
      acc[24] = fmaf(xv, xv, acc[24]);
    }
    __syncthreads();
  }
  const int64_t row = row0 + tid;
  if (row < batch) {
    float* o = part + (row * ks + slice) * 25;
#pragma unroll
    for (int j = 0; j < 25; ++j) o[j] = acc[j];
  }
}

// grad_x[row,k] = sum_j d_raw[row,j] phi[k,j] + coef[row] x[row,k] for a (32 rows x 256 k) tile.
__global__ void __launch_bounds__(256)
k_dw_bwd_gx_rows(const float* __restrict__ x, const float* __restrict__ phi, const float* __restrict__ buf,
                 float* __restrict__ grad_x, int64_t batch, int64_t K) {
  __shared__ float s_draw[kBwdRowTile][25];
  pdl_prologue();
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r0 = (int64_t)blockIdx.y * kBwdRowTile;
  const int nr = (int)min((int64_t)kBwdRowTile, batch - r0);
  for (int i = threadIdx.x; i < nr * 25; i += blockDim.x) {
    const int rr = i / 25, jj = i % 25;
    s_draw[rr][jj] = __ldg(buf + (r0 + rr) * kBwdStrideRows + 24 + jj);  // d_raw[24] then coef
  }
  __syncthreads();
  if (k >= K) return;
  float p[24];
#pragma unroll
  for (int j = 0; j < 24; ++j) p[j] = __ldg(phi + k * 24 + j);
  for (int rr = 0; rr < nr; ++rr) {
    const float xv = __ldg(x + (r0 + rr) * K + k);
    float gx = s_draw[rr][24] * xv;
#pragma unroll
    for (int j = 0; j < 24; ++j) gx = fmaf(s_draw[rr][j], p[j], gx);
    grad_x[(r0 + rr) * K + k] = gx;
  }
}

// phi_part[tile, k, j] = sum over the tile's rows of x[row,k] d_raw[row,j]  (rows in index order, fp32).
__global__ void __launch_bounds__(256)
k_dw_bwd_phi_rows(const float* __restrict__ x, const float* __restrict__ buf, float* __restrict__ phi_part,
                  int64_t batch, int64_t K, int64_t rows_per_tile) {
  __shared__ float s_draw[kBwdRowTile][24];
  pdl_prologue();
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t t0 = (int64_t)blockIdx.y * rows_per_tile, t1 = min(t0 + rows_per_tile, batch);
  float acc[24];
#pragma unroll
  for (int j = 0; j < 24; ++j) acc[j] = 0.f;
  for (int64_t r0 = t0; r0 < t1; r0 += kBwdRowTile) {
    const int nr = (int)min((int64_t)kBwdRowTile, t1 - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < nr * 24; i += blockDim.x) {
      const int rr = i / 24, jj = i % 24;
      s_draw[rr][jj] = __ldg(buf + (r0 + rr) * kBwdStrideRows + 24 + jj);
    }
    __syncthreads();
    if (k < K) {
      for (int rr = 0; rr < nr; ++rr) {
        const float xv = __ldg(x + (r0 + rr) * K + k);
#pragma unroll
        for (int j = 0; j < 24; ++j) acc[j] = fmaf(xv, s_draw[rr][j], acc[j]);
      }
    }
  }
  if (k < K) {
    float* o = phi_part + ((int64_t)blockIdx.y * K + k) * 24;
#pragma unroll
    for (int j = 0; j < 24; ++j) o[j] = acc[j];
  }
}

// grad_phi[k,j] (+)= sum_tile phi_part[tile,k,j], tiles in index order, fp64.
__global__ void __launch_bounds__(256)
k_dw_bwd_phi_finish(const float* __restrict__ phi_part, float* __restrict__ grad_phi, int64_t n, int tiles,
                    int accumulate) {
  pdl_prologue();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  double a = 0.0;
  for (int t = 0; t < tiles; ++t) a += (double)__ldg(phi_part + (int64_t)t * n + i);
  grad_phi[i] = accumulate ? grad_phi[i] + (float)a : (float)a;
}

// grad_bias[j] = sum_rows ds[row,j];  grad_alpha[g] = sum_rows ga[row,g].  One CTA: thread t adds rows
// t, t+256, ... in fp64, warps are tree-added by shuffles and joined in index order.
__global__ void __launch_bounds__(256)
k_dw_bwd_param_sums(const float* __restrict__ buf, float* __restrict__ grad_bias, float* __restrict__ grad_alpha,
                    int64_t batch, int accumulate) {
  __shared__ double sm[8][27];
  pdl_prologue();
  double a[27];
#pragma unroll
  for (int j = 0; j < 27; ++j) a[j] = 0.0;
  for (int64_t r = threadIdx.x; r < batch; r += 256) {
    const float* q = buf + r * kBwdStrideRows;
#pragma unroll
    for (int j = 0; j < 27; ++j) a[j] += (double)__ldg(q + (j < 24 ? j : 49 + (j - 24)));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < 27; ++j) {
    const double t = warp_sum_f64(a[j]);
    if (lane == 0) sm[warp][j] = t;
  }
  __syncthreads();
  const int j = threadIdx.x;
  if (j < 27) {
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sm[w][j];
    float* dst = j < 24 ? grad_bias + j : grad_alpha + (j - 24);
    *dst = accumulate ? *dst + (float)t : (float)t;
  }
}

// ------------------------------------------------------------------------------ host side
int project_rows_launch(const float* x, const float* phi, float* part, int64_t batch, int64_t K, int ks_max,
                        cudaStream_t st, int* ks_used) {
  const int64_t row_ctas = (batch + kRowsPerCta - 1) / kRowsPerCta;
  int64_t ks = (2 * 148 + row_ctas - 1) / row_ctas;   // enough CTAs to fill the GPU twice
  if (ks > ks_max) ks = ks_max;
  if (ks > (K + kKT - 1) / kKT) ks = (K + kKT - 1) / kKT;
  if (ks < 1) ks = 1;
  if (row_ctas * ks > kMaxGridItems) return fail(MHC_ERR_BAD_SHAPE, "dynamic_weights_fwd: batch too large");
  {
    ProfScope ps("k_dw_project_rows", st);
    launch_k(k_dw_project_rows, (unsigned)(row_ctas * ks), kRowsPerCta, 0, st, x, phi, part, batch, K, (int)ks);
  }
  *ks_used = (int)ks;
  return check_launch("dynamic_weights_fwd(project rows)");
}

int bwd_rows_launch(const float* x, const float* phi, const float* buf, float* phi_part, float* grad_x, float* grad_phi,
                    float* grad_bias, float* grad_alpha, int64_t batch, int64_t K, int accumulate, cudaStream_t st) {
  const unsigned kblocks = (unsigned)((K + 255) / 256);
  const int64_t row_tiles = (batch + kBwdRowTile - 1) / kBwdRowTile;
  if (row_tiles > 65535) return fail(MHC_ERR_BAD_SHAPE, "dynamic_weights_bwd: more than 2097120 rows");
  {
    ProfScope ps("k_dw_bwd_gx_rows", st);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kblocks, (unsigned)row_tiles);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    (void)cudaLaunchKernelEx(&cfg, k_dw_bwd_gx_rows, x, phi, buf, grad_x, batch, K);
  }
  if (int e = check_launch("dynamic_weights_bwd(grad_x rows)")) return e;
  const int tiles = phi_row_tiles(batch);
  {
    ProfScope ps("k_dw_bwd_phi_rows", st);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kblocks, (unsigned)tiles);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    (void)cudaLaunchKernelEx(&cfg, k_dw_bwd_phi_rows, x, buf, phi_part, batch, K, phi_rows_per_tile(batch));
  }
  if (int e = check_launch("dynamic_weights_bwd(grad_phi rows)")) return e;
  const int64_t n = K * 24;
  {
    ProfScope ps("k_dw_bwd_phi_finish", st);
    launch_k(k_dw_bwd_phi_finish, (unsigned)((n + 255) / 256), 256, 0, st, (const float*)phi_part, grad_phi, n, tiles,
             accumulate);
  }
  if (int e = check_launch("dynamic_weights_bwd(grad_phi finish)")) return e;
  {
    ProfScope ps("k_dw_bwd_param_sums", st);
    launch_k(k_dw_bwd_param_sums, 1u, 256, 0, st, buf, grad_bias, grad_alpha, batch, accumulate);
  }
  return check_launch("dynamic_weights_bwd(param sums)");
}

}  // namespace mhc

// Dynamic weights for MANY rows (per-token use: x [B*S, 4D]).  The few-rows kernels in weights.cu
// give every row its own CTAs, which re-reads phi once per row; from kManyRows rows on, these
// kernels tile over rows instead so that phi (forward) and x (backward) are read once per tile:
//   forward : one thread per row, 128 rows per CTA, x and phi staged through shared memory in
//             32-wide K tiles; same [row, slice, 25] partial layout, so k_dw_finish is shared;
//             (the register-tiled kernel below replaces it when K % 4 == 0 and the pointers are aligned);
//   backward: one pass over x per (256 k) x (row tile) block gives grad_x and the grad_phi partial sums
//             of the tile (fp32 inside a tile, tiles added in index order in fp64); bias / alpha column
//             sums by up to 64 CTAs and one joining warp, in a fixed order.
#include "common.cuh"
#include "launch.h"

namespace mhc {

constexpr int kRowsPerCta = 128;
constexpr int kKT = 32;
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

// ---------------------------------------------------------------------------------------
// Register-tiled projection for K % 4 == 0 and 16-byte aligned x / phi.
// CTA = 128 rows x one K slice, 128 threads; thread (rg, cg) owns rows rg, rg+32, rg+64, rg+96 and
// columns 6cg .. 6cg+5, i.e. 24 accumulators fed by 4 + 6 shared-memory float4 loads per 4 k:
// 96 FMAs per 10 loads, so the FMA pipe is the limit, not shared memory.  Tiles of 32 k are
// double-buffered with cp.async (x as 16-byte copies, phi transposed to [col][k] by 4-byte copies);
// rows past the batch and k past the slice are zero-filled by the copy.  The row stride of 36
// floats keeps float4 alignment and makes both load patterns bank-conflict free.
// sum(x^2) is taken by the thread that copied the values (8 float4 per tile, fixed rows), then
// added across the 8 lanes that share a row.
constexpr int kPR = 128, kPK = 32, kPS = kPK + 4;

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
  const int n = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(kPR)
k_dw_project_rows_v4(const float* __restrict__ x, const float* __restrict__ phi, float* __restrict__ part,
                     int64_t batch, int64_t K, int ks) {
  __shared__ __align__(16) float xs[2][kPR][kPS];
  __shared__ __align__(16) float ps[2][24][kPS];
  pdl_prologue();
  const int tid = threadIdx.x;
  const int cg = tid & 3, rg = tid >> 2;
  const int64_t row0 = (int64_t)(blockIdx.x / ks) * kPR;
  const int slice = (int)(blockIdx.x % ks);
  int64_t per = (K + ks - 1) / ks;
  per = (per + kPK - 1) / kPK * kPK;
  const int64_t k0 = slice * per, k1 = min(k0 + per, K);
  const int ntile = k1 > k0 ? (int)((k1 - k0 + kPK - 1) / kPK) : 0;

  // copy assignments: 8 float4 of x (rows lr + 16 i, k offset 4 lq) and up to 2 float4-worth of phi
  const int lr = tid >> 3, lq = tid & 7;
  auto issue = [&](int t, int b) {
    const int64_t kt = k0 + (int64_t)t * kPK;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = lr + 16 * i;
      const int64_t row = row0 + r, k = kt + 4 * lq;
      const bool ok = row < batch && k < k1;
      cp_async16(&xs[b][r][4 * lq], x + (ok ? row * K + k : 0), ok);
    }
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      const int f = i * kPR + tid;            // 0 .. 767 : element of the [32 k][24] tile
      const int kk = f / 24, j = f % 24;
      const bool ok = kt + kk < k1;
      cp_async4(&ps[b][j][kk], phi + (ok ? (kt + kk) * 24 + j : 0), ok);
    }
    cp_async_commit();
  };

  float acc[4][6];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 6; ++c) acc[i][c] = 0.f;
  float sq[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sq[i] = 0.f;

  if (ntile > 0) issue(0, 0);
  for (int t = 0; t < ntile; ++t) {
    const int b = t & 1;
    if (t + 1 < ntile) { issue(t + 1, b ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
#pragma unroll
    for (int i = 0; i < 8; ++i) {   // this thread's own copies are visible to it after the wait
      const float4 v = *reinterpret_cast<const float4*>(&xs[b][lr + 16 * i][4 * lq]);
      sq[i] = fmaf(v.x, v.x, sq[i]); sq[i] = fmaf(v.y, v.y, sq[i]);
      sq[i] = fmaf(v.z, v.z, sq[i]); sq[i] = fmaf(v.w, v.w, sq[i]);
    }
    __syncthreads();
#pragma unroll
    for (int k4 = 0; k4 < kPK / 4; ++k4) {
      float4 xv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = *reinterpret_cast<const float4*>(&xs[b][rg + 32 * i][4 * k4]);
#pragma unroll
      for (int c = 0; c < 6; ++c) {
        const float4 pv = *reinterpret_cast<const float4*>(&ps[b][6 * cg + c][4 * k4]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float a = acc[i][c];
          a = fmaf(xv[i].x, pv.x, a); a = fmaf(xv[i].y, pv.y, a);
          a = fmaf(xv[i].z, pv.z, a); a = fmaf(xv[i].w, pv.w, a);
          acc[i][c] = a;
        }
      }
    }
    __syncthreads();   // the other buffer is refilled at the top of the next iteration
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t row = row0 + rg + 32 * i;
    if (row < batch) {
      float* o = part + (row * ks + slice) * 25 + 6 * cg;
#pragma unroll
      for (int c = 0; c < 6; ++c) o[c] = acc[i][c];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float v = sq[i];
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    const int64_t row = row0 + lr + 16 * i;
    if (lq == 0 && row < batch) part[(row * ks + slice) * 25 + 24] = v;
  }
}

// Backward over x in one pass: for a (256 k) x (row tile) block,
//   grad_x[row,k]       = coef[row] x[row,k] + sum_j d_raw[row,j] phi[k,j]
//   phi_part[tile,k,j]  = sum over the tile's rows of x[row,k] d_raw[row,j]   (rows in index order, fp32)
// One thread per k keeps phi[k,:] and the 24 partial sums in registers; the per-row records
// (d_raw[24], coef) are staged 64 rows at a time through shared memory and read as broadcast float4s;
// x is read once, four rows ahead of the arithmetic.
constexpr int kBwdStage = 64;

__global__ void __launch_bounds__(256, 2)
k_dw_bwd_x_rows(const float* __restrict__ x, const float* __restrict__ phi, const float* __restrict__ buf,
                float* __restrict__ grad_x, float* __restrict__ phi_part, int64_t batch, int64_t K,
                int64_t rows_per_tile) {
  __shared__ __align__(16) float s_d[kBwdStage][28];   // d_raw[24], coef, 3 unused
  pdl_prologue();
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = k < K;
  const int64_t kc = active ? k : K - 1;
  const int64_t t0 = (int64_t)blockIdx.y * rows_per_tile, t1 = min(t0 + rows_per_tile, batch);
  float p[24], acc[24];
#pragma unroll
  for (int j = 0; j < 24; ++j) { p[j] = __ldg(phi + kc * 24 + j); acc[j] = 0.f; }
  for (int64_t r0 = t0; r0 < t1; r0 += kBwdStage) {
    const int nr = (int)min((int64_t)kBwdStage, t1 - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < kBwdStage * 25; i += blockDim.x) {
      const int rr = i / 25, jj = i % 25;
      s_d[rr][jj] = rr < nr ? __ldg(buf + (r0 + rr) * kBwdStrideRows + 24 + jj) : 0.f;
    }
    __syncthreads();
    const float* xp = x + r0 * K + kc;
    float xn[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) xn[u] = u < nr ? __ldg(xp + (int64_t)u * K) : 0.f;
    for (int rr = 0; rr < nr; rr += 4) {
      float xv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) xv[u] = xn[u];
#pragma unroll
      for (int u = 0; u < 4; ++u) xn[u] = rr + 4 + u < nr ? __ldg(xp + (int64_t)(rr + 4 + u) * K) : 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float4* dq = reinterpret_cast<const float4*>(&s_d[rr + u][0]);
        float d[24];
#pragma unroll
        for (int q = 0; q < 6; ++q) {
          const float4 v = dq[q];
          d[4 * q] = v.x; d[4 * q + 1] = v.y; d[4 * q + 2] = v.z; d[4 * q + 3] = v.w;
        }
        float gx = s_d[rr + u][24] * xv[u];
#pragma unroll
        for (int j = 0; j < 24; ++j) {
          gx = fmaf(d[j], p[j], gx);
          acc[j] = fmaf(xv[u], d[j], acc[j]);     // rows past the tile have d = 0 and x = 0
        }
        if (active && rr + u < nr) grad_x[(r0 + rr + u) * K + k] = gx;
      }
    }
  }
  if (active) {
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

// grad_bias[j] = sum_rows ds[row,j];  grad_alpha[g] = sum_rows ga[row,g], in two steps so that the
// rows are read by many CTAs: each CTA adds a contiguous range of rows in fp64 (thread t takes rows
// t, t+256, ... of the range; warps are tree-added by shuffles and joined in index order) and leaves
// 27 doubles; one warp then adds the CTAs' results in index order.
constexpr int kSumCtas = 64;

__global__ void __launch_bounds__(256)
k_dw_bwd_param_partials(const float* __restrict__ buf, double* __restrict__ psum, int64_t batch, int64_t rows_per_cta) {
  __shared__ double sm[8][27];
  pdl_prologue();
  const int64_t r0 = (int64_t)blockIdx.x * rows_per_cta, r1 = min(r0 + rows_per_cta, batch);
  double a[27];
#pragma unroll
  for (int j = 0; j < 27; ++j) a[j] = 0.0;
  for (int64_t r = r0 + threadIdx.x; r < r1; r += 256) {
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
    psum[(int64_t)blockIdx.x * 27 + j] = t;
  }
}

__global__ void __launch_bounds__(32)
k_dw_bwd_param_finish(const double* __restrict__ psum, int nctas, float* __restrict__ grad_bias,
                      float* __restrict__ grad_alpha, int accumulate) {
  pdl_prologue();
  const int j = threadIdx.x;
  if (j >= 27) return;
  double t = 0.0;
  for (int c = 0; c < nctas; ++c) t += psum[c * 27 + j];
  float* dst = j < 24 ? grad_bias + j : grad_alpha + (j - 24);
  *dst = accumulate ? *dst + (float)t : (float)t;
}

// ------------------------------------------------------------------------------ host side
int64_t rows_bwd_extra_floats(int64_t batch, int64_t K) {
  // grad_phi partial sums per row tile, then the 27 fp64 column sums of each summing CTA (+ alignment slack)
  return (int64_t)phi_row_tiles(batch) * K * 24 + (int64_t)kSumCtas * 27 * 2 + 2;
}

// K slices per 128-row block for the tiled projection: the smallest count whose CTAs fill whole waves of
// the 4 CTAs per SM x 148 SMs that the kernel's registers and shared memory allow to at least 90 %
// (otherwise the best fill).  Depends on the shape only.
static int pick_project_slices(int64_t row_ctas, int64_t kslices_max) {
  const int64_t slots = 4 * 148;
  int best = 1;
  double best_eff = 0.0;
  const int64_t top = kslices_max < 24 ? kslices_max : 24;
  for (int64_t ks = 1; ks <= top; ++ks) {
    const int64_t ctas = row_ctas * ks;
    const int64_t waves = (ctas + slots - 1) / slots;
    const double eff = (double)ctas / (double)(waves * slots);
    if (eff >= 0.9) return (int)ks;
    if (eff > best_eff) { best_eff = eff; best = (int)ks; }
  }
  return best;
}

int project_rows_launch(const float* x, const float* phi, float* part, int64_t batch, int64_t K, int ks_max,
                        cudaStream_t st, int* ks_used) {
  const bool tiled = (K % 4 == 0) && is_aligned16(x) && is_aligned16(phi);
  const int rows_per_cta = tiled ? kPR : kRowsPerCta;
  const int ktile = tiled ? kPK : kKT;
  const int64_t row_ctas = (batch + rows_per_cta - 1) / rows_per_cta;
  int64_t kmax = (K + ktile - 1) / ktile;
  if (kmax > ks_max) kmax = ks_max;
  if (kmax < 1) kmax = 1;
  int64_t ks;
  if (tiled) {
    ks = pick_project_slices(row_ctas, kmax);
  } else {
    ks = (2 * 148 + row_ctas - 1) / row_ctas;   // enough CTAs to fill the GPU twice
    if (ks > kmax) ks = kmax;
  }
  if (row_ctas * ks > kMaxGridItems) return fail(MHC_ERR_BAD_SHAPE, "dynamic_weights_fwd: batch too large");
  if (tiled) {
    ProfScope ps("k_dw_project_rows_v4", st);
    launch_k(k_dw_project_rows_v4, (unsigned)(row_ctas * ks), kPR, 0, st, x, phi, part, batch, K, (int)ks);
  } else {
    ProfScope ps("k_dw_project_rows", st);
    launch_k(k_dw_project_rows, (unsigned)(row_ctas * ks), kRowsPerCta, 0, st, x, phi, part, batch, K, (int)ks);
  }
  *ks_used = (int)ks;
  return check_launch("dynamic_weights_fwd(project rows)");
}

int bwd_rows_launch(const float* x, const float* phi, const float* buf, float* phi_part, float* grad_x, float* grad_phi,
                    float* grad_bias, float* grad_alpha, int64_t batch, int64_t K, int accumulate, cudaStream_t st) {
  const unsigned kblocks = (unsigned)((K + 255) / 256);
  const int tiles = phi_row_tiles(batch);
  {
    ProfScope ps("k_dw_bwd_x_rows", st);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kblocks, (unsigned)tiles);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    (void)cudaLaunchKernelEx(&cfg, k_dw_bwd_x_rows, x, phi, buf, grad_x, phi_part, batch, K, phi_rows_per_tile(batch));
  }
  if (int e = check_launch("dynamic_weights_bwd(x rows)")) return e;
  const int64_t n = K * 24;
  {
    ProfScope ps("k_dw_bwd_phi_finish", st);
    launch_k(k_dw_bwd_phi_finish, (unsigned)((n + 255) / 256), 256, 0, st, (const float*)phi_part, grad_phi, n, tiles,
             accumulate);
  }
  if (int e = check_launch("dynamic_weights_bwd(grad_phi finish)")) return e;
  double* psum = reinterpret_cast<double*>((reinterpret_cast<uintptr_t>(phi_part + (int64_t)tiles * n) + 7) & ~(uintptr_t)7);
  int64_t nctas = (batch + 255) / 256;
  if (nctas > kSumCtas) nctas = kSumCtas;
  const int64_t rows_per_cta = (batch + nctas - 1) / nctas;
  {
    ProfScope ps("k_dw_bwd_param_partials", st);
    launch_k(k_dw_bwd_param_partials, (unsigned)nctas, 256, 0, st, buf, psum, batch, rows_per_cta);
  }
  if (int e = check_launch("dynamic_weights_bwd(param partials)")) return e;
  {
    ProfScope ps("k_dw_bwd_param_finish", st);
    launch_k(k_dw_bwd_param_finish, 1u, 32, 0, st, (const double*)psum, (int)nctas, grad_bias, grad_alpha, accumulate);
  }
  return check_launch("dynamic_weights_bwd(param finish)");
}

}  // namespace mhc

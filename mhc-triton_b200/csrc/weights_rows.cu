// Dynamic weights for MANY rows (per-token use: x [B*S, 4D]).  The few-rows kernels in weights.cu
// give every row its own CTAs, which re-reads phi once per row; from kManyRows rows on, these
// kernels tile over rows instead so that phi (forward) and x (backward) are read once per tile:
//   forward : 128 rows x one K slice per CTA, x and phi staged through shared memory; same
//             [row, slice, 25] partial layout as the few-rows kernel, so k_dw_finish is shared;
//   backward: one pass over x per (k block) x (row tile) gives grad_x and the grad_phi partial sums of
//             the tile (tiles added in index order in fp64); bias / alpha column sums by up to 64 CTAs
//             and one joining warp, in a fixed order.
// Both directions run on the tensor cores (mma.sync TF32 with the 3xTF32 split) when K % 4 == 0 and the
// pointers are 16-byte aligned, and as plain fp32 FMA kernels otherwise.
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
// cp.async helpers: a copy with valid = false writes zeros and reads nothing.
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

// ---------------------------------------------------------------------------------------
// Tensor-core projection (K % 4 == 0, 16-byte aligned x / phi): mma.sync m16n8k8 TF32 with the
// 3xTF32 split (x = hi + lo, both TF32; hi*hi + hi*lo + lo*hi, fp32 accumulate), which keeps fp32-level
// accuracy.  CTA = 128 rows x one K slice, 4 warps; warp w owns rows 32w .. 32w+31 (two 16-row MMA
// tiles) and all 24 columns (three 8-column tiles).  Tiles of 32 k are double-buffered with 16-byte
// cp.async: x as [row][k] with a stride of 36 floats, phi as [k][col] with a stride of 40 floats, which
// makes the A-fragment loads (bank 4g + t) and the B-fragment loads (bank 8t + g) conflict free.
// sum(x^2) as in the FMA kernel: by the copying thread, then across the 8 lanes that share a row.
constexpr int kMR = 128, kMK = 32, kMXS = 36, kMPS = 40;

// v = hi + lo with hi and lo TF32 values (10 mantissa bits), both rounded to nearest with ties away from
// zero - the rounding of cvt.rna.tf32.f32, done with integer adds and masks, which issue at full rate
// (the conversion instruction goes through a narrower pipe; this form measured 6-10 % faster).
__device__ __forceinline__ void split_tf32(float v, uint32_t& hi, uint32_t& lo) {
  hi = (__float_as_uint(v) + 0x1000u) & 0xffffe000u;
  const float rest = v - __uint_as_float(hi);      // exact
  lo = (__float_as_uint(rest) + 0x1000u) & 0xffffe000u;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// d = a * b (no accumulator input).
__device__ __forceinline__ void mma_tf32_first(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "f"(0.f));
}
// c += a * b with the 3xTF32 terms (small ones first).  The tensor core adds into its accumulator with
// truncation, which over hundreds of steps grows into a bias of several fp32 ulps; so the three products
// of one 8-deep step are summed inside the tensor core starting from zero, and the running sum is kept
// with an ordinary round-to-nearest fp32 add.
__device__ __forceinline__ void mma_3xtf32_add(float (&c)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                               const uint32_t (&bh)[2], const uint32_t (&bl)[2]) {
  float d[4];
  mma_tf32_first(d, al, bh);
  mma_tf32(d, ah, bl);
  mma_tf32(d, ah, bh);
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] += d[i];
}

__global__ void __launch_bounds__(128, 4)
k_dw_project_rows_mma(const float* __restrict__ x, const float* __restrict__ phi, float* __restrict__ part,
                      int64_t batch, int64_t K, int ks) {
  __shared__ __align__(16) float xs[2][kMR][kMXS];
  __shared__ __align__(16) float ps[2][kMK][kMPS];
  pdl_prologue();
  const int tid = threadIdx.x;
  const int w = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int64_t row0 = (int64_t)(blockIdx.x / ks) * kMR;
  const int slice = (int)(blockIdx.x % ks);
  int64_t per = (K + ks - 1) / ks;
  per = (per + kMK - 1) / kMK * kMK;
  const int64_t k0 = slice * per, k1 = min(k0 + per, K);
  const int ntile = k1 > k0 ? (int)((k1 - k0 + kMK - 1) / kMK) : 0;

  const int lr = tid >> 3, lq = tid & 7;       // x copies: rows lr + 16 i, k offset 4 lq
  const float* xsrc = x + (row0 + lr) * K + 4 * lq;
  const int rows_left = (int)min((int64_t)kMR, batch - row0) - lr;   // row lr + 16 i exists iff 16 i < rows_left
  auto issue = [&](int tt, int b) {
    const int64_t kt = k0 + (int64_t)tt * kMK;
    const bool kok = kt + 4 * lq < k1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool ok = kok && 16 * i < rows_left;
      cp_async16(&xs[b][lr + 16 * i][4 * lq], ok ? xsrc + (int64_t)(16 * i) * K + kt : x, ok);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int f = i * 128 + tid;              // 0 .. 191 : float4 of the [32 k][24] tile
      if (f < kMK * 6) {
        const int kk = f / 6, q = f % 6;
        const bool ok = kt + kk < k1;
        cp_async16(&ps[b][kk][4 * q], ok ? phi + (kt + kk) * 24 + 4 * q : phi, ok);
      }
    }
    cp_async_commit();
  };

  float acc[2][3][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < 3; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;
  float sq[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sq[i] = 0.f;

  if (ntile > 0) issue(0, 0);
  for (int tt = 0; tt < ntile; ++tt) {
    const int b = tt & 1;
    if (tt + 1 < ntile) { issue(tt + 1, b ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
#pragma unroll
    for (int i = 0; i < 8; ++i) {   // this thread's own copies are visible to it after the wait
      const float4 v = *reinterpret_cast<const float4*>(&xs[b][lr + 16 * i][4 * lq]);
      sq[i] = fmaf(v.x, v.x, sq[i]); sq[i] = fmaf(v.y, v.y, sq[i]);
      sq[i] = fmaf(v.z, v.z, sq[i]); sq[i] = fmaf(v.w, v.w, sq[i]);
    }
    __syncthreads();
#pragma unroll
    for (int k8 = 0; k8 < kMK / 8; ++k8) {
      uint32_t bh[3][2], bl[3][2];
#pragma unroll
      for (int n = 0; n < 3; ++n)
#pragma unroll
        for (int h = 0; h < 2; ++h) split_tf32(ps[b][8 * k8 + t + 4 * h][8 * n + g], bh[n][h], bl[n][h]);
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const int r = 32 * w + 16 * m + g;
        uint32_t ah[4], al[4];
        split_tf32(xs[b][r][8 * k8 + t], ah[0], al[0]);
        split_tf32(xs[b][r + 8][8 * k8 + t], ah[1], al[1]);
        split_tf32(xs[b][r][8 * k8 + t + 4], ah[2], al[2]);
        split_tf32(xs[b][r + 8][8 * k8 + t + 4], ah[3], al[3]);
#pragma unroll
        for (int n = 0; n < 3; ++n) mma_3xtf32_add(acc[m][n], ah, al, bh[n], bl[n]);
      }
    }
    __syncthreads();   // the other buffer is refilled at the top of the next iteration
  }

#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t row = row0 + 32 * w + 16 * m + g + 8 * h;
      if (row < batch) {
        float* o = part + (row * ks + slice) * 25 + 2 * t;
#pragma unroll
        for (int n = 0; n < 3; ++n) { o[8 * n] = acc[m][n][2 * h]; o[8 * n + 1] = acc[m][n][2 * h + 1]; }
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
// (d_raw[24], coef) are staged 64 rows at a time through shared memory and read as broadcast float4s.
// x is read once: every thread copies its own column 32 rows ahead of the arithmetic into a
// shared-memory ring with 4-byte cp.async (8 groups of 4 rows in flight), which keeps enough bytes in
// flight to cover the memory latency without spending registers; a thread only ever reads what it
// copied itself, so the ring needs no barrier.
constexpr int kBwdStage = 64, kXG = 8;

__global__ void __launch_bounds__(256, 2)
k_dw_bwd_x_rows(const float* __restrict__ x, const float* __restrict__ phi, const float* __restrict__ buf,
                float* __restrict__ grad_x, float* __restrict__ phi_part, int64_t batch, int64_t K,
                int64_t rows_per_tile) {
  __shared__ __align__(16) float s_d[kBwdStage][28];   // d_raw[24], coef, 3 unused
  __shared__ float xs[kXG][4][256];
  pdl_prologue();
  const int tid = threadIdx.x;
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + tid;
  const bool active = k < K;
  const int64_t kc = active ? k : K - 1;
  const int64_t t0 = (int64_t)blockIdx.y * rows_per_tile, t1 = min(t0 + rows_per_tile, batch);
  const int64_t ng = t1 > t0 ? (t1 - t0 + 3) / 4 : 0;
  auto issue = [&](int64_t g) {     // group g = rows t0 + 4g .. t0 + 4g + 3, zero-filled past the tile
    const int slot = (int)(g % kXG);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t row = t0 + 4 * g + u;
      const bool ok = active && row < t1;
      cp_async4(&xs[slot][u][tid], x + (ok ? row * K + k : 0), ok);
    }
    cp_async_commit();
  };
  float p[24], acc[24];
#pragma unroll
  for (int j = 0; j < 24; ++j) { p[j] = __ldg(phi + kc * 24 + j); acc[j] = 0.f; }
#pragma unroll
  for (int g = 0; g < kXG; ++g) issue(g);
  for (int64_t g = 0; g < ng; ++g) {
    const int sg = (int)(g % (kBwdStage / 4));
    if (sg == 0) {
      const int64_t r0 = t0 + 4 * g;
      const int nr = (int)min((int64_t)kBwdStage, t1 - r0);
      __syncthreads();
      for (int i = tid; i < kBwdStage * 25; i += blockDim.x) {
        const int rr = i / 25, jj = i % 25;
        s_d[rr][jj] = rr < nr ? __ldg(buf + (r0 + rr) * kBwdStrideRows + 24 + jj) : 0.f;
      }
      __syncthreads();
    }
    cp_async_wait<kXG - 1>();       // group g has landed; the 7 younger groups may still be in flight
    const int slot = (int)(g % kXG);
    float xv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) xv[u] = xs[slot][u][tid];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int rr = 4 * sg + u;
      const float4* dq = reinterpret_cast<const float4*>(&s_d[rr][0]);
      float d[24];
#pragma unroll
      for (int q = 0; q < 6; ++q) {
        const float4 v = dq[q];
        d[4 * q] = v.x; d[4 * q + 1] = v.y; d[4 * q + 2] = v.z; d[4 * q + 3] = v.w;
      }
      float gx = s_d[rr][24] * xv[u];
#pragma unroll
      for (int j = 0; j < 24; ++j) {
        gx = fmaf(d[j], p[j], gx);
        acc[j] = fmaf(xv[u], d[j], acc[j]);     // rows past the tile have d = 0 and x = 0
      }
      const int64_t row = t0 + 4 * g + u;
      if (active && row < t1) grad_x[row * K + k] = gx;
    }
    issue(g + kXG);                 // refill the slot just consumed
  }
  cp_async_wait<0>();
  if (active) {
    float* o = phi_part + ((int64_t)blockIdx.y * K + k) * 24;
#pragma unroll
    for (int j = 0; j < 24; ++j) o[j] = acc[j];
  }
}

// ---------------------------------------------------------------------------------------
// Tensor-core backward over x (K % 4 == 0, 16-byte aligned x): the two products of the one-pass
// backward as mma.sync m16n8k8 TF32 with the 3xTF32 split.  CTA = 64 k columns x one row tile, 4 warps;
// warp w owns k columns 16w .. 16w+15 (the M side of both products):
//   phi_part[k, j]  += sum_row x[row, k] d_raw[row, j]      A = x^T (from shared memory),  B = d_raw
//   grad_x[row, k]   = coef[row] x[row, k] + sum_j phi[k, j] d_raw[row, j]
//                                                             A = phi (registers, loaded once), B = d_raw^T
// Rows are walked 32 at a time.  x stages ([32 rows][64 k], stride 72 floats) are copied with 16-byte
// cp.async two stages ahead of the arithmetic; the per-row records are read one stage ahead into
// registers, split into TF32 hi / lo once, and kept as [row][j ^ 4*(row/4 & 1)] with a stride of 40
// floats, a layout that serves both B-fragment patterns without bank conflicts.
constexpr int kTK = 64, kTR = 32, kTXS = kTK + 8, kTDS = 40;

__global__ void __launch_bounds__(128, 4)
k_dw_bwd_x_rows_mma(const float* __restrict__ x, const float* __restrict__ phi, const float* __restrict__ buf,
                    float* __restrict__ grad_x, float* __restrict__ phi_part, int64_t batch, int64_t K,
                    int64_t rows_per_tile) {
  __shared__ __align__(16) float xs[3][kTR][kTXS];
  __shared__ uint32_t dh[2][kTR][kTDS], dl[2][kTR][kTDS];
  __shared__ float s_coef[2][kTR];
  pdl_prologue();
  const int tid = threadIdx.x;
  const int w = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int64_t kc0 = (int64_t)blockIdx.x * kTK;
  const int64_t t0 = (int64_t)blockIdx.y * rows_per_tile, t1 = min(t0 + rows_per_tile, batch);
  const int nst = t1 > t0 ? (int)((t1 - t0 + kTR - 1) / kTR) : 0;

  const int rows = (int)(t1 - t0);          // rows of this tile (rows_per_tile is far below 2^31)

  // x copies: this thread always copies rows cr + 8 i (i < 4) of a stage at k offset 4 cq
  const int cr = tid >> 4, cq = tid & 15;
  const bool ck_ok = kc0 + 4 * cq < K;
  const float* xsrc = x + (t0 + cr) * K + (ck_ok ? kc0 + 4 * cq : 0);
  auto issue = [&](int st) {       // x rows t0 + 32 st .. + 31 into ring slot st % 3 (zero-filled outside)
    if (st < nst) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = st * kTR + 8 * i + cr;
        const bool ok = ck_ok && r < rows;
        cp_async16(&xs[st % 3][8 * i + cr][4 * cq], ok ? xsrc + (int64_t)(st * kTR + 8 * i) * K : x, ok);
      }
    }
    cp_async_commit();
  };
  // records: this thread always handles row dr of a stage, values 6 dp .. 6 dp + 5 (and coef when dp == 0)
  const int dr = tid >> 2, dp = tid & 3;
  const float* dsrc = buf + (t0 + dr) * kBwdStrideRows + 24 + 6 * dp;
  float dreg[6], dcoef = 0.f;
  auto load_d = [&](int st) {      // records of stage st into registers (zeros outside the tile)
    const bool ok = st < nst && st * kTR + dr < rows;
    const float* q = dsrc + (int64_t)st * (kTR * kBwdStrideRows);
#pragma unroll
    for (int e = 0; e < 6; ++e) dreg[e] = ok ? __ldg(q + e) : 0.f;
    if (dp == 0) dcoef = ok ? __ldg(q + 24) : 0.f;
  };
  auto store_d = [&](int b) {
    const int sw = ((dr >> 2) & 1) << 2;
#pragma unroll
    for (int e = 0; e < 6; ++e) {
      uint32_t hi, lo;
      split_tf32(dreg[e], hi, lo);
      const int c = (6 * dp + e) ^ sw;
      dh[b][dr][c] = hi;
      dl[b][dr][c] = lo;
    }
    if (dp == 0) s_coef[b][dr] = dcoef;
  };

  // phi rows of this warp's 16 k columns as A fragments of the grad_x product (3 steps over j)
  uint32_t ph[3][4], pl[3][4];
#pragma unroll
  for (int q = 0; q < 3; ++q)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t k = kc0 + 16 * w + g + 8 * (i & 1);
      const int j = 8 * q + t + 4 * (i >> 1);
      split_tf32(k < K ? __ldg(phi + k * 24 + j) : 0.f, ph[q][i], pl[q][i]);
    }
  float acc[3][4];
#pragma unroll
  for (int n = 0; n < 3; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
  // grad_x destination of c[0] in stage 0, row tile 0: row 2t, k column 16w + g
  const bool ka_ok = kc0 + 16 * w + g < K, ka8_ok = kc0 + 16 * w + g + 8 < K;
  float* gdst = grad_x + (t0 + 2 * t) * K + kc0 + 16 * w + g;

  issue(0);
  issue(1);
  load_d(0);
  store_d(0);
  for (int st = 0; st < nst; ++st) {
    const int b = st & 1, xb = st % 3;
    load_d(st + 1);
    cp_async_wait<1>();              // stage st has landed (stage st + 1 may still be in flight)
    __syncthreads();                 // everyone is past stage st - 1: its x slot and record buffer are free
    issue(st + 2);

    // phi_part: 4 steps of 8 rows
#pragma unroll
    for (int s8 = 0; s8 < kTR / 8; ++s8) {
      uint32_t ah[4], al[4];
      split_tf32(xs[xb][8 * s8 + t][16 * w + g], ah[0], al[0]);
      split_tf32(xs[xb][8 * s8 + t][16 * w + g + 8], ah[1], al[1]);
      split_tf32(xs[xb][8 * s8 + t + 4][16 * w + g], ah[2], al[2]);
      split_tf32(xs[xb][8 * s8 + t + 4][16 * w + g + 8], ah[3], al[3]);
#pragma unroll
      for (int n = 0; n < 3; ++n) {
        uint32_t bh[2], bl[2];
        bh[0] = dh[b][8 * s8 + t][8 * n + g];            bl[0] = dl[b][8 * s8 + t][8 * n + g];
        bh[1] = dh[b][8 * s8 + t + 4][(8 * n + g) ^ 4];  bl[1] = dl[b][8 * s8 + t + 4][(8 * n + g) ^ 4];
        mma_3xtf32_add(acc[n], ah, al, bh, bl);
      }
    }
    // grad_x: 4 tiles of 8 rows
#pragma unroll
    for (int n = 0; n < kTR / 8; ++n) {
      const int ra = 8 * n + 2 * t;
      const float ca = s_coef[b][ra], cb = s_coef[b][ra + 1];
      float c[4];
      c[0] = ca * xs[xb][ra][16 * w + g];
      c[1] = cb * xs[xb][ra + 1][16 * w + g];
      c[2] = ca * xs[xb][ra][16 * w + g + 8];
      c[3] = cb * xs[xb][ra + 1][16 * w + g + 8];
      const int rb = 8 * n + g, sw = ((rb >> 2) & 1) << 2;
      float d[3][4];               // three independent MMA chains (one per 8 values of j), then fp32 adds
#pragma unroll
      for (int q = 0; q < 3; ++q) {
        uint32_t bh[2], bl[2];
        bh[0] = dh[b][rb][(8 * q + t) ^ sw];      bl[0] = dl[b][rb][(8 * q + t) ^ sw];
        bh[1] = dh[b][rb][(8 * q + t + 4) ^ sw];  bl[1] = dl[b][rb][(8 * q + t + 4) ^ sw];
        mma_tf32_first(d[q], pl[q], bh);
        mma_tf32(d[q], ph[q], bl);
        mma_tf32(d[q], ph[q], bh);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] += (d[0][i] + d[1][i]) + d[2][i];
      const int left = rows - st * kTR - ra;                 // rows of the tile from row ra of this stage on
      float* o = gdst + (int64_t)(st * kTR + 8 * n) * K;
      if (left > 0) {
        if (ka_ok) o[0] = c[0];
        if (ka8_ok) o[8] = c[2];
      }
      if (left > 1) {
        if (ka_ok) o[K] = c[1];
        if (ka8_ok) o[K + 8] = c[3];
      }
    }
    store_d(b ^ 1);                  // records of stage st + 1; visible to the others after the next barrier
  }
  cp_async_wait<0>();
#pragma unroll
  for (int n = 0; n < 3; ++n)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t k = kc0 + 16 * w + g + 8 * h;
      if (k < K) {
        float* o = phi_part + ((int64_t)blockIdx.y * K + k) * 24 + 8 * n + 2 * t;
        o[0] = acc[n][2 * h];
        o[1] = acc[n][2 * h + 1];
      }
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
  // grad_phi partial sums per row tile, then the 27 fp64 column sums of each summing CTA (+ alignment slack),
  // then the tensor-core pass's split copy of phi (+ slack to align it to 256 bytes)
  return (int64_t)phi_row_tiles(batch) * K * 24 + (int64_t)kSumCtas * 27 * 2 + 2 + 64 + rows_tc_bwd_scratch_floats(K);
}

// K slices per 128-row block for the tensor-core projection: the smallest count whose CTAs fill whole
// waves of 4 CTAs per SM x 148 SMs to at least 90 % (otherwise the best fill).  Depends on the shape only.
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
  const bool mma = (K % 4 == 0) && is_aligned16(x) && is_aligned16(phi);
  const int rows_per_cta = mma ? kMR : kRowsPerCta;
  const int ktile = mma ? kMK : kKT;
  const int64_t row_ctas = (batch + rows_per_cta - 1) / rows_per_cta;
  int64_t kmax = (K + ktile - 1) / ktile;
  if (kmax > ks_max) kmax = ks_max;
  if (kmax < 1) kmax = 1;
  int64_t ks;
  if (mma) {
    ks = pick_project_slices(row_ctas, kmax);
  } else {
    ks = (2 * 148 + row_ctas - 1) / row_ctas;   // enough CTAs to fill the GPU twice
    if (ks > kmax) ks = kmax;
  }
  if (row_ctas * ks > kMaxGridItems) return fail(MHC_ERR_BAD_SHAPE, "dynamic_weights_fwd: batch too large");
  if (mma) {
    ProfScope ps("k_dw_project_rows_mma", st);
    launch_k(k_dw_project_rows_mma, (unsigned)(row_ctas * ks), 128, 0, st, x, phi, part, batch, K, (int)ks);
  } else {
    ProfScope ps("k_dw_project_rows", st);
    launch_k(k_dw_project_rows, (unsigned)(row_ctas * ks), kRowsPerCta, 0, st, x, phi, part, batch, K, (int)ks);
  }
  *ks_used = (int)ks;
  return check_launch("dynamic_weights_fwd(project rows)");
}

int bwd_rows_launch(const float* x, const float* phi, const float* buf, float* phi_part, float* grad_x, float* grad_phi,
                    float* grad_bias, float* grad_alpha, int64_t batch, int64_t K, int accumulate, cudaStream_t st) {
  int tiles = phi_row_tiles(batch);
  const int64_t n_part = (int64_t)tiles * K * 24;
  if (rows_tc_usable(x, batch, K) && is_aligned16(grad_x)) {   // tcgen05 pass; its scratch follows the column sums
    float* tc_scratch = reinterpret_cast<float*>(
        (reinterpret_cast<uintptr_t>(phi_part + n_part + (int64_t)kSumCtas * 27 * 2 + 2) + 255) & ~(uintptr_t)255);
    if (int e = rows_bwd_tc_launch(x, phi, buf, phi_part, grad_x, tc_scratch, batch, K, tiles, st, &tiles)) return e;
  } else if (K % 4 == 0 && is_aligned16(x)) {
    ProfScope ps("k_dw_bwd_x_rows_mma", st);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((K + kTK - 1) / kTK), (unsigned)tiles);
    cfg.blockDim = dim3(128);
    cfg.stream = st;
    (void)cudaLaunchKernelEx(&cfg, k_dw_bwd_x_rows_mma, x, phi, buf, grad_x, phi_part, batch, K, phi_rows_per_tile(batch));
  } else {
    const unsigned kblocks = (unsigned)((K + 255) / 256);
    ProfScope ps("k_dw_bwd_x_rows", st);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kblocks, (unsigned)tiles);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    (void)cudaLaunchKernelEx(&cfg, k_dw_bwd_x_rows, x, phi, buf, grad_x, phi_part, batch, K, phi_rows_per_tile(batch));
  }
  if (int e = check_launch("dynamic_weights_bwd(x rows)")) return e;
  const int64_t n = K * 24;   // `tiles` sets of partial sums were written
  {
    ProfScope ps("k_dw_bwd_phi_finish", st);
    launch_k(k_dw_bwd_phi_finish, (unsigned)((n + 255) / 256), 256, 0, st, (const float*)phi_part, grad_phi, n, tiles,
             accumulate);
  }
  if (int e = check_launch("dynamic_weights_bwd(grad_phi finish)")) return e;
  double* psum = reinterpret_cast<double*>((reinterpret_cast<uintptr_t>(phi_part + n_part) + 7) & ~(uintptr_t)7);
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

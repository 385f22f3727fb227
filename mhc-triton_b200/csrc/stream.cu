// HBM-streaming kernels over the hyper-hidden state H[B, S, 4, D]: stream mix, add residual,
// their backwards with deterministic per-CTA partial sums, and the sequence mean-pool.
// Each thread owns one 16-byte pack position along D and walks the tokens of its chunk, so the
// 20 mixing coefficients of the batch element (and, in the apply pass, the pooled-state gradient
// of its columns) stay in registers and every warp access is 512 contiguous bytes.
#include <initializer_list>

#include "common.cuh"
#include "launch.h"

namespace mhc {

// ------------------------------------------------------------------------------- stream mix
template <typename T, int V>
__global__ void __launch_bounds__(256)
k_stream_mix_fwd(const T* __restrict__ H, const float* __restrict__ Hpre, const float* __restrict__ Hres,
                 T* __restrict__ bi, T* __restrict__ Hr, Geo g) {
  const Item it = decode_item(g);
  if (it.col >= g.DV) return;
  float w[4], R[16];
#pragma unroll
  for (int n = 0; n < 4; ++n) w[n] = __ldg(Hpre + it.b * 4 + n);
#pragma unroll
  for (int k = 0; k < 16; ++k) R[k] = __ldg(Hres + it.b * 16 + k);
  const int64_t D = g.D;
  const int64_t tok0 = it.b * g.S + it.s0;
  const T* h = H + tok0 * 4 * D + (int64_t)it.col * V;
  T* o = Hr + tok0 * 4 * D + (int64_t)it.col * V;
  T* q = bi + tok0 * D + (int64_t)it.col * V;
#pragma unroll 2
  for (int64_t s = it.s0; s < it.s1; ++s, h += 4 * D, o += 4 * D, q += D) {
    float x[4][V];
#pragma unroll
    for (int n = 0; n < 4; ++n) PackIO<T, V>::load(h + n * D, x[n]);
    float y[V];
#pragma unroll
    for (int e = 0; e < V; ++e) y[e] = ((w[0] * x[0][e] + w[1] * x[1][e]) + w[2] * x[2][e]) + w[3] * x[3][e];
    PackIO<T, V>::store(q, y);
#pragma unroll
    for (int n = 0; n < 4; ++n) {
#pragma unroll
      for (int e = 0; e < V; ++e)
        y[e] = ((R[4 * n] * x[0][e] + R[4 * n + 1] * x[1][e]) + R[4 * n + 2] * x[2][e]) + R[4 * n + 3] * x[3][e];
      PackIO<T, V>::store(o + n * D, y);
    }
  }
}

// ------------------------------------------------------------------------------ add residual
template <typename T, int V>
__global__ void __launch_bounds__(256)
k_add_residual_fwd(const T* __restrict__ Hr, const T* __restrict__ bo, const float* __restrict__ Hpost,
                   T* __restrict__ Hn, Geo g) {
  const Item it = decode_item(g);
  if (it.col >= g.DV) return;
  float p[4];
#pragma unroll
  for (int n = 0; n < 4; ++n) p[n] = __ldg(Hpost + it.b * 4 + n);
  const int64_t D = g.D;
  const int64_t tok0 = it.b * g.S + it.s0;
  const T* r = Hr + tok0 * 4 * D + (int64_t)it.col * V;
  T* o = Hn + tok0 * 4 * D + (int64_t)it.col * V;
  const T* q = bo + tok0 * D + (int64_t)it.col * V;
#pragma unroll 2
  for (int64_t s = it.s0; s < it.s1; ++s, r += 4 * D, o += 4 * D, q += D) {
    float x[4][V], y[V];
    PackIO<T, V>::load(q, y);
#pragma unroll
    for (int n = 0; n < 4; ++n) PackIO<T, V>::load(r + n * D, x[n]);
#pragma unroll
    for (int n = 0; n < 4; ++n) {
#pragma unroll
      for (int e = 0; e < V; ++e) x[n][e] = x[n][e] + p[n] * y[e];
      PackIO<T, V>::store(o + n * D, x[n]);
    }
  }
}

// d_branch_output[s,d] = sum_n H_post[n] g[s,n,d];  partial dH_post[n] = sum_{s,d} g[s,n,d] bo[s,d].
// part: [B, slots, 4].
template <typename T, int V>
__global__ void __launch_bounds__(256)
k_add_residual_bwd(const T* __restrict__ G, const T* __restrict__ bo, const float* __restrict__ Hpost,
                   T* __restrict__ dbo, float* __restrict__ part, Geo g) {
  __shared__ float red[32 * 4];
  const Item it = decode_item(g);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (it.col < g.DV) {
    float p[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) p[n] = __ldg(Hpost + it.b * 4 + n);
    const int64_t D = g.D;
    const int64_t tok0 = it.b * g.S + it.s0;
    const T* gp = G + tok0 * 4 * D + (int64_t)it.col * V;
    const T* q = bo + tok0 * D + (int64_t)it.col * V;
    T* o = dbo + tok0 * D + (int64_t)it.col * V;
#pragma unroll 2
    for (int64_t s = it.s0; s < it.s1; ++s, gp += 4 * D, q += D, o += D) {
      float x[4][V], y[V], z[V];
      PackIO<T, V>::load(q, y);
#pragma unroll
      for (int n = 0; n < 4; ++n) PackIO<T, V>::load(gp + n * D, x[n]);
#pragma unroll
      for (int e = 0; e < V; ++e) z[e] = ((p[0] * x[0][e] + p[1] * x[1][e]) + p[2] * x[2][e]) + p[3] * x[3][e];
      PackIO<T, V>::store(o, z);
#pragma unroll
      for (int n = 0; n < 4; ++n) {
#pragma unroll
        for (int e = 0; e < V; ++e) acc[n] = fmaf(x[n][e], y[e], acc[n]);
      }
    }
  }
  block_reduce_store<4>(acc, part + (it.b * geo_slots_dev(g) + it.slot) * 4, red);
}

// ---------------------------------------------------------------------- stream mix backward
// MODE 0: dH and partials.  MODE 1: partials only (the apply pass writes dH later).
// part: [B, slots, 20] = dH_pre[4] then dH_res[4][4] row-major.
template <typename T, int V, int MODE>
__global__ void __launch_bounds__(256)
k_stream_mix_bwd(const T* __restrict__ dbi, const T* __restrict__ dHr, const T* __restrict__ H,
                 const float* __restrict__ Hpre, const float* __restrict__ Hres, T* __restrict__ dH,
                 float* __restrict__ part, Geo g) {
  __shared__ float red[32 * 20];
  const Item it = decode_item(g);
  float acc[20];
#pragma unroll
  for (int k = 0; k < 20; ++k) acc[k] = 0.f;
  if (it.col < g.DV) {
    float w[4], R[16];
    if (MODE == 0) {
#pragma unroll
      for (int n = 0; n < 4; ++n) w[n] = __ldg(Hpre + it.b * 4 + n);
#pragma unroll
      for (int k = 0; k < 16; ++k) R[k] = __ldg(Hres + it.b * 16 + k);
    }
    const int64_t D = g.D;
    const int64_t tok0 = it.b * g.S + it.s0;
    const int64_t off4 = tok0 * 4 * D + (int64_t)it.col * V;
    const T* hp = H + off4;
    const T* rp = dHr + off4;
    T* op = dH + off4;
    const T* qp = dbi + tok0 * D + (int64_t)it.col * V;
    for (int64_t s = it.s0; s < it.s1; ++s, hp += 4 * D, rp += 4 * D, op += 4 * D, qp += D) {
      float h[4][V], r[4][V], q[V];
      PackIO<T, V>::load(qp, q);
#pragma unroll
      for (int n = 0; n < 4; ++n) PackIO<T, V>::load(rp + n * D, r[n]);
#pragma unroll
      for (int n = 0; n < 4; ++n) PackIO<T, V>::load(hp + n * D, h[n]);
      if (MODE == 0) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          float y[V];
#pragma unroll
          for (int e = 0; e < V; ++e)
            y[e] = w[m] * q[e] + (((R[m] * r[0][e] + R[4 + m] * r[1][e]) + R[8 + m] * r[2][e]) + R[12 + m] * r[3][e]);
          PackIO<T, V>::store(op + m * D, y);
        }
      }
#pragma unroll
      for (int n = 0; n < 4; ++n) {
#pragma unroll
        for (int e = 0; e < V; ++e) acc[n] = fmaf(q[e], h[n][e], acc[n]);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
#pragma unroll
          for (int e = 0; e < V; ++e) acc[4 + 4 * n + m] = fmaf(r[n][e], h[m][e], acc[4 + 4 * n + m]);
        }
      }
    }
  }
  block_reduce_store<20>(acc, part + (it.b * geo_slots_dev(g) + it.slot) * 20, red);
}

// dH[s,m,d] = H_pre[m] d_bi[s,d] + sum_n H_res[n,m] dH_residual[s,n,d] + inv_S * gx[m*D + d].
template <typename T, int V>
__global__ void __launch_bounds__(256)
k_stream_mix_bwd_apply(const T* __restrict__ dbi, const T* __restrict__ dHr, const float* __restrict__ Hpre,
                       const float* __restrict__ Hres, const float* __restrict__ gx, float inv_S,
                       T* __restrict__ dH, Geo g) {
  const Item it = decode_item(g);
  if (it.col >= g.DV) return;
  float w[4], R[16], c[4][V];
#pragma unroll
  for (int n = 0; n < 4; ++n) w[n] = __ldg(Hpre + it.b * 4 + n);
#pragma unroll
  for (int k = 0; k < 16; ++k) R[k] = __ldg(Hres + it.b * 16 + k);
  const int64_t D = g.D;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
#pragma unroll
    for (int e = 0; e < V; ++e)
      c[m][e] = gx ? inv_S * __ldg(gx + it.b * 4 * D + m * D + (int64_t)it.col * V + e) : 0.f;
  }
  const int64_t tok0 = it.b * g.S + it.s0;
  const int64_t off4 = tok0 * 4 * D + (int64_t)it.col * V;
  const T* rp = dHr + off4;
  T* op = dH + off4;
  const T* qp = dbi + tok0 * D + (int64_t)it.col * V;
#pragma unroll 2
  for (int64_t s = it.s0; s < it.s1; ++s, rp += 4 * D, op += 4 * D, qp += D) {
    float r[4][V], q[V];
    PackIO<T, V>::load(qp, q);
#pragma unroll
    for (int n = 0; n < 4; ++n) PackIO<T, V>::load(rp + n * D, r[n]);
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      float y[V];
#pragma unroll
      for (int e = 0; e < V; ++e)
        y[e] = (w[m] * q[e] + (((R[m] * r[0][e] + R[4 + m] * r[1][e]) + R[8 + m] * r[2][e]) + R[12 + m] * r[3][e])) +
               c[m][e];
      PackIO<T, V>::store(op + m * D, y);
    }
  }
}

// --------------------------------------------------------------------------------- mean-pool
// part[b, chunk, n*D + d] = sum over the chunk's tokens of H[b,s,n,d]  (fp32).
// blockDim.x = cols * sub: thread (col, j) sums tokens j, j+sub, ... of the chunk; the sub-groups
// are then added in index order through shared memory.
template <typename T, int V>
__global__ void __launch_bounds__(256)
k_meanpool_partial(const T* __restrict__ H, float* __restrict__ part, Geo g) {
  extern __shared__ float sm[];  // [4*V][sub][cols]
  const Item it = decode_item(g);
  const int64_t D = g.D;
  float acc[4][V];
#pragma unroll
  for (int n = 0; n < 4; ++n)
#pragma unroll
    for (int e = 0; e < V; ++e) acc[n][e] = 0.f;
  const bool live = it.col < g.DV;
  if (live) {
    const T* h = H + ((it.b * g.S + it.s0 + it.sub) * 4) * D + (int64_t)it.col * V;
    const int64_t step = (int64_t)g.sub * 4 * D;
#pragma unroll 2
    for (int64_t s = it.s0 + it.sub; s < it.s1; s += g.sub, h += step) {
      float x[4][V];
#pragma unroll
      for (int n = 0; n < 4; ++n) PackIO<T, V>::load(h + n * D, x[n]);
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < V; ++e) acc[n][e] += x[n][e];
    }
  }
  const int c = threadIdx.x % g.cols;
  if (g.sub > 1) {
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < V; ++e) sm[((n * V + e) * g.sub + it.sub) * g.cols + c] = acc[n][e];
    __syncthreads();
    if (it.sub == 0) {
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < V; ++e) {
          float t = acc[n][e];
          for (int j = 1; j < g.sub; ++j) t += sm[((n * V + e) * g.sub + j) * g.cols + c];
          acc[n][e] = t;
        }
    }
  }
  if (live && it.sub == 0) {
    float* o = part + (it.b * g.nchunk + it.chunk) * 4 * D + (int64_t)it.col * V;
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < V; ++e) o[n * D + e] = acc[n][e];
  }
}

// x[b,k] = scale * sum_chunk part[b, chunk, k], chunks added in index order in fp64.
__global__ void __launch_bounds__(256)
k_meanpool_finish(const float* __restrict__ part, float* __restrict__ x, int64_t K, int nchunk, double scale,
                  int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int64_t b = i / K, k = i - b * K;
  const float* p = part + b * nchunk * K + k;
  double s = 0.0;
  for (int c = 0; c < nchunk; ++c) s += (double)__ldg(p + (int64_t)c * K);
  x[i] = (float)(s * scale);
}

// out[b, j] = sum_p part[b, p, j] for j < W, slots added in index order in fp64 (four interleaved
// chains, combined in a fixed order).  Columns [0, W0) go to out0, the rest to out1.
__global__ void k_reduce_partials(const float* __restrict__ part, int64_t slots, int W, int W0,
                                  float* __restrict__ out0, float* __restrict__ out1) {
  const int j = threadIdx.x;
  if (j >= W) return;
  const int64_t b = blockIdx.x;
  const float* p = part + b * slots * W + j;
  double a[4] = {0.0, 0.0, 0.0, 0.0};
  int64_t s = 0;
  for (; s + 4 <= slots; s += 4) {
#pragma unroll
    for (int u = 0; u < 4; ++u) a[u] += (double)__ldg(p + (s + u) * W);
  }
  for (int u = 0; s < slots; ++s, ++u) a[u] += (double)__ldg(p + s * W);
  const float v = (float)((a[0] + a[1]) + (a[2] + a[3]));
  if (j < W0) out0[b * W0 + j] = v;
  else out1[b * (W - W0) + (j - W0)] = v;
}

// -------------------------------------------------------------------------------- host side
Geo make_geo(int64_t S, int64_t D, int vec, bool pool) {
  Geo g;
  g.S = S;
  g.D = D;
  g.DV = (int32_t)(D / vec);
  const int max_cols = pool ? 64 : 256;
  int cols = 32;
  while (cols < max_cols && cols < g.DV) cols <<= 1;
  g.cols = cols;
  g.CG = (g.DV + cols - 1) / cols;
  if (pool) {
    g.sub = 256 / cols;
    g.tpc = 128;
  } else {
    g.sub = 1;
    int64_t t = S / 256;
    g.tpc = (int32_t)(t < 4 ? 4 : (t > 32 ? 32 : t));
  }
  g.nchunk = (int32_t)((S + g.tpc - 1) / g.tpc);
  return g;
}

int pick_vec(int dtype, int64_t D, std::initializer_list<const void*> ptrs) {
  const int v = dtype == MHC_F32 ? 4 : 8;
  if (D % v != 0) return 1;
  for (const void* p : ptrs)
    if (p && !is_aligned16(p)) return 1;
  return v;
}

static int check_bsd(const char* what, int64_t B, int64_t S, int64_t D, int dtype) {
  if (dtype != MHC_F32 && dtype != MHC_BF16 && dtype != MHC_F16) return fail(MHC_ERR_BAD_DTYPE, "%s: unknown dtype %d", what, dtype);
  if (B < 0 || S < 0 || D < 0) return fail(MHC_ERR_BAD_SHAPE, "%s: negative size", what);
  if (D > (1LL << 28) || S > (1LL << 31)) return fail(MHC_ERR_BAD_SHAPE, "%s: size out of range", what);
  return MHC_OK;
}

static int check_grid(const char* what, int64_t items) {
  if (items > kMaxGridItems) return fail(MHC_ERR_BAD_SHAPE, "%s: too many work items (%lld)", what, (long long)items);
  return MHC_OK;
}

#define MHC_DISPATCH(dtype, vec, CALL)                                                      \
  do {                                                                                      \
    if ((dtype) == MHC_F32) {                                                               \
      if ((vec) == 1) { using T = float; constexpr int V = 1; CALL; }                       \
      else { using T = float; constexpr int V = 4; CALL; }                                  \
    } else if ((dtype) == MHC_BF16) {                                                       \
      if ((vec) == 1) { using T = __nv_bfloat16; constexpr int V = 1; CALL; }               \
      else { using T = __nv_bfloat16; constexpr int V = 8; CALL; }                          \
    } else {                                                                                \
      if ((vec) == 1) { using T = __half; constexpr int V = 1; CALL; }                      \
      else { using T = __half; constexpr int V = 8; CALL; }                                 \
    }                                                                                       \
  } while (0)

}  // namespace mhc

using namespace mhc;

extern "C" int64_t mhc_scratch_bytes(int op, int64_t B, int64_t S, int64_t D, int dtype) {
  if (B < 0 || S < 0 || D < 0) return -1;
  // Sized for the scalar path (vec = 1), which has the most column groups.
  switch (op) {
    case MHC_OP_ADD_RESIDUAL_BWD: return B * geo_slots(make_geo(S, D, 1, false)) * 4 * (int64_t)sizeof(float);
    case MHC_OP_STREAM_MIX_BWD: return B * geo_slots(make_geo(S, D, 1, false)) * 20 * (int64_t)sizeof(float);
    case MHC_OP_MEANPOOL_FWD: return B * make_geo(S, D, 1, true).nchunk * 4 * D * (int64_t)sizeof(float);
    case MHC_OP_DYNAMIC_WEIGHTS_FWD: return weights_fwd_scratch_bytes(B, 4 * D);
    case MHC_OP_DYNAMIC_WEIGHTS_BWD: return weights_bwd_scratch_bytes(B, 4 * D);
  }
  (void)dtype;
  return -1;
}

extern "C" int mhc_stream_mix_fwd(const void* H, const float* H_pre, const float* H_res, void* branch_input,
                                  void* H_residual, int64_t B, int64_t S, int64_t D, int dtype,
                                  mhc_stream_t stream) {
  if (int e = check_bsd("stream_mix_fwd", B, S, D, dtype)) return e;
  if (B == 0 || S == 0 || D == 0) return MHC_OK;
  if (!H || !H_pre || !H_res || !branch_input || !H_residual) return fail(MHC_ERR_NULL_POINTER, "stream_mix_fwd: null pointer");
  const int vec = pick_vec(dtype, D, {H, branch_input, H_residual});
  const Geo g = make_geo(S, D, vec, false);
  const int64_t items = B * geo_slots(g);
  if (int e = check_grid("stream_mix_fwd", items)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  MHC_DISPATCH(dtype, vec, (k_stream_mix_fwd<T, V><<<(unsigned)items, geo_block(g), 0, st>>>(
                               (const T*)H, H_pre, H_res, (T*)branch_input, (T*)H_residual, g)));
  return check_launch("stream_mix_fwd");
}

extern "C" int mhc_add_residual_fwd(const void* H_residual, const void* branch_output, const float* H_post,
                                    void* H_new, int64_t B, int64_t S, int64_t D, int dtype, mhc_stream_t stream) {
  if (int e = check_bsd("add_residual_fwd", B, S, D, dtype)) return e;
  if (B == 0 || S == 0 || D == 0) return MHC_OK;
  if (!H_residual || !branch_output || !H_post || !H_new) return fail(MHC_ERR_NULL_POINTER, "add_residual_fwd: null pointer");
  const int vec = pick_vec(dtype, D, {H_residual, branch_output, H_new});
  const Geo g = make_geo(S, D, vec, false);
  const int64_t items = B * geo_slots(g);
  if (int e = check_grid("add_residual_fwd", items)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  MHC_DISPATCH(dtype, vec, (k_add_residual_fwd<T, V><<<(unsigned)items, geo_block(g), 0, st>>>(
                               (const T*)H_residual, (const T*)branch_output, H_post, (T*)H_new, g)));
  return check_launch("add_residual_fwd");
}

static int launch_reduce(const float* part, int64_t B, int64_t slots, int W, int W0, float* out0, float* out1,
                         cudaStream_t st, const char* what) {
  k_reduce_partials<<<(unsigned)B, 32, 0, st>>>(part, slots, W, W0, out0, out1);
  return check_launch(what);
}

extern "C" int mhc_add_residual_bwd(const void* dH_new, const void* branch_output, const float* H_post,
                                    void* d_branch_output, float* dH_post, void* scratch, int64_t scratch_bytes,
                                    int64_t B, int64_t S, int64_t D, int dtype, mhc_stream_t stream) {
  if (int e = check_bsd("add_residual_bwd", B, S, D, dtype)) return e;
  if (B == 0) return MHC_OK;
  if (!dH_post) return fail(MHC_ERR_NULL_POINTER, "add_residual_bwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if (S == 0 || D == 0) {
    if (cudaMemsetAsync(dH_post, 0, B * 4 * sizeof(float), st) != cudaSuccess) return check_launch("add_residual_bwd");
    return MHC_OK;
  }
  if (!dH_new || !branch_output || !H_post || !d_branch_output || !scratch)
    return fail(MHC_ERR_NULL_POINTER, "add_residual_bwd: null pointer");
  const int vec = pick_vec(dtype, D, {dH_new, branch_output, d_branch_output});
  const Geo g = make_geo(S, D, vec, false);
  const int64_t slots = geo_slots(g), items = B * slots;
  if (int e = check_grid("add_residual_bwd", items)) return e;
  if (scratch_bytes < items * 4 * (int64_t)sizeof(float))
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "add_residual_bwd: scratch %lld < %lld bytes", (long long)scratch_bytes,
                (long long)(items * 4 * sizeof(float)));
  MHC_DISPATCH(dtype, vec, (k_add_residual_bwd<T, V><<<(unsigned)items, geo_block(g), 0, st>>>(
                               (const T*)dH_new, (const T*)branch_output, H_post, (T*)d_branch_output,
                               (float*)scratch, g)));
  if (int e = check_launch("add_residual_bwd")) return e;
  return launch_reduce((const float*)scratch, B, slots, 4, 4, dH_post, nullptr, st, "add_residual_bwd(reduce)");
}

static int mix_bwd_common(const char* what, int mode, const void* dbi, const void* dHr, const void* H,
                          const float* H_pre, const float* H_res, void* dH, float* dH_pre, float* dH_res,
                          void* scratch, int64_t scratch_bytes, int64_t B, int64_t S, int64_t D, int dtype,
                          cudaStream_t st) {
  if (int e = check_bsd(what, B, S, D, dtype)) return e;
  if (B == 0) return MHC_OK;
  if (!dH_pre || !dH_res) return fail(MHC_ERR_NULL_POINTER, "%s: null pointer", what);
  if (S == 0 || D == 0) {
    if (cudaMemsetAsync(dH_pre, 0, B * 4 * sizeof(float), st) != cudaSuccess ||
        cudaMemsetAsync(dH_res, 0, B * 16 * sizeof(float), st) != cudaSuccess)
      return check_launch(what);
    return MHC_OK;
  }
  if (!dbi || !dHr || !H || !scratch || (mode == 0 && (!dH || !H_pre || !H_res)))
    return fail(MHC_ERR_NULL_POINTER, "%s: null pointer", what);
  const int vec = pick_vec(dtype, D, {dbi, dHr, H, dH});
  const Geo g = make_geo(S, D, vec, false);
  const int64_t slots = geo_slots(g), items = B * slots;
  if (int e = check_grid(what, items)) return e;
  if (scratch_bytes < items * 20 * (int64_t)sizeof(float))
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "%s: scratch %lld < %lld bytes", what, (long long)scratch_bytes,
                (long long)(items * 20 * sizeof(float)));
  if (mode == 0) {
    MHC_DISPATCH(dtype, vec, (k_stream_mix_bwd<T, V, 0><<<(unsigned)items, geo_block(g), 0, st>>>(
                                 (const T*)dbi, (const T*)dHr, (const T*)H, H_pre, H_res, (T*)dH, (float*)scratch, g)));
  } else {
    MHC_DISPATCH(dtype, vec, (k_stream_mix_bwd<T, V, 1><<<(unsigned)items, geo_block(g), 0, st>>>(
                                 (const T*)dbi, (const T*)dHr, (const T*)H, nullptr, nullptr, nullptr,
                                 (float*)scratch, g)));
  }
  if (int e = check_launch(what)) return e;
  return launch_reduce((const float*)scratch, B, slots, 20, 4, dH_pre, dH_res, st, what);
}

extern "C" int mhc_stream_mix_bwd(const void* d_branch_input, const void* dH_residual, const void* H,
                                  const float* H_pre, const float* H_res, void* dH, float* dH_pre, float* dH_res,
                                  void* scratch, int64_t scratch_bytes, int64_t B, int64_t S, int64_t D, int dtype,
                                  mhc_stream_t stream) {
  return mix_bwd_common("stream_mix_bwd", 0, d_branch_input, dH_residual, H, H_pre, H_res, dH, dH_pre, dH_res,
                        scratch, scratch_bytes, B, S, D, dtype, (cudaStream_t)stream);
}

extern "C" int mhc_stream_mix_bwd_reduce(const void* d_branch_input, const void* dH_residual, const void* H,
                                         float* dH_pre, float* dH_res, void* scratch, int64_t scratch_bytes,
                                         int64_t B, int64_t S, int64_t D, int dtype, mhc_stream_t stream) {
  return mix_bwd_common("stream_mix_bwd_reduce", 1, d_branch_input, dH_residual, H, nullptr, nullptr, nullptr,
                        dH_pre, dH_res, scratch, scratch_bytes, B, S, D, dtype, (cudaStream_t)stream);
}

extern "C" int mhc_stream_mix_bwd_apply(const void* d_branch_input, const void* dH_residual, const float* H_pre,
                                        const float* H_res, const float* grad_x, float inv_S, void* dH, int64_t B,
                                        int64_t S, int64_t D, int dtype, mhc_stream_t stream) {
  if (int e = check_bsd("stream_mix_bwd_apply", B, S, D, dtype)) return e;
  if (B == 0 || S == 0 || D == 0) return MHC_OK;
  if (!d_branch_input || !dH_residual || !H_pre || !H_res || !dH)
    return fail(MHC_ERR_NULL_POINTER, "stream_mix_bwd_apply: null pointer");
  const int vec = pick_vec(dtype, D, {d_branch_input, dH_residual, dH});
  const Geo g = make_geo(S, D, vec, false);
  const int64_t items = B * geo_slots(g);
  if (int e = check_grid("stream_mix_bwd_apply", items)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  MHC_DISPATCH(dtype, vec, (k_stream_mix_bwd_apply<T, V><<<(unsigned)items, geo_block(g), 0, st>>>(
                               (const T*)d_branch_input, (const T*)dH_residual, H_pre, H_res, grad_x, inv_S,
                               (T*)dH, g)));
  return check_launch("stream_mix_bwd_apply");
}

extern "C" int mhc_meanpool_fwd(const void* H, float* x, void* scratch, int64_t scratch_bytes, int64_t B, int64_t S,
                                int64_t D, int dtype, mhc_stream_t stream) {
  if (int e = check_bsd("meanpool_fwd", B, S, D, dtype)) return e;
  if (B == 0 || D == 0) return MHC_OK;
  if (S == 0) return fail(MHC_ERR_BAD_SHAPE, "meanpool_fwd: empty sequence");
  if (!H || !x || !scratch) return fail(MHC_ERR_NULL_POINTER, "meanpool_fwd: null pointer");
  const int vec = pick_vec(dtype, D, {H});
  const Geo g = make_geo(S, D, vec, true);
  const int64_t items = B * geo_slots(g);
  if (int e = check_grid("meanpool_fwd", items)) return e;
  const int64_t need = B * g.nchunk * 4 * D * (int64_t)sizeof(float);
  if (scratch_bytes < need)
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "meanpool_fwd: scratch %lld < %lld bytes", (long long)scratch_bytes, (long long)need);
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)4 * vec * geo_block(g) * sizeof(float);
  MHC_DISPATCH(dtype, vec, (k_meanpool_partial<T, V><<<(unsigned)items, geo_block(g), smem, st>>>(
                               (const T*)H, (float*)scratch, g)));
  if (int e = check_launch("meanpool_fwd")) return e;
  const int64_t total = B * 4 * D;
  k_meanpool_finish<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const float*)scratch, x, 4 * D, g.nchunk,
                                                                      1.0 / (double)S, total);
  return check_launch("meanpool_fwd(finish)");
}

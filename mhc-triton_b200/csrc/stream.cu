// HBM-streaming kernels over the hyper-hidden state H[B, S, 4, D]: stream mix, add residual,
// their backwards with deterministic per-CTA partial sums, and the sequence mean-pool.
// Each thread owns one 16-byte pack position along D and walks the tokens of its chunk, so the
// 20 mixing coefficients of the batch element (and, in the apply pass, the pooled-state gradient
// of its columns) stay in registers and every warp access is 512 contiguous bytes.
#include <initializer_list>

#include "common.cuh"
#include "launch.h"

namespace mhc {

// Tuning constants.  The defaults are the best configuration found by sweeps on a B200 with bf16
// H(8, 4096, 4, 4096); `build.py -D NAME=value --out other.so` builds a variant and the environment
// variable MHC_B200_LIB points the Python package at it.
//   *_PIPE  1: prefetch the next token's packs while computing the current one (worth it when few
//              CTAs fit an SM);  0: rely on more resident CTAs instead.
//   *_MINB  minimum resident CTAs per SM asked of the compiler (caps the registers per thread).
//   *_TPC   tokens walked by one CTA.  Short chunks make consecutive CTAs sweep memory almost
//           linearly (faster), long chunks amortise per-CTA state (coefficients, grad_x columns,
//           partial sums).
#ifndef MHC_MIXFWD_PIPE
#define MHC_MIXFWD_PIPE 0
#endif
#ifndef MHC_MIXFWD_MINB
#define MHC_MIXFWD_MINB 4
#endif
#ifndef MHC_ADDFWD_PIPE
#define MHC_ADDFWD_PIPE 1
#endif
#ifndef MHC_ADDFWD_MINB
#define MHC_ADDFWD_MINB 4
#endif
#ifndef MHC_APPLY_PIPE
#define MHC_APPLY_PIPE 0
#endif
#ifndef MHC_APPLY_MINB
#define MHC_APPLY_MINB 3
#endif

// Mean-pool: tokens per CTA (adjusted to fill whole waves, see wave_tpc), packs along D per CTA (the CTA
// has 4 x MHC_POOL_COLS threads, one per stream row and pack), loads in flight per thread, and
// the resident CTAs per SM the chunking is sized for.
#ifndef MHC_POOL_TPC
#define MHC_POOL_TPC 112
#endif
#ifndef MHC_POOL_COLS
#define MHC_POOL_COLS 32
#endif
#ifndef MHC_POOL_DEPTH
#define MHC_POOL_DEPTH 8
#endif
#ifndef MHC_POOL_OCC
#define MHC_POOL_OCC 7
#endif
// Walking direction per kernel (bit set = from the end of the tensor to its start): bit 0 mean-pool,
// 1 stream mix, 2 add residual, 3 add-residual backward, 4 stream-mix backward reduce / full,
// 5 stream-mix backward apply.  Consecutive kernels of a layer step walk in opposite directions so
// that what the previous kernel touched last (still in L2) is what the next one touches first.
#ifndef MHC_REV_MASK
#define MHC_REV_MASK 18
#endif
#ifndef MHC_MAX_COLS
#define MHC_MAX_COLS 256
#endif
// Tokens per CTA, per kernel.
#ifndef MHC_TPC_MIXFWD
#define MHC_TPC_MIXFWD 1
#endif
#ifndef MHC_TPC_ADDFWD
#define MHC_TPC_ADDFWD 1
#endif
#ifndef MHC_TPC_APPLY
#define MHC_TPC_APPLY 4
#endif
#ifndef MHC_TPC_ADDBWD
#define MHC_TPC_ADDBWD 4
#endif
// The reduction pass holds 20 running sums per thread and ends every CTA with a block reduction and a
// ticket: long chunks (one wave of CTAs per sequence at S = 4096, D = 4096) beat short ones by 3 % at
// eight sequences and 9 % at one.
#ifndef MHC_TPC_MIXBWD
#define MHC_TPC_MIXBWD 28
#endif
// Add-residual backward and apply pass on rows that take narrow column groups (several tokens abreast, e.g.
// D = 7168): tokens per thread = this x the constants above.  Every CTA of these two kernels has fixed work
// (a block reduction and a ticket; 32 registers of grad_x columns to load) that short chunks repeat often.
// At full SM clock the chunk length makes no difference at that width (111 / 172 us against 114 / 171 at
// D = 7168, two sequences), but between the GEMMs of an MLP branch, where the power cap holds the SMs near
// 1.4 GHz, 16 tokens per thread take 129 / 188 us against 156 / 202 for 4.  Wide rows (D = 4096, 2048)
// keep the short chunks, which are 1-4 % faster there at full clock.
#ifndef MHC_NARROW_MULT
#define MHC_NARROW_MULT 4
#endif
// Resident CTAs per SM of the add-residual backward (80 registers x 256 threads), for wave_tpc.
#ifndef MHC_ADDBWD_OCC
#define MHC_ADDBWD_OCC 3
#endif


template <typename T, int V>
__device__ __forceinline__ void unpack(const RawPack<T, V>& r, float (&o)[V]) {
#pragma unroll
  for (int e = 0; e < V; ++e) o[e] = raw_get<V>(r, e);
}

// ------------------------------------------------------------------------------- stream mix
template <typename T, int V>
__global__ void __launch_bounds__(MHC_MAX_COLS, MHC_MIXFWD_MINB)
k_stream_mix_fwd(const T* __restrict__ H, const float* __restrict__ Hpre, const float* __restrict__ Hres,
                 T* __restrict__ bi, T* __restrict__ Hr, Geo g) {
  pdl_prologue();
  const Item it = decode_item(g);
  if (it.col >= g.DV) return;
  float w[4], R[16];
#pragma unroll
  for (int n = 0; n < 4; ++n) w[n] = __ldg(Hpre + it.b * 4 + n);
#pragma unroll
  for (int k = 0; k < 16; ++k) R[k] = __ldg(Hres + it.b * 16 + k);
  const int64_t D = g.D, c0 = (int64_t)it.col * V, tok = it.b * g.S;
  using B4 = Bundle<T, V, 4>;
  for_tokens<MHC_MIXFWD_PIPE != 0, B4>(
      it.s0 + it.sub, it.s1, g.sub,
      [&](B4& u, int64_t s) {
        const T* h = H + (tok + s) * 4 * D + c0;
#pragma unroll
        for (int n = 0; n < 4; ++n) u.p[n] = ld_raw<T, V>(h + n * D);
      },
      [&](const B4& u, int64_t s) {
        float x[4][V], y[V];
#pragma unroll
        for (int n = 0; n < 4; ++n) unpack<T, V>(u.p[n], x[n]);
#pragma unroll
        for (int e = 0; e < V; ++e) y[e] = ((w[0] * x[0][e] + w[1] * x[1][e]) + w[2] * x[2][e]) + w[3] * x[3][e];
        PackIO<T, V>::store(bi + (tok + s) * D + c0, y);
        T* o = Hr + (tok + s) * 4 * D + c0;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
          for (int e = 0; e < V; ++e)
            y[e] = ((R[4 * n] * x[0][e] + R[4 * n + 1] * x[1][e]) + R[4 * n + 2] * x[2][e]) + R[4 * n + 3] * x[3][e];
          PackIO<T, V>::store(o + n * D, y);
        }
      });
}

// Pre-mix only: branch_input[s,d] = sum_n H_pre[n] H[s,n,d].  Used when the residual mix is not
// materialised (it is then recomputed from H inside k_add_residual_mix_fwd).
#ifndef MHC_TPC_PREMIX
#define MHC_TPC_PREMIX 2
#endif
template <typename T, int V>
__global__ void __launch_bounds__(MHC_MAX_COLS, 4)
k_stream_premix_fwd(const T* __restrict__ H, const float* __restrict__ Hpre, T* __restrict__ bi, Geo g) {
  pdl_prologue();
  const Item it = decode_item(g);
  if (it.col >= g.DV) return;
  float w[4];
#pragma unroll
  for (int n = 0; n < 4; ++n) w[n] = __ldg(Hpre + it.b * 4 + n);
  const int64_t D = g.D, c0 = (int64_t)it.col * V, tok = it.b * g.S;
  using B4 = Bundle<T, V, 4>;
  for_tokens_pipelined<B4>(
      it.s0 + it.sub, it.s1, g.sub,
      [&](B4& u, int64_t s) {
        const T* h = H + (tok + s) * 4 * D + c0;
#pragma unroll
        for (int n = 0; n < 4; ++n) u.p[n] = ld_raw<T, V>(h + n * D);
      },
      [&](const B4& u, int64_t s) {
        float y[V];
#pragma unroll
        for (int e = 0; e < V; ++e)
          y[e] = ((w[0] * raw_get<V>(u.p[0], e) + w[1] * raw_get<V>(u.p[1], e)) + w[2] * raw_get<V>(u.p[2], e)) +
                 w[3] * raw_get<V>(u.p[3], e);
        PackIO<T, V>::store(bi + (tok + s) * D + c0, y);
      });
}

// ------------------------------------------------------------------------------ add residual
template <typename T, int V>
__global__ void __launch_bounds__(MHC_MAX_COLS, MHC_ADDFWD_MINB)
k_add_residual_fwd(const T* __restrict__ Hr, const T* __restrict__ bo, const float* __restrict__ Hpost,
                   T* __restrict__ Hn, Geo g) {
  pdl_prologue();
  const Item it = decode_item(g);
  if (it.col >= g.DV) return;
  float p[4];
#pragma unroll
  for (int n = 0; n < 4; ++n) p[n] = __ldg(Hpost + it.b * 4 + n);
  const int64_t D = g.D, c0 = (int64_t)it.col * V, tok = it.b * g.S;
  using B5 = Bundle<T, V, 5>;
  for_tokens<MHC_ADDFWD_PIPE != 0, B5>(
      it.s0 + it.sub, it.s1, g.sub,
      [&](B5& u, int64_t s) {
        const T* r = Hr + (tok + s) * 4 * D + c0;
        u.p[4] = ld_raw<T, V>(bo + (tok + s) * D + c0);
#pragma unroll
        for (int n = 0; n < 4; ++n) u.p[n] = ld_raw<T, V>(r + n * D);
      },
      [&](const B5& u, int64_t s) {
        float y[V], x[V];
        unpack<T, V>(u.p[4], y);
        T* o = Hn + (tok + s) * 4 * D + c0;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          unpack<T, V>(u.p[n], x);
#pragma unroll
          for (int e = 0; e < V; ++e) x[e] = x[e] + p[n] * y[e];
          PackIO<T, V>::store(o + n * D, x);
        }
      });
}

// Add residual that also leaves the token sums of its own output for the NEXT layer's mean-pool:
// pool[b, chunk, n*D + d] = sum over the chunk's tokens of H_new[b,s,n,d] (the values as stored,
// i.e. after rounding to T).  Same layout as k_meanpool_partial's output, so the next layer's
// projection kernel consumes it directly and that layer's pass over H for pooling disappears.
#ifndef MHC_TPC_ADDPOOL
#define MHC_TPC_ADDPOOL 64
#endif
#ifndef MHC_ADDPOOL_PIPE
#define MHC_ADDPOOL_PIPE 0
#endif
// Tokens' worth of loads the pooling add-residual kernels keep in a per-thread shared-memory ring (see
// for_tokens_staged; 0: none, loads go straight to registers): stages * 5 packs * 16 bytes per thread.
// Their 32 pooling sums leave too few registers to keep enough loads in flight otherwise.
#ifndef MHC_ADDPOOL_STAGES
#define MHC_ADDPOOL_STAGES 4
#endif
template <typename T, int V>
__global__ void __launch_bounds__(MHC_MAX_COLS, 2)
k_add_residual_pool_fwd(const T* __restrict__ Hr, const T* __restrict__ bo, const float* __restrict__ Hpost,
                        T* __restrict__ Hn, float* __restrict__ pool, Geo g) {
  extern __shared__ __align__(16) float sm[];  // [2*V][sub][cols], used when several tokens are walked abreast
  pdl_prologue();
  const Item it = decode_item(g);
  const int64_t D = g.D, c0 = (int64_t)it.col * V, tok = it.b * g.S;
  float acc[4][V];
#pragma unroll
  for (int n = 0; n < 4; ++n)
#pragma unroll
    for (int e = 0; e < V; ++e) acc[n][e] = 0.f;
  const bool live = it.col < g.DV;
  if (live) {
    float p[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) p[n] = __ldg(Hpost + it.b * 4 + n);
    using B5 = Bundle<T, V, 5>;
    auto load = [&](B5& u, int64_t s) {
      const T* r = Hr + (tok + s) * 4 * D + c0;
      u.p[4] = ld_raw<T, V>(bo + (tok + s) * D + c0);
#pragma unroll
      for (int n = 0; n < 4; ++n) u.p[n] = ld_raw<T, V>(r + n * D);
    };
    auto compute = [&](const B5& u, int64_t s) {
      float y[V], x[V];
      unpack<T, V>(u.p[4], y);
      T* o = Hn + (tok + s) * 4 * D + c0;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        unpack<T, V>(u.p[n], x);
#pragma unroll
        for (int e = 0; e < V; ++e) x[e] = x[e] + p[n] * y[e];
        PackIO<T, V>::store_round(o + n * D, x);   // x now holds what a later read of H_new returns
#pragma unroll
        for (int e = 0; e < V; ++e) acc[n][e] += x[e];
      }
    };
    if constexpr (V > 1 && MHC_ADDPOOL_STAGES > 0) {
      for_tokens_staged<T, V, 5, MHC_ADDPOOL_STAGES>(
          it.s0 + it.sub, it.s1, g.sub, (uint32_t)__cvta_generic_to_shared(sm),
          [&](int64_t s, int n) -> const T* {
            return n == 4 ? bo + (tok + s) * D + c0 : Hr + ((tok + s) * 4 + n) * D + c0;
          },
          compute);
    } else {
      for_tokens<MHC_ADDPOOL_PIPE != 0, B5>(it.s0 + it.sub, it.s1, g.sub, load, compute);
    }
  }
  const int c = threadIdx.x % g.cols;
  if (g.sub > 1) {  // add the sub-groups in index order, two stream rows at a time (halves the shared memory)
    if (V > 1 && MHC_ADDPOOL_STAGES > 0) __syncthreads();   // the sums below reuse the ring's shared memory
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (half) __syncthreads();
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < V; ++e) sm[((n * V + e) * g.sub + it.sub) * g.cols + c] = acc[2 * half + n][e];
      __syncthreads();
      if (it.sub == 0) {
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int e = 0; e < V; ++e) {
            float t = acc[2 * half + n][e];
            for (int j = 1; j < g.sub; ++j) t += sm[((n * V + e) * g.sub + j) * g.cols + c];
            acc[2 * half + n][e] = t;
          }
      }
    }
  }
  if (live && it.sub == 0) {
    float* o = pool + (it.b * g.nchunk + it.chunk) * 4 * D + c0;
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < V; ++e) o[n * D + e] = acc[n][e];
  }
}

// H_new[s,n,d] = (sum_m H_res[n,m] H[s,m,d]) + H_post[n] branch_output[s,d]: the residual mix is
// recomputed from H here instead of being written by the stream-mix kernel and read back (saves
// 8 of the 46 D*e bytes per token of a layer step).  The sum is formed first and the branch term
// added last, the order the two separate kernels use.  POOL: also leave the per-chunk token sums
// of H_new for the next layer (see k_add_residual_pool_fwd).
#ifndef MHC_TPC_ADDMIX
#define MHC_TPC_ADDMIX 1
#endif
#ifndef MHC_ADDMIX_PIPE
#define MHC_ADDMIX_PIPE 0
#endif
#ifndef MHC_ADDMIX_MINB
#define MHC_ADDMIX_MINB 4
#endif
#ifndef MHC_ADDMIXPOOL_PIPE
#define MHC_ADDMIXPOOL_PIPE 0
#endif
#ifndef MHC_ADDMIXPOOL_MINB
#define MHC_ADDMIXPOOL_MINB 2
#endif

template <typename T, int V, bool POOL>
__global__ void __launch_bounds__(MHC_MAX_COLS, POOL ? MHC_ADDMIXPOOL_MINB : MHC_ADDMIX_MINB)
k_add_residual_mix_fwd(const T* __restrict__ H, const float* __restrict__ Hres, const T* __restrict__ bo,
                       const float* __restrict__ Hpost, T* __restrict__ Hn, float* __restrict__ pool, Geo g) {
  extern __shared__ __align__(16) float sm[];  // POOL: [2*V][sub][cols]
  pdl_prologue();
  const Item it = decode_item(g);
  const int64_t D = g.D, c0 = (int64_t)it.col * V, tok = it.b * g.S;
  float acc[POOL ? 4 : 1][V];
  if (POOL) {
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < V; ++e) acc[POOL ? n : 0][e] = 0.f;
  }
  const bool live = it.col < g.DV;
  if (!POOL && !live) return;
  if (live) {
    float p[4], R[16];
#pragma unroll
    for (int n = 0; n < 4; ++n) p[n] = __ldg(Hpost + it.b * 4 + n);
#pragma unroll
    for (int k = 0; k < 16; ++k) R[k] = __ldg(Hres + it.b * 16 + k);
    using B5 = Bundle<T, V, 5>;
    auto load = [&](B5& u, int64_t s) {
      const T* h = H + (tok + s) * 4 * D + c0;
      u.p[4] = ld_raw<T, V>(bo + (tok + s) * D + c0);
#pragma unroll
      for (int n = 0; n < 4; ++n) u.p[n] = ld_raw<T, V>(h + n * D);
    };
    auto compute = [&](const B5& u, int64_t s) {
      float x[4][V], y[V], o[V];
      unpack<T, V>(u.p[4], y);
#pragma unroll
      for (int n = 0; n < 4; ++n) unpack<T, V>(u.p[n], x[n]);
      T* op = Hn + (tok + s) * 4 * D + c0;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
#pragma unroll
        for (int e = 0; e < V; ++e)
          o[e] = (((R[4 * n] * x[0][e] + R[4 * n + 1] * x[1][e]) + R[4 * n + 2] * x[2][e]) + R[4 * n + 3] * x[3][e]) +
                 p[n] * y[e];
        if (POOL) {
          PackIO<T, V>::store_round(op + n * D, o);
#pragma unroll
          for (int e = 0; e < V; ++e) acc[POOL ? n : 0][e] += o[e];
        } else {
          PackIO<T, V>::store(op + n * D, o);
        }
      }
    };
    if constexpr (POOL && V > 1 && MHC_ADDPOOL_STAGES > 0) {
      // the pooling sums take the registers that would hold loads in flight: stage those in shared memory
      for_tokens_staged<T, V, 5, MHC_ADDPOOL_STAGES>(
          it.s0 + it.sub, it.s1, g.sub, (uint32_t)__cvta_generic_to_shared(sm),
          [&](int64_t s, int n) -> const T* {
            return n == 4 ? bo + (tok + s) * D + c0 : H + ((tok + s) * 4 + n) * D + c0;
          },
          compute);
    } else {
      for_tokens<(POOL ? MHC_ADDMIXPOOL_PIPE != 0 : MHC_ADDMIX_PIPE != 0), B5>(it.s0 + it.sub, it.s1, g.sub, load, compute);
    }
  }
  if (POOL) {
    const int c = threadIdx.x % g.cols;
    if (g.sub > 1) {
      if (V > 1 && MHC_ADDPOOL_STAGES > 0) __syncthreads();   // the sums below reuse the ring's shared memory
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (half) __syncthreads();
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int e = 0; e < V; ++e) sm[((n * V + e) * g.sub + it.sub) * g.cols + c] = acc[POOL ? 2 * half + n : 0][e];
        __syncthreads();
        if (it.sub == 0) {
#pragma unroll
          for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < V; ++e) {
              float t = acc[POOL ? 2 * half + n : 0][e];
              for (int j = 1; j < g.sub; ++j) t += sm[((n * V + e) * g.sub + j) * g.cols + c];
              acc[POOL ? 2 * half + n : 0][e] = t;
            }
        }
      }
    }
    if (live && it.sub == 0) {
      float* o = pool + (it.b * g.nchunk + it.chunk) * 4 * D + c0;
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < V; ++e) o[n * D + e] = acc[POOL ? n : 0][e];
    }
  }
}

// Sum the [slots, W] per-CTA partial sums of batch element b (written by the CTAs of THIS kernel) in
// fp64, fixed order, exactly as k_reduce_partials does; columns [0, W0) go to out0, the rest to
// out1.  Called by the one CTA of the batch element that arrived last (cta_arrives_last); `sm` is
// 8 x 20 doubles of shared memory no longer used for anything else.
__device__ __forceinline__ void finish_partials(const float* __restrict__ part, int64_t b, int64_t slots, int W, int W0,
                                                float* __restrict__ out0, float* __restrict__ out1,
                                                double (*sm)[20]) {
  if (W == 20) block_column_sums_fast<20, true>(part + b * slots * W, slots, sm);
  else if (W == 4) block_column_sums_fast<4, true>(part + b * slots * W, slots, sm);
  else block_column_sums_f64<true>(part + b * slots * W, slots, W, sm);
  const int j = threadIdx.x;
  if (j < W) {
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sm[w][j];
    if (j < W0) out0[b * W0 + j] = (float)t;
    else out1[b * (W - W0) + (j - W0)] = (float)t;
  }
}

// d_branch_output[s,d] = sum_n H_post[n] g[s,n,d];  partial dH_post[n] = sum_{s,d} g[s,n,d] bo[s,d].
// part: [B, slots, 4].  With tickets (one zeroed counter per batch element) the CTA of a batch
// element that stores its partial last also adds them all up into dH_post[b].
#ifndef MHC_ADDBWD_MINB
#define MHC_ADDBWD_MINB 3
#endif
#ifndef MHC_ADDBWD_PIPE
#define MHC_ADDBWD_PIPE 1
#endif
template <typename T, int V>
__global__ void __launch_bounds__(MHC_MAX_COLS, MHC_ADDBWD_MINB)
k_add_residual_bwd(const T* __restrict__ G, const T* __restrict__ bo, const float* __restrict__ Hpost,
                   T* __restrict__ dbo, float* __restrict__ part, Geo g, int* tickets, float* __restrict__ dH_post) {
  pdl_prologue();
  __shared__ __align__(8) float red[32 * 20];
  const Item it = decode_item(g);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (it.col < g.DV) {
    float p[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) p[n] = __ldg(Hpost + it.b * 4 + n);
    const int64_t D = g.D, c0 = (int64_t)it.col * V, tok = it.b * g.S;
    using B5 = Bundle<T, V, 5>;
    for_tokens<MHC_ADDBWD_PIPE != 0, B5>(
        it.s0 + it.sub, it.s1, g.sub,
        [&](B5& u, int64_t s) {
          const T* gp = G + (tok + s) * 4 * D + c0;
          u.p[4] = ld_raw<T, V>(bo + (tok + s) * D + c0);
#pragma unroll
          for (int n = 0; n < 4; ++n) u.p[n] = ld_raw<T, V>(gp + n * D);
        },
        [&](const B5& u, int64_t s) {
          float y[V], z[V], x[V];
          unpack<T, V>(u.p[4], y);
#pragma unroll
          for (int e = 0; e < V; ++e) z[e] = 0.f;
#pragma unroll
          for (int n = 0; n < 4; ++n) {
            unpack<T, V>(u.p[n], x);
#pragma unroll
            for (int e = 0; e < V; ++e) {
              z[e] = fmaf(p[n], x[e], z[e]);
              acc[n] = fmaf(x[e], y[e], acc[n]);
            }
          }
          PackIO<T, V>::store(dbo + (tok + s) * D + c0, z);
        });
  }
  block_reduce_store<4>(acc, part + (it.b * geo_slots_dev(g) + it.slot) * 4, red);
  if (!tickets) return;
  const int64_t slots = geo_slots_dev(g);
  if (cta_arrives_last(tickets + it.b, (int)slots))
    finish_partials(part, it.b, slots, 4, 4, dH_post, nullptr, reinterpret_cast<double (*)[20]>(red));
}

// ---------------------------------------------------------------------- stream mix backward
// MODE 0: dH and partials.  MODE 1: partials only (the apply pass writes dH later).
// part: [B, slots, 20] = dH_pre[4] then dH_res[4][4] row-major.  With tickets (one zeroed counter per
// batch element) the CTA of a batch element that stores its partial last also adds them all up into
// dH_pre[b] / dH_res[b].
template <typename T, int V, int MODE>
__global__ void __launch_bounds__(MHC_MAX_COLS, MODE == 0 ? 1 : 512 / MHC_MAX_COLS)
k_stream_mix_bwd(const T* __restrict__ dbi, const T* __restrict__ dHr, const T* __restrict__ H,
                 const float* __restrict__ Hpre, const float* __restrict__ Hres, T* __restrict__ dH,
                 float* __restrict__ part, Geo g, int* tickets, float* __restrict__ dH_pre,
                 float* __restrict__ dH_res) {
  pdl_prologue();
  __shared__ __align__(8) float red[32 * 20];
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
    const int64_t D = g.D, c0 = (int64_t)it.col * V, tok = it.b * g.S;
    using B9 = Bundle<T, V, 9>;  // 0..3 H rows, 4..7 dH_residual rows, 8 d_branch_input
    for_tokens_pipelined<B9>(
        it.s0 + it.sub, it.s1, g.sub,
        [&](B9& u, int64_t s) {
          const int64_t o4 = (tok + s) * 4 * D + c0;
          u.p[8] = ld_raw<T, V>(dbi + (tok + s) * D + c0);
#pragma unroll
          for (int n = 0; n < 4; ++n) u.p[4 + n] = ld_raw<T, V>(dHr + o4 + n * D);
#pragma unroll
          for (int n = 0; n < 4; ++n) u.p[n] = ld_raw<T, V>(H + o4 + n * D);
        },
        [&](const B9& u, int64_t s) {
          float y[4][V];
#pragma unroll
          for (int e = 0; e < V; ++e) {
            float h[4], r[4];
            const float q = raw_get<V>(u.p[8], e);
#pragma unroll
            for (int n = 0; n < 4; ++n) { h[n] = raw_get<V>(u.p[n], e); r[n] = raw_get<V>(u.p[4 + n], e); }
            if (MODE == 0) {
#pragma unroll
              for (int m = 0; m < 4; ++m)
                y[m][e] = w[m] * q + (((R[m] * r[0] + R[4 + m] * r[1]) + R[8 + m] * r[2]) + R[12 + m] * r[3]);
            }
#pragma unroll
            for (int n = 0; n < 4; ++n) {
              acc[n] = fmaf(q, h[n], acc[n]);
#pragma unroll
              for (int m = 0; m < 4; ++m) acc[4 + 4 * n + m] = fmaf(r[n], h[m], acc[4 + 4 * n + m]);
            }
          }
          if (MODE == 0) {
            T* op = dH + (tok + s) * 4 * D + c0;
#pragma unroll
            for (int m = 0; m < 4; ++m) PackIO<T, V>::store(op + m * D, y[m]);
          }
        });
  }
  block_reduce_store<20>(acc, part + (it.b * geo_slots_dev(g) + it.slot) * 20, red);
  if (!tickets) return;
  const int64_t slots = geo_slots_dev(g);
  if (cta_arrives_last(tickets + it.b, (int)slots))
    finish_partials(part, it.b, slots, 20, 4, dH_pre, dH_res, reinterpret_cast<double (*)[20]>(red));
}

// dH[s,m,d] = H_pre[m] d_bi[s,d] + sum_n H_res[n,m] dH_residual[s,n,d] + inv_S * gx[m*D + d].
template <typename T, int V>
__global__ void __launch_bounds__(MHC_MAX_COLS, MHC_APPLY_MINB)
k_stream_mix_bwd_apply(const T* __restrict__ dbi, const T* __restrict__ dHr, const float* __restrict__ Hpre,
                       const float* __restrict__ Hres, const float* __restrict__ gx, float inv_S,
                       T* __restrict__ dH, Geo g) {
  pdl_prologue();
  const Item it = decode_item(g);
  if (it.col >= g.DV) return;
  float w[4], R[16], c[4][V];
#pragma unroll
  for (int n = 0; n < 4; ++n) w[n] = __ldg(Hpre + it.b * 4 + n);
#pragma unroll
  for (int k = 0; k < 16; ++k) R[k] = __ldg(Hres + it.b * 16 + k);
  const int64_t D = g.D, c0 = (int64_t)it.col * V, tok = it.b * g.S;
  // this thread's columns of grad_x / S (fp32), 16-byte loads when the pack is a full vector
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const float* gp = gx + it.b * 4 * D + m * D + c0;
    if (!gx) {
#pragma unroll
      for (int e = 0; e < V; ++e) c[m][e] = 0.f;
    } else if constexpr (V % 4 == 0) {
#pragma unroll
      for (int e = 0; e < V; e += 4) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(gp + e));
        c[m][e] = inv_S * t.x; c[m][e + 1] = inv_S * t.y; c[m][e + 2] = inv_S * t.z; c[m][e + 3] = inv_S * t.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) c[m][e] = inv_S * __ldg(gp + e);
    }
  }
  using B5 = Bundle<T, V, 5>;
  auto load = [&](B5& u, int64_t s) {
    const T* rp = dHr + (tok + s) * 4 * D + c0;
    u.p[4] = ld_raw<T, V>(dbi + (tok + s) * D + c0);
#pragma unroll
    for (int n = 0; n < 4; ++n) u.p[n] = ld_raw<T, V>(rp + n * D);
  };
  auto compute = [&](const B5& u, int64_t s) {
    float r[4][V], q[V], y[V];
    unpack<T, V>(u.p[4], q);
#pragma unroll
    for (int n = 0; n < 4; ++n) unpack<T, V>(u.p[n], r[n]);
    T* op = dH + (tok + s) * 4 * D + c0;
#pragma unroll
    for (int m = 0; m < 4; ++m) {
#pragma unroll
      for (int e = 0; e < V; ++e)
        y[e] = (w[m] * q[e] + (((R[m] * r[0][e] + R[4 + m] * r[1][e]) + R[8 + m] * r[2][e]) + R[12 + m] * r[3][e])) +
               c[m][e];
      PackIO<T, V>::store(op + m * D, y);
    }
  };
  for_tokens<MHC_APPLY_PIPE != 0, B5>(it.s0 + it.sub, it.s1, g.sub, load, compute);
}

// --------------------------------------------------------------------------------- mean-pool
// part[b, chunk, n*D + d] = sum over the chunk's tokens of H[b,s,n,d]  (fp32, tokens in index order).
// blockDim.x = 4 * cols: thread (n, c) owns one 16-byte pack of stream row n and walks all tokens of
// the chunk with MHC_POOL_DEPTH loads in flight.  One pack per thread keeps the state small (V
// accumulators), so many CTAs fit an SM and a single sequence still fills the machine.
template <typename T, int V>
__global__ void __launch_bounds__(4 * MHC_POOL_COLS)
k_meanpool_partial(const T* __restrict__ H, float* __restrict__ part, Geo g) {
  pdl_prologue();
  const Item it = decode_item(g);   // it.col = pack along D, it.sub = stream row n
  if (it.col >= g.DV) return;
  const int64_t D = g.D, c0 = (int64_t)it.col * V;
  const T* h = H + (it.b * g.S * 4 + it.sub) * D + c0;
  float acc[V];
#pragma unroll
  for (int e = 0; e < V; ++e) acc[e] = 0.f;
  constexpr int kDepth = MHC_POOL_DEPTH;
  for (int64_t s = it.s0; s < it.s1; s += kDepth) {
    RawPack<T, V> r[kDepth];
#pragma unroll
    for (int u = 0; u < kDepth; ++u)
      if (s + u < it.s1) r[u] = ld_raw<T, V>(h + (s + u) * 4 * D);
#pragma unroll
    for (int u = 0; u < kDepth; ++u)
      if (s + u < it.s1) {
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] += raw_get<V>(r[u], e);
      }
  }
  float* o = part + (it.b * g.nchunk + it.chunk) * 4 * D + it.sub * D + c0;
  if constexpr (V % 4 == 0) {
#pragma unroll
    for (int e = 0; e < V; e += 4) *reinterpret_cast<float4*>(o + e) = make_float4(acc[e], acc[e + 1], acc[e + 2], acc[e + 3]);
  } else {
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = acc[e];
  }
}

// x[b,k] = scale * sum_chunk part[b, chunk, k], chunks added in a fixed order in fp64.
__global__ void __launch_bounds__(256)
k_meanpool_finish(const float* __restrict__ part, float* __restrict__ x, int64_t K, int nchunk, double scale,
                  int64_t total) {
  pdl_prologue();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int64_t b = i / K, k = i - b * K;
  const float* p = part + b * nchunk * K + k;
  x[i] = (float)(sum_strided_f64(p, K, nchunk) * scale);
}

// out[b, j] = sum_p part[b, p, j] for j < W (W <= 20).  One CTA of 256 threads per batch element:
// thread t adds slots t, t+256, ... in fp64, a xor-shuffle tree adds the lanes of each warp, and
// thread j adds the 8 warp sums in index order.  Columns [0, W0) go to out0, the rest to out1.
__global__ void __launch_bounds__(256)
k_reduce_partials(const float* __restrict__ part, int64_t slots, int W, int W0, float* __restrict__ out0,
                  float* __restrict__ out1) {
  pdl_prologue();
  __shared__ double sm[8][20];
  const int64_t b = blockIdx.x;
  const float* p = part + b * slots * W;
  if (W == 20) block_column_sums_fast<20, false>(p, slots, sm);
  else if (W == 4) block_column_sums_fast<4, false>(p, slots, sm);
  else block_column_sums_f64(p, slots, W, sm);
  const int j = threadIdx.x;
  if (j < W) {
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sm[w][j];
    if (j < W0) out0[b * W0 + j] = (float)t;
    else out1[b * (W - W0) + (j - W0)] = (float)t;
  }
}

// -------------------------------------------------------------------------------- host side
// launch_k for kernels whose dynamic shared memory may exceed the 48 KiB a kernel gets without asking
// (the attribute is per device and per kernel; setting it is a host-side call of about a microsecond).
template <typename... KArgs, typename... Args>
static inline void launch_pool_k(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t st,
                                 Args&&... args) {
  if (smem > 48 * 1024) (void)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_k(kernel, grid, block, smem, st, std::forward<Args>(args)...);
}

int sm_count() {
  static const int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
      (void)cudaGetLastError();
      v = 148;   // no device (size queries on a build machine): the B200 count
    }
    return v;
  }();
  return n;
}

// Range of tokens per CTA that wave_tpc may choose from around `base`.
static inline int tpc_lo(int base) { return base - base / 4 > 1 ? base - base / 4 : 1; }
static inline int tpc_hi(int base) { return base + base / 4; }

// Tokens per CTA near `base` such that the CTAs of ONE batch element fill whole waves of the
// device's `occ` resident CTAs per SM.  Every thread of these kernels keeps a fixed number of bytes
// in flight, so a CTA takes about the same time however many others run beside it, and a last wave
// that is one-third full costs as much as a full one: with a single sequence per GPU (a batch
// sharded over many GPUs) that was up to 14 % of a kernel.  Kernels whose CTAs all fit the device
// at once keep `base`.  The choice depends on S, the column groups and the device, never on the
// batch, so the partial-sum layout of a batch element is the same whatever batch it is part of.
// `abreast` = tokens a CTA walks side by side.
static int wave_tpc(int64_t S, int CG, int abreast, int base, int occ) {
  if (occ <= 0 || S <= 0) return base;
  const int64_t slots = (int64_t)sm_count() * occ;
  auto fill = [&](int t, int64_t* waves_out) {   // share of the slot-time the CTAs use, in 1/1000
    const int64_t chunks = (S + (int64_t)t * abreast - 1) / ((int64_t)t * abreast);
    const int64_t items = chunks * CG, waves = (items + slots - 1) / slots;
    *waves_out = waves;
    return items * 1000 / (waves * slots);
  };
  int64_t waves = 0;
  int best = base;
  int64_t best_fill = fill(base, &waves);
  if (waves <= 1) return base;
  for (int t = tpc_lo(base); t <= tpc_hi(base); ++t) {
    const int64_t f = fill(t, &waves);
    if (f > best_fill + 30 && f > fill(best, &waves)) { best = t; }
  }
  return best;
}

// occ > 0: adjust the tokens per CTA to the device's waves (wave_tpc); occ < 0: the smallest chunk
// wave_tpc could choose, i.e. an upper bound of the number of chunks (scratch-size queries).
Geo make_geo(int64_t S, int64_t D, int vec, GeoKind kind, int tpc, int occ, bool fit_cols, int narrow_mult) {
  Geo g;
  g.reverse = 0;
  g.S = S;
  g.D = D;
  g.DV = (int32_t)(D / vec);
  const bool pool = kind == GeoKind::Pool;
  const int max_cols = pool ? MHC_POOL_COLS : MHC_MAX_COLS;
  int cols = 32;
  while (cols < max_cols && cols < g.DV) cols <<= 1;
  // A row whose packs do not fill whole groups of `cols` leaves lanes of its last group idle (D = 7168 in
  // bf16: 896 packs = 3.5 x 256, one lane in eight).  Take the widest narrower group that fits the row to
  // within 1/32 instead; the CTA keeps its thread count by walking more tokens abreast.
  if (fit_cols && !pool) {
    auto waste = [&](int c) { return (g.DV + c - 1) / c * c - g.DV; };
    if (waste(cols) * 32 > g.DV)
      for (int c = cols >> 1; c >= 64; c >>= 1)
        if (waste(c) * 32 <= g.DV) { cols = c; break; }
  }
  g.cols = cols;
  g.CG = (g.DV + cols - 1) / cols;
  if (pool) {
    g.sub = 4;   // the four stream rows: blockDim.x = 4 * cols
    g.tpc = occ < 0 ? tpc_lo(tpc) : wave_tpc(S, g.CG, 1, tpc, occ);
  } else {
    // Tokens per CTA: a per-kernel constant (adjusted to the device's waves), so the chunking (and
    // with it the layout of the per-CTA partial sums) depends on S and D only, never on the batch size.
    // Narrow rows (fewer than 256 packs): the CTA keeps 256 threads by walking 256/cols tokens abreast.
    g.sub = MHC_MAX_COLS / cols;
    if (g.sub > 1) tpc *= narrow_mult;
    const int t = occ < 0 ? tpc_lo(tpc) : wave_tpc(S, g.CG, g.sub, tpc, occ);
    g.tpc = t * g.sub;
  }
  if (g.tpc > S) g.tpc = (int32_t)(S > 0 ? S : 1);
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

// The in-kernel finish of the per-CTA partial sums is written for CTAs of 256 threads.
bool ticket_finish_supported() { return MHC_MAX_COLS == 256; }

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

// Launch sequences shared by the single-op and the fused entry points.  Arguments are validated by
// the callers; these pick the pack width, build the geometry and launch.
int stream_mix_fwd_impl(const void* H, const float* H_pre, const float* H_res, void* bi, void* Hr, int64_t B, int64_t S,
                        int64_t D, int dtype, cudaStream_t st) {
  const int vec = pick_vec(dtype, D, {H, bi, Hr});
  Geo g = make_geo(S, D, vec, GeoKind::Stream, MHC_TPC_MIXFWD);
  g.reverse = (MHC_REV_MASK >> 1) & 1;
  const int64_t items = B * geo_slots(g);
  if (int e = check_grid("stream_mix_fwd", items)) return e;
  if (!Hr) {  // branch_input only; the residual mix is recomputed by mhc_add_residual_mix_fwd
    Geo gp = make_geo(S, D, vec, GeoKind::Stream, MHC_TPC_PREMIX);
    gp.reverse = g.reverse;
    const int64_t n = B * geo_slots(gp);
    if (int e = check_grid("stream_mix_fwd", n)) return e;
    ProfScope ps("k_stream_premix_fwd", st);
    MHC_DISPATCH(dtype, vec, (launch_k(k_stream_premix_fwd<T, V>, (unsigned)n, geo_block(gp), 0, st, (const T*)H, H_pre,
                                       (T*)bi, gp)));
  } else {
    ProfScope ps("k_stream_mix_fwd", st);
    MHC_DISPATCH(dtype, vec, (launch_k(k_stream_mix_fwd<T, V>, (unsigned)items, geo_block(g), 0, st, 
                                 (const T*)H, H_pre, H_res, (T*)bi, (T*)Hr, g)));
  }
  return check_launch("stream_mix_fwd");
}

// Scratch sizes are upper bounds over the pack widths and the chunk lengths a launch may pick.
int64_t meanpool_scratch_floats(int64_t B, int64_t S, int64_t D) { return B * make_geo(S, D, 1, GeoKind::Pool, MHC_POOL_TPC, -1).nchunk * 4 * D; }
int64_t mix_bwd_scratch_floats(int64_t B, int64_t S, int64_t D) { return B * geo_slots(make_geo(S, D, 1, GeoKind::Reduce, MHC_TPC_MIXBWD, -1)) * 20; }

int meanpool_partial_impl(const void* H, float* part, int64_t B, int64_t S, int64_t D, int dtype, cudaStream_t st,
                          int* nchunk) {
  const int vec = pick_vec(dtype, D, {H});
  Geo g = make_geo(S, D, vec, GeoKind::Pool, MHC_POOL_TPC, MHC_POOL_OCC);
  g.reverse = MHC_REV_MASK & 1;
  const int64_t items = B * geo_slots(g);
  if (int e = check_grid("meanpool_fwd", items)) return e;
  {
    ProfScope ps("k_meanpool_partial", st);
    MHC_DISPATCH(dtype, vec, (launch_k(k_meanpool_partial<T, V>, (unsigned)items, geo_block(g), 0, st, (const T*)H, part, g)));
  }
  *nchunk = g.nchunk;
  return check_launch("meanpool_fwd");
}

// mode 0: dH + partials; mode 1: partials only.
// tickets != null: the kernel itself finishes the sums into dH_pre / dH_res (see k_stream_mix_bwd).
int mix_bwd_partials_impl(int mode, const void* dbi, const void* dHr, const void* H, const float* H_pre,
                          const float* H_res, void* dH, float* part, int64_t B, int64_t S, int64_t D, int dtype,
                          cudaStream_t st, int64_t* slots, int* tickets, float* dH_pre, float* dH_res) {
  if (!ticket_finish_supported()) tickets = nullptr;
  const int vec = pick_vec(dtype, D, {dbi, dHr, H, dH});
  Geo g = make_geo(S, D, vec, GeoKind::Reduce, MHC_TPC_MIXBWD, mode == 0 ? 1 : 512 / MHC_MAX_COLS);
  g.reverse = (MHC_REV_MASK >> 4) & 1;
  *slots = geo_slots(g);
  const int64_t items = B * *slots;
  if (int e = check_grid("stream_mix_bwd", items)) return e;
  if (mode == 0) {
    ProfScope ps("k_stream_mix_bwd_full", st);
    MHC_DISPATCH(dtype, vec, (launch_k(k_stream_mix_bwd<T, V, 0>, (unsigned)items, geo_block(g), 0, st, 
                                 (const T*)dbi, (const T*)dHr, (const T*)H, H_pre, H_res, (T*)dH, part, g, tickets,
                                 dH_pre, dH_res)));
  } else {
    ProfScope ps("k_stream_mix_bwd_reduce", st);
    MHC_DISPATCH(dtype, vec, (launch_k(k_stream_mix_bwd<T, V, 1>, (unsigned)items, geo_block(g), 0, st, 
                                 (const T*)dbi, (const T*)dHr, (const T*)H, nullptr, nullptr, nullptr, part, g, tickets,
                                 dH_pre, dH_res)));
  }
  return check_launch("stream_mix_bwd");
}

int mix_bwd_apply_impl(const void* dbi, const void* dHr, const float* H_pre, const float* H_res, const float* gx,
                       float inv_S, void* dH, int64_t B, int64_t S, int64_t D, int dtype, cudaStream_t st) {
  const int vec = pick_vec(dtype, D, {dbi, dHr, dH});
  Geo g = make_geo(S, D, vec, GeoKind::Stream, MHC_TPC_APPLY, MHC_APPLY_MINB, MHC_FIT_COLS != 0, MHC_NARROW_MULT);
  g.reverse = (MHC_REV_MASK >> 5) & 1;
  const int64_t items = B * geo_slots(g);
  if (int e = check_grid("stream_mix_bwd_apply", items)) return e;
  {
    ProfScope ps("k_stream_mix_bwd_apply", st);
    MHC_DISPATCH(dtype, vec, (launch_k(k_stream_mix_bwd_apply<T, V>, (unsigned)items, geo_block(g), 0, st, 
                                 (const T*)dbi, (const T*)dHr, H_pre, H_res, gx, inv_S, (T*)dH, g)));
  }
  return check_launch("stream_mix_bwd_apply");
}

// Exact scratch requirement of mhc_add_residual_bwd for these arguments (the pack width, and with it
// the number of per-CTA partial sums, depends on D and on the alignment of the three tensors).
int64_t add_residual_bwd_need_bytes(const void* dH_new, const void* bo, const void* dbo, int64_t B, int64_t S,
                                    int64_t D, int dtype) {
  if (B <= 0 || S <= 0 || D <= 0) return 0;
  const int vec = pick_vec(dtype, D, {dH_new, bo, dbo});
  return B * geo_slots(make_geo(S, D, vec, GeoKind::Reduce, MHC_TPC_ADDBWD, MHC_ADDBWD_OCC, MHC_FIT_COLS != 0, MHC_NARROW_MULT)) * 4 * (int64_t)sizeof(float);
}

int check_bsd_pub(const char* what, int64_t B, int64_t S, int64_t D, int dtype) { return check_bsd(what, B, S, D, dtype); }

static int launch_reduce(const float* part, int64_t B, int64_t slots, int W, int W0, float* out0, float* out1,
                         cudaStream_t st, const char* what) {
  {
    ProfScope ps("k_reduce_partials", st);
    launch_k(k_reduce_partials, (unsigned)B, 256, 0, st, part, slots, W, W0, out0, out1);
  }
  return check_launch(what);
}

}  // namespace mhc

using namespace mhc;

extern "C" int64_t mhc_scratch_bytes(int op, int64_t B, int64_t S, int64_t D, int dtype) {
  if (B < 0 || S < 0 || D < 0) return -1;
  (void)dtype;
  const int64_t f = (int64_t)sizeof(float);
  // Sized for the scalar path (pack width 1), which has the most column groups.
  switch (op) {
    case MHC_OP_ADD_RESIDUAL_BWD: return B * geo_slots(make_geo(S, D, 1, GeoKind::Reduce, MHC_TPC_ADDBWD, -1)) * 4 * f;
    case MHC_OP_STREAM_MIX_BWD: return mix_bwd_scratch_floats(B, S, D) * f;
    case MHC_OP_MEANPOOL_FWD: return meanpool_scratch_floats(B, S, D) * f;
    case MHC_OP_DYNAMIC_WEIGHTS_FWD: return weights_fwd_scratch_bytes(B, 4 * D);
    case MHC_OP_DYNAMIC_WEIGHTS_BWD: return weights_bwd_scratch_bytes(B, 4 * D);
    case MHC_OP_HC_MIX_FWD: return meanpool_scratch_floats(B, S, D) * f + weights_fwd_scratch_bytes(B, 4 * D);
    case MHC_OP_HC_MIX_BWD: return mix_bwd_scratch_floats(B, S, D) * f + weights_bwd_scratch_bytes(B, 4 * D);
  }
  return -1;
}

extern "C" int mhc_stream_mix_fwd(const void* H, const float* H_pre, const float* H_res, void* branch_input,
                                  void* H_residual, int64_t B, int64_t S, int64_t D, int dtype,
                                  mhc_stream_t stream) {
  if (int e = check_bsd("stream_mix_fwd", B, S, D, dtype)) return e;
  if (B == 0 || S == 0 || D == 0) return MHC_OK;
  if (!H || !H_pre || !branch_input || (H_residual && !H_res)) return fail(MHC_ERR_NULL_POINTER, "stream_mix_fwd: null pointer");
  return stream_mix_fwd_impl(H, H_pre, H_res, branch_input, H_residual, B, S, D, dtype, (cudaStream_t)stream);
}

extern "C" int mhc_add_residual_fwd(const void* H_residual, const void* branch_output, const float* H_post,
                                    void* H_new, int64_t B, int64_t S, int64_t D, int dtype, mhc_stream_t stream) {
  if (int e = check_bsd("add_residual_fwd", B, S, D, dtype)) return e;
  if (B == 0 || S == 0 || D == 0) return MHC_OK;
  if (!H_residual || !branch_output || !H_post || !H_new) return fail(MHC_ERR_NULL_POINTER, "add_residual_fwd: null pointer");
  const int vec = pick_vec(dtype, D, {H_residual, branch_output, H_new});
  Geo g = make_geo(S, D, vec, GeoKind::Stream, MHC_TPC_ADDFWD);
  g.reverse = (MHC_REV_MASK >> 2) & 1;
  const int64_t items = B * geo_slots(g);
  if (int e = check_grid("add_residual_fwd", items)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  {
    ProfScope ps("k_add_residual_fwd", st);
    MHC_DISPATCH(dtype, vec, (launch_k(k_add_residual_fwd<T, V>, (unsigned)items, geo_block(g), 0, st, 
                                 (const T*)H_residual, (const T*)branch_output, H_post, (T*)H_new, g)));
  }
  return check_launch("add_residual_fwd");
}

// Tokens per chunk of the add-residual kernels that also pool: MHC_TPC_ADDPOOL adjusted so that one batch
// element's CTAs fill whole waves (two resident CTAs per SM; column groups counted for 16-byte packs of
// 2-byte elements, the common case; other layouts get the same chunk length, only a less even fill).
// A function of S, D and the device only, shared by the launch and by mhc_add_residual_pool_chunks.
static int addpool_tpc(int64_t S, int64_t D) {
  const int64_t dv = D >= 8 ? D / 8 : 1;
  const int cg = (int)((dv + MHC_MAX_COLS - 1) / MHC_MAX_COLS);
  return wave_tpc(S, cg, 1, MHC_TPC_ADDPOOL, MHC_ADDMIXPOOL_MINB);
}

extern "C" int64_t mhc_add_residual_pool_chunks(int64_t S, int64_t D) {
  if (S <= 0) return 0;
  const int tpc = addpool_tpc(S, D);
  return (S + tpc - 1) / tpc;
}

extern "C" int mhc_add_residual_mix_fwd(const void* H, const float* H_res, const void* branch_output,
                                        const float* H_post, void* H_new, float* pool_partials, int64_t B, int64_t S,
                                        int64_t D, int dtype, mhc_stream_t stream) {
  if (int e = check_bsd("add_residual_mix_fwd", B, S, D, dtype)) return e;
  if (B == 0 || S == 0 || D == 0) return MHC_OK;
  if (!H || !H_res || !branch_output || !H_post || !H_new)
    return fail(MHC_ERR_NULL_POINTER, "add_residual_mix_fwd: null pointer");
  const int vec = pick_vec(dtype, D, {H, branch_output, H_new});
  cudaStream_t st = (cudaStream_t)stream;
  if (pool_partials) {
    Geo g = make_geo(S, D, vec, GeoKind::Reduce, MHC_TPC_ADDPOOL);
    const int ptpc = addpool_tpc(S, D);
    g.tpc = (int32_t)(S < ptpc ? S : ptpc);
    g.nchunk = (int32_t)mhc_add_residual_pool_chunks(S, D);
    g.reverse = (MHC_REV_MASK >> 2) & 1;
    const int64_t items = B * geo_slots(g);
    if (int e = check_grid("add_residual_mix_fwd", items)) return e;
    size_t smem = g.sub > 1 ? (size_t)2 * vec * geo_block(g) * sizeof(float) : 0;
    if (vec > 1 && MHC_ADDPOOL_STAGES > 0) smem = std::max(smem, (size_t)MHC_ADDPOOL_STAGES * 5 * 16 * geo_block(g));
    ProfScope ps("k_add_residual_mix_pool_fwd", st);
    MHC_DISPATCH(dtype, vec, (launch_pool_k(k_add_residual_mix_fwd<T, V, true>, (unsigned)items, geo_block(g), smem, st,
                                            (const T*)H, H_res, (const T*)branch_output, H_post, (T*)H_new, pool_partials, g)));
  } else {
    Geo g = make_geo(S, D, vec, GeoKind::Stream, MHC_TPC_ADDMIX);
    g.reverse = (MHC_REV_MASK >> 2) & 1;
    const int64_t items = B * geo_slots(g);
    if (int e = check_grid("add_residual_mix_fwd", items)) return e;
    ProfScope ps("k_add_residual_mix_fwd", st);
    MHC_DISPATCH(dtype, vec, (launch_k(k_add_residual_mix_fwd<T, V, false>, (unsigned)items, geo_block(g), 0, st,
                                       (const T*)H, H_res, (const T*)branch_output, H_post, (T*)H_new, (float*)nullptr,
                                       g)));
  }
  return check_launch("add_residual_mix_fwd");
}


extern "C" int mhc_add_residual_pool_fwd(const void* H_residual, const void* branch_output, const float* H_post,
                                         void* H_new, float* pool_partials, int64_t B, int64_t S, int64_t D, int dtype,
                                         mhc_stream_t stream) {
  if (int e = check_bsd("add_residual_pool_fwd", B, S, D, dtype)) return e;
  if (B == 0 || S == 0 || D == 0) return MHC_OK;
  if (!H_residual || !branch_output || !H_post || !H_new || !pool_partials)
    return fail(MHC_ERR_NULL_POINTER, "add_residual_pool_fwd: null pointer");
  const int vec = pick_vec(dtype, D, {H_residual, branch_output, H_new});
  Geo g = make_geo(S, D, vec, GeoKind::Reduce, MHC_TPC_ADDPOOL);
  // Chunks are addpool_tpc tokens whatever the pack width (token sub-groups share a chunk), so the
  // number of partial rows is a function of S and D only.
  const int ptpc = addpool_tpc(S, D);
  g.tpc = (int32_t)(S < ptpc ? S : ptpc);
  g.nchunk = (int32_t)mhc_add_residual_pool_chunks(S, D);
  g.reverse = (MHC_REV_MASK >> 2) & 1;
  const int64_t items = B * geo_slots(g);
  if (int e = check_grid("add_residual_pool_fwd", items)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  size_t smem = g.sub > 1 ? (size_t)2 * vec * geo_block(g) * sizeof(float) : 0;
  if (vec > 1 && MHC_ADDPOOL_STAGES > 0) smem = std::max(smem, (size_t)MHC_ADDPOOL_STAGES * 5 * 16 * geo_block(g));
  {
    ProfScope ps("k_add_residual_pool_fwd", st);
    MHC_DISPATCH(dtype, vec, (launch_pool_k(k_add_residual_pool_fwd<T, V>, (unsigned)items, geo_block(g), smem, st,
                                       (const T*)H_residual, (const T*)branch_output, H_post, (T*)H_new, pool_partials, g)));
  }
  return check_launch("add_residual_pool_fwd");
}

extern "C" int mhc_add_residual_bwd(const void* dH_new, const void* branch_output, const float* H_post,
                                    void* d_branch_output, float* dH_post, void* scratch, int64_t scratch_bytes,
                                    int32_t* tickets, int64_t B, int64_t S, int64_t D, int dtype,
                                    mhc_stream_t stream) {
  if (int e = check_bsd("add_residual_bwd", B, S, D, dtype)) return e;
  if (B == 0) return MHC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (S == 0 || D == 0) {
    if (!dH_post) return fail(MHC_ERR_NULL_POINTER, "add_residual_bwd: null pointer");
    if (cudaMemsetAsync(dH_post, 0, B * 4 * sizeof(float), st) != cudaSuccess) return check_launch("add_residual_bwd");
    return MHC_OK;
  }
  // sizes first, pointers last: a call whose scratch is too small says so even with null pointers
  const int vec = pick_vec(dtype, D, {dH_new, branch_output, d_branch_output});
  Geo g = make_geo(S, D, vec, GeoKind::Reduce, MHC_TPC_ADDBWD, MHC_ADDBWD_OCC, MHC_FIT_COLS != 0, MHC_NARROW_MULT);
  g.reverse = (MHC_REV_MASK >> 3) & 1;
  const int64_t slots = geo_slots(g), items = B * slots;
  if (int e = check_grid("add_residual_bwd", items)) return e;
  if (scratch_bytes < items * 4 * (int64_t)sizeof(float))
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "add_residual_bwd: scratch %lld < %lld bytes", (long long)scratch_bytes,
                (long long)(items * 4 * sizeof(float)));
  if (!dH_new || !branch_output || !H_post || !d_branch_output || !dH_post || !scratch)
    return fail(MHC_ERR_NULL_POINTER, "add_residual_bwd: null pointer");
  if (!is_aligned_to(tickets, 4) || !is_aligned_to(scratch, 4) || !is_aligned_to(dH_post, 4))
    return fail(MHC_ERR_MISALIGNED, "add_residual_bwd: tickets / scratch / dH_post must be 4-byte aligned");
  if (!ticket_finish_supported()) tickets = nullptr;
  {
    ProfScope ps("k_add_residual_bwd", st);
    MHC_DISPATCH(dtype, vec, (launch_k(k_add_residual_bwd<T, V>, (unsigned)items, geo_block(g), 0, st, 
                                 (const T*)dH_new, (const T*)branch_output, H_post, (T*)d_branch_output,
                                 (float*)scratch, g, (int*)tickets, dH_post)));
  }
  if (int e = check_launch("add_residual_bwd")) return e;
  if (tickets) return MHC_OK;   // the last CTA of every batch element has written dH_post
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
  if (scratch_bytes < mix_bwd_scratch_floats(B, S, D) * (int64_t)sizeof(float))
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "%s: scratch %lld < %lld bytes", what, (long long)scratch_bytes,
                (long long)(mix_bwd_scratch_floats(B, S, D) * sizeof(float)));
  int64_t slots = 0;
  if (int e = mix_bwd_partials_impl(mode, dbi, dHr, H, H_pre, H_res, dH, (float*)scratch, B, S, D, dtype, st, &slots,
                                    nullptr, nullptr, nullptr))
    return e;
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
  return mix_bwd_apply_impl(d_branch_input, dH_residual, H_pre, H_res, grad_x, inv_S, dH, B, S, D, dtype,
                            (cudaStream_t)stream);
}

extern "C" int mhc_meanpool_fwd(const void* H, float* x, void* scratch, int64_t scratch_bytes, int64_t B, int64_t S,
                                int64_t D, int dtype, mhc_stream_t stream) {
  if (int e = check_bsd("meanpool_fwd", B, S, D, dtype)) return e;
  if (B == 0 || D == 0) return MHC_OK;
  if (S == 0) return fail(MHC_ERR_BAD_SHAPE, "meanpool_fwd: empty sequence");
  if (!H || !x || !scratch) return fail(MHC_ERR_NULL_POINTER, "meanpool_fwd: null pointer");
  const int64_t need = meanpool_scratch_floats(B, S, D) * (int64_t)sizeof(float);
  if (scratch_bytes < need)
    return fail(MHC_ERR_SCRATCH_TOO_SMALL, "meanpool_fwd: scratch %lld < %lld bytes", (long long)scratch_bytes, (long long)need);
  cudaStream_t st = (cudaStream_t)stream;
  int nchunk = 0;
  if (int e = meanpool_partial_impl(H, (float*)scratch, B, S, D, dtype, st, &nchunk)) return e;
  const int64_t total = B * 4 * D;
  {
    ProfScope ps("k_meanpool_finish", st);
    launch_k(k_meanpool_finish, (unsigned)((total + 255) / 256), 256, 0, st, (const float*)scratch, x, 4 * D, nchunk,
                                                                        1.0 / (double)S, total);
  }
  return check_launch("meanpool_fwd(finish)");
}

// Shared device helpers for the sm_100a hyper-connection kernels: 128-bit element packs,
// the (batch element, token chunk, column group) work decomposition used by every streaming
// kernel, and the fixed-order block reduction behind the deterministic weight gradients.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mhc {

// First statement of every kernel: let the next kernel on the stream start being scheduled, then
// wait until the previous kernel has completed and its writes are visible (both are no-ops for a
// launch without the programmatic-serialization attribute).
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

constexpr int kStreams = 4;
constexpr int kOut = 24;        // 4 pre + 4 post + 16 res
constexpr int kSavedStride = 32;  // floats per row of the forward's saved buffer

// ---------------------------------------------------------------------------------------
// Element packs: V elements of T moved as one access (16 bytes when V == vec_width<T>),
// always computed on as fp32.
// ---------------------------------------------------------------------------------------
template <typename T> struct vec_width;
template <> struct vec_width<float> { static constexpr int value = 4; };
template <> struct vec_width<__nv_bfloat16> { static constexpr int value = 8; };
template <> struct vec_width<__half> { static constexpr int value = 8; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Read-only 16-byte load that does not allocate in L1 (every byte is used exactly once per kernel).
// Volatile with a memory clobber so that the compiler never moves it above griddepcontrol.wait: the
// tensor may have been written by the kernel before this one on the stream, which can still be
// running when a kernel launched with programmatic serialization starts.  After that wait nobody
// writes the tensor any more, and no line of it can sit in this SM's L1 from earlier (the loads never
// allocate there), so the non-coherent path returns what the previous kernel wrote.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p)
               : "memory");
  return r;
}
#ifndef MHC_ST_MODE
#define MHC_ST_MODE 0
#endif
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
#if MHC_ST_MODE == 1
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
#elif MHC_ST_MODE == 2
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
#else
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
#endif
}

template <typename T, int V> struct PackIO;

template <typename T> struct PackIO<T, 1> {
  static __device__ __forceinline__ void load(const T* __restrict__ p, float (&o)[1]) { o[0] = to_f32(__ldg(p)); }
  static __device__ __forceinline__ void store(T* __restrict__ p, const float (&v)[1]) { *p = from_f32<T>(v[0]); }
  // store, and leave in v the values as a later load would return them (rounded to T)
  static __device__ __forceinline__ void store_round(T* __restrict__ p, float (&v)[1]) {
    const T t = from_f32<T>(v[0]);
    *p = t;
    v[0] = to_f32(t);
  }
};

template <> struct PackIO<float, 4> {
  static __device__ __forceinline__ void load(const float* __restrict__ p, float (&o)[4]) {
    uint4 r = ld_stream16(p);
    o[0] = __uint_as_float(r.x); o[1] = __uint_as_float(r.y);
    o[2] = __uint_as_float(r.z); o[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ void store(float* __restrict__ p, const float (&v)[4]) {
    st_stream16(p, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]),
                              __float_as_uint(v[3])));
  }
  static __device__ __forceinline__ void store_round(float* __restrict__ p, float (&v)[4]) { store(p, v); }
};

template <> struct PackIO<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* __restrict__ p, float (&o)[8]) {
    uint4 r = ld_stream16(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // bf16 -> fp32 is a 16-bit shift
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* __restrict__ p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    st_stream16(p, make_uint4(w[0], w[1], w[2], w[3]));
  }
  static __device__ __forceinline__ void store_round(__nv_bfloat16* __restrict__ p, float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
    st_stream16(p, make_uint4(w[0], w[1], w[2], w[3]));
  }
};

template <> struct PackIO<__half, 8> {
  static __device__ __forceinline__ void load(const __half* __restrict__ p, float (&o)[8]) {
    uint4 r = ld_stream16(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      o[2 * i] = f.x;
      o[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* __restrict__ p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    st_stream16(p, make_uint4(w[0], w[1], w[2], w[3]));
  }
  static __device__ __forceinline__ void store_round(__half* __restrict__ p, float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
      const float2 f = __half22float2(h);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
    st_stream16(p, make_uint4(w[0], w[1], w[2], w[3]));
  }
};

// Raw (unconverted) packs: what a load leaves in registers until the arithmetic needs it.  Keeping
// the next token's packs raw lets a thread hold a second token in flight for 4 registers per pack.
template <typename T, int V> struct RawPack { uint4 w; };
template <typename T> struct RawPack<T, 1> { T w; };

template <typename T, int V> __device__ __forceinline__ RawPack<T, V> ld_raw(const T* __restrict__ p) {
  RawPack<T, V> r;
  r.w = ld_stream16(p);
  return r;
}
template <> __device__ __forceinline__ RawPack<float, 1> ld_raw<float, 1>(const float* __restrict__ p) {
  RawPack<float, 1> r; r.w = __ldg(p); return r;
}
template <> __device__ __forceinline__ RawPack<__nv_bfloat16, 1> ld_raw<__nv_bfloat16, 1>(const __nv_bfloat16* __restrict__ p) {
  RawPack<__nv_bfloat16, 1> r; r.w = __ldg(p); return r;
}
template <> __device__ __forceinline__ RawPack<__half, 1> ld_raw<__half, 1>(const __half* __restrict__ p) {
  RawPack<__half, 1> r; r.w = __ldg(p); return r;
}

// Element e (compile-time constant after unrolling) of a raw pack, as fp32.
template <int V> __device__ __forceinline__ float raw_get(const RawPack<float, V>& r, int e) {
  if constexpr (V == 1) return r.w;
  else return __uint_as_float(e == 0 ? r.w.x : e == 1 ? r.w.y : e == 2 ? r.w.z : r.w.w);
}
template <int V> __device__ __forceinline__ float raw_get(const RawPack<__nv_bfloat16, V>& r, int e) {
  if constexpr (V == 1) return __bfloat162float(r.w);
  else {
    const uint32_t w = (e >> 1) == 0 ? r.w.x : (e >> 1) == 1 ? r.w.y : (e >> 1) == 2 ? r.w.z : r.w.w;
    return __uint_as_float((e & 1) ? (w & 0xffff0000u) : (w << 16));
  }
}
template <int V> __device__ __forceinline__ float raw_get(const RawPack<__half, V>& r, int e) {
  if constexpr (V == 1) return __half2float(r.w);
  else {
    const uint32_t w = (e >> 1) == 0 ? r.w.x : (e >> 1) == 1 ? r.w.y : (e >> 1) == 2 ? r.w.z : r.w.w;
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    return (e & 1) ? __high2float(h) : __low2float(h);
  }
}

// The packs a thread holds for one token (N rows of 16 bytes, or N scalars).
template <typename T, int V, int N> struct Bundle { RawPack<T, V> p[N]; };

// Plain token loop: load, then compute (more resident CTAs cover the latency instead).
template <class Bundle, class Load, class Compute>
__device__ __forceinline__ void for_tokens_simple(int64_t s0, int64_t s1, int64_t step, Load load, Compute compute) {
  for (int64_t s = s0; s < s1; s += step) {
    Bundle a;
    load(a, s);
    compute(a, s);
  }
}

// Software pipeline over the tokens s0, s0+step, ... < s1: the loads of the next token are issued
// before the arithmetic of the current one, so every thread always has one token's packs in flight.
template <class Bundle, class Load, class Compute>
__device__ __forceinline__ void for_tokens_pipelined(int64_t s0, int64_t s1, int64_t step, Load load, Compute compute) {
  if (s0 >= s1) return;
  Bundle a, b;
  load(a, s0);
  for (int64_t s = s0; s < s1; s += 2 * step) {
    const bool second = s + step < s1;
    if (second) load(b, s + step);
    compute(a, s);
    if (second) {
      if (s + 2 * step < s1) load(a, s + 2 * step);
      compute(b, s + step);
    }
  }
}

// Token loop whose loads in flight live in shared memory instead of registers: every thread copies the N
// packs of the next DEPTH-1 tokens with cp.async (16 bytes each, L2 only) into slots of its own and reads
// a token's packs back when its copy group has landed.  A thread only ever reads what it copied itself,
// so no barrier is involved, and a kernel whose accumulators leave no registers for packs in flight
// still keeps (DEPTH-1) * N * 16 bytes per thread on the way.  Slot (stage d, pack n) of thread t is at
// ring + ((d * N + n) * blockDim.x + t) * 16: conflict-free for the copies and for the reads.
// `addr(s, n)` returns the global address of pack n of token s.  Needs 16-byte packs (V > 1).
template <typename T, int V, int N, int DEPTH, class Addr, class Compute>
__device__ __forceinline__ void for_tokens_staged(int64_t s0, int64_t s1, int64_t step, uint32_t ring, Addr addr,
                                                  Compute compute) {
  static_assert(DEPTH >= 2 && DEPTH <= 8, "ring depth");
  const uint32_t mine = ring + threadIdx.x * 16u, pitch = blockDim.x * 16u;
  auto issue = [&](int d, int64_t s) {
#pragma unroll
    for (int n = 0; n < N; ++n)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(mine + (uint32_t)(d * N + n) * pitch), "l"(addr(s, n))
                   : "memory");
  };
  int64_t next = s0;
#pragma unroll
  for (int d = 0; d < DEPTH - 1; ++d) {
    if (next < s1) issue(d, next);
    asm volatile("cp.async.commit_group;" ::: "memory");
    next += step;
  }
  int d = 0;
  for (int64_t s = s0; s < s1; s += step) {
    const int dn = d == 0 ? DEPTH - 1 : d - 1;   // the stage read in the previous iteration
    if (next < s1) issue(dn, next);
    asm volatile("cp.async.commit_group;" ::: "memory");
    next += step;
    asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
    Bundle<T, V, N> a;
#pragma unroll
    for (int n = 0; n < N; ++n)
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(a.p[n].w.x), "=r"(a.p[n].w.y), "=r"(a.p[n].w.z), "=r"(a.p[n].w.w)
                   : "r"(mine + (uint32_t)(d * N + n) * pitch)
                   : "memory");
    compute(a, s);
    d = d + 1 == DEPTH ? 0 : d + 1;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <bool PIPE, class Bundle, class Load, class Compute>
__device__ __forceinline__ void for_tokens(int64_t s0, int64_t s1, int64_t step, Load load, Compute compute) {
  if constexpr (PIPE) for_tokens_pipelined<Bundle>(s0, s1, step, load, compute);
  else for_tokens_simple<Bundle>(s0, s1, step, load, compute);
}

// ---------------------------------------------------------------------------------------
// Work decomposition.  One CTA = one (batch element b, chunk of `tpc` consecutive tokens,
// group of blockDim.x consecutive packs along D).  The layout of the per-CTA partial sums
// depends only on (S, D, dtype, alignment), never on the batch size or the grid, so a batch
// shard reduces in exactly the same order as the full batch does.
// ---------------------------------------------------------------------------------------
struct Geo {
  int64_t S;       // tokens per batch element
  int64_t D;       // elements per stream row
  int32_t DV;      // packs per stream row (D / V)
  int32_t CG;      // column groups per row = ceil(DV / columns per CTA)
  int32_t tpc;     // tokens per chunk
  int32_t nchunk;  // ceil(S / tpc)
  int32_t cols;    // columns (packs) per CTA
  int32_t sub;     // token sub-groups inside a CTA (blockDim.x = cols * sub)
  int32_t reverse; // walk the work items from the end of the tensor towards its start
};

struct Item {
  int64_t b;
  int32_t chunk, cg;
  int64_t s0, s1;  // token range
  int32_t col;     // pack index along D for this thread (may be >= DV: idle lane)
  int32_t sub;
  int32_t slot;    // index of this CTA's partial inside its batch element: chunk * CG + cg
};

__device__ __forceinline__ Item decode_item(const Geo& g) {
  Item it;
  const int64_t w = g.reverse ? (int64_t)gridDim.x - 1 - blockIdx.x : (int64_t)blockIdx.x;
  it.cg = (int32_t)(w % g.CG);
  const int64_t r = w / g.CG;
  it.chunk = (int32_t)(r % g.nchunk);
  it.b = r / g.nchunk;
  it.s0 = (int64_t)it.chunk * g.tpc;
  it.s1 = min(it.s0 + (int64_t)g.tpc, g.S);
  it.col = it.cg * g.cols + (int32_t)(threadIdx.x % g.cols);
  it.sub = (int32_t)(threadIdx.x / g.cols);
  it.slot = it.chunk * g.CG + it.cg;
  return it;
}

__device__ __forceinline__ int64_t geo_slots_dev(const Geo& g) { return (int64_t)g.nchunk * g.CG; }

// ---------------------------------------------------------------------------------------
// Fixed-order block reduction of W per-thread accumulators: xor-shuffle tree inside each warp,
// then one thread per value sums the warps in index order.  blockDim.x must be a multiple of
// 32 and every thread of the CTA must call this.  `out` receives W floats.
// ---------------------------------------------------------------------------------------
template <int W>
__device__ __forceinline__ void block_reduce_store(float (&acc)[W], float* __restrict__ out, float* smem) {
#pragma unroll
  for (int i = 0; i < W; ++i) {
    float v = acc[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    acc[i] = v;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < W; ++i) smem[warp * W + i] = acc[i];
  }
  __syncthreads();
  if (threadIdx.x < W) {
    float s = 0.f;
    for (int w = 0; w < nw; ++w) s += smem[w * W + threadIdx.x];
    out[threadIdx.x] = s;
  }
}

// 1/x with one MUFU instruction (relative error about 1 ulp); every divisor here is >= eps > 0.
__device__ __forceinline__ float rcp_fast(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Sum over the 32 lanes of a warp in fp64, xor-shuffle tree (the same order on every lane).
__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// sum_{c < n} p[c * stride] in fp64: four interleaved chains (c = 0,4,8,.. / 1,5,.. / ...) so that the
// loads overlap, joined in a fixed order.  Used wherever the mean-pool's per-chunk sums are added.
__device__ __forceinline__ double sum_strided_f64(const float* __restrict__ p, int64_t stride, int n) {
  double t[4] = {0.0, 0.0, 0.0, 0.0};
  int c = 0;
  for (; c + 16 <= n; c += 16) {   // sixteen loads in flight; same chains, same order as the 4-wide loop below
    float v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) v[u] = __ldg(p + (int64_t)(c + u) * stride);
#pragma unroll
    for (int u = 0; u < 16; ++u) t[u & 3] += (double)v[u];
  }
  for (; c + 4 <= n; c += 4) {
#pragma unroll
    for (int u = 0; u < 4; ++u) t[u] += (double)__ldg(p + (int64_t)(c + u) * stride);
  }
  for (; c < n; ++c) t[0] += (double)__ldg(p + (int64_t)c * stride);
  return (t[0] + t[1]) + (t[2] + t[3]);
}

// Column sums of a [slots, W] fp32 array (W <= 20) by a CTA of 256 threads: thread t adds rows
// t, t+256, ... (all loads issued before any use), a xor-shuffle tree adds the lanes of each warp,
// and after the barrier sm[w][j] holds warp w's sum of column j; callers add the 8 warps in index
// order.  fp64 throughout; the order depends only on `slots`.
// FRESH: the rows were written by other CTAs of the SAME kernel (last-arriving-CTA finish), so they
// are read with ld.global.cg (L2, never a stale or non-coherent cache line).
template <bool FRESH = false>
__device__ __forceinline__ void block_column_sums_f64(const float* __restrict__ p, int64_t slots, int W,
                                                      double (*sm)[20]) {
  double a[20];
#pragma unroll
  for (int j = 0; j < 20; ++j) a[j] = 0.0;
  for (int64_t s = threadIdx.x; s < slots; s += 256) {
    const float* q = p + s * W;
#pragma unroll
    for (int j = 0; j < 20; ++j)
      if (j < W) a[j] += (double)(FRESH ? __ldcg(q + j) : __ldg(q + j));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < 20; ++j) {
    if (j < W) {
      const double t = warp_sum_f64(a[j]);
      if (lane == 0) sm[warp][j] = t;
    }
  }
  __syncthreads();
}

// Last-arriving-CTA detection for a group of `expected` CTAs that share the counter *ticket.
// Every CTA of the group calls this after its global writes; exactly one call (the one that
// arrives last) returns true, and by then the writes of all the others are visible to it (read
// them with ld.global.cg).  The counter must be 0 before the kernel starts and is 0 again when the
// kernel ends, so one zero-initialised buffer serves every launch on a stream.  Only an integer
// counter is contended: whatever the last CTA then sums, it sums in a fixed order.
// All threads of the CTA must call this (it contains barriers).
__device__ __forceinline__ bool cta_arrives_last(int* ticket, int expected) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(ticket, 1);
    s_last = (old == expected - 1) ? 1 : 0;
    if (s_last) *ticket = 0;
  }
  __syncthreads();
  const bool last = s_last != 0;
  if (last) __threadfence();
  return last;
}

// The same sums in the same order (thread t adds rows t, t + 256, ... one after the other in fp64)
// for a compile-time W that is a multiple of 4: rows are read as 16-byte vectors, several rows of
// loads in flight before the first add (two rows of 20 or eight rows of 4), which is what bounds the single CTA that finishes a batch
// element's partial sums while the rest of the GPU waits.  Falls back to 4-byte loads when the
// array is not 16-byte aligned.
template <int W, bool FRESH>
__device__ __forceinline__ void block_column_sums_fast(const float* __restrict__ p, int64_t slots, double (*sm)[20]) {
  static_assert(W % 4 == 0 && W <= 20, "row width");
  double a[W];
#pragma unroll
  for (int j = 0; j < W; ++j) a[j] = 0.0;
  const bool vec = (reinterpret_cast<uintptr_t>(p) & 15u) == 0;   // row pitch W * 4 bytes is a multiple of 16
  constexpr int kRows = W > 8 ? 2 : 8;   // rows in flight per thread: 40 or 32 values
  for (int64_t s0 = threadIdx.x; s0 < slots; s0 += 256 * kRows) {
    float v[kRows][W];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int64_t s = s0 + (int64_t)r * 256;
      if (s < slots) {
        const float* q = p + s * W;
        if (vec) {
#pragma unroll
          for (int j = 0; j < W; j += 4) {
            const float4 t = FRESH ? __ldcg(reinterpret_cast<const float4*>(q + j))
                                   : __ldg(reinterpret_cast<const float4*>(q + j));
            v[r][j] = t.x; v[r][j + 1] = t.y; v[r][j + 2] = t.z; v[r][j + 3] = t.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < W; ++j) v[r][j] = FRESH ? __ldcg(q + j) : __ldg(q + j);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r)
      if (s0 + (int64_t)r * 256 < slots) {
#pragma unroll
        for (int j = 0; j < W; ++j) a[j] += (double)v[r][j];
      }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < W; ++j) {
    const double t = warp_sum_f64(a[j]);
    if (lane == 0) sm[warp][j] = t;
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------
// One Sinkhorn-Knopp iteration on a register-resident 4x4 matrix (row-major m[16]):
// divide rows by (row sum + eps), then columns by (column sum + eps).  Optionally hands back the
// sums and the row-normalised matrix, which the backward needs.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void sinkhorn_step(float (&m)[16], float eps, float (&r)[4], float (&mr)[16],
                                              float (&c)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    r[i] = ((m[4 * i] + m[4 * i + 1]) + m[4 * i + 2]) + m[4 * i + 3] + eps;
    const float inv = rcp_fast(r[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) mr[4 * i + j] = m[4 * i + j] * inv;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    c[j] = ((mr[j] + mr[4 + j]) + mr[8 + j]) + mr[12 + j] + eps;
    const float inv = rcp_fast(c[j]);
#pragma unroll
    for (int i = 0; i < 4; ++i) m[4 * i + j] = mr[4 * i + j] * inv;
  }
}

__device__ __forceinline__ void sinkhorn_step(float (&m)[16], float eps) {
  float r[4], c[4], mr[16];
  sinkhorn_step(m, eps, r, mr, c);
}

// Pull a gradient d (on the output of one iteration) back to the iteration's input.
// For y = x / (sum(x) + eps) along an axis: dx = (dy - <dy, y>) / (sum(x) + eps).
__device__ __forceinline__ void sinkhorn_step_bwd(float (&d)[16], const float (&m_out)[16], const float (&r)[4],
                                                  const float (&mr)[16], const float (&c)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float dot = ((d[j] * m_out[j] + d[4 + j] * m_out[4 + j]) + d[8 + j] * m_out[8 + j]) +
                      d[12 + j] * m_out[12 + j];
    const float inv = rcp_fast(c[j]);
#pragma unroll
    for (int i = 0; i < 4; ++i) d[4 * i + j] = (d[4 * i + j] - dot) * inv;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float dot = ((d[4 * i] * mr[4 * i] + d[4 * i + 1] * mr[4 * i + 1]) + d[4 * i + 2] * mr[4 * i + 2]) +
                      d[4 * i + 3] * mr[4 * i + 3];
    const float inv = rcp_fast(r[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) d[4 * i + j] = (d[4 * i + j] - dot) * inv;
  }
}

// Gradient d (with respect to the output of `iters` Sinkhorn iterations started from |m0| + eps) pulled
// back to the start matrix, in place, with no stored states: the iterations are cut into kSinkhornCk + 1
// segments of L = ceil(iters / (kSinkhornCk + 1)); one forward sweep keeps the state entering each segment
// in registers, and the state entering iteration t is then recomputed from its segment's checkpoint (at
// most L - 1 steps) instead of from m0 (t steps).  The recomputation runs the same step function
// from the same values, so the result is bit-identical to recomputing from m0 every time, for about
// iters * (L + 3) / 2 steps instead of iters * (iters + 1) / 2.  The sign of m0 is NOT applied.
constexpr int kSinkhornCk = 4;
__device__ __forceinline__ void sinkhorn_backward_ck(const float (&m0)[16], float (&d)[16], int iters, float eps) {
  const int L = (iters + kSinkhornCk) / (kSinkhornCk + 1);
  float ck[kSinkhornCk][16];
  {
    float m[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) m[k] = fabsf(m0[k]) + eps;
#pragma unroll
    for (int k = 0; k < kSinkhornCk; ++k) {
      const int t1 = min((k + 1) * L, iters);
      for (int t = k * L; t < t1; ++t) sinkhorn_step(m, eps);
#pragma unroll
      for (int e = 0; e < 16; ++e) ck[k][e] = m[e];  // state entering iteration (k + 1) * L
    }
  }
#pragma unroll
  for (int k = kSinkhornCk; k >= 0; --k) {
    const int t0 = k * L, t1 = min((k + 1) * L, iters);
    for (int t = t1 - 1; t >= t0; --t) {
      float m[16], r[4], c[4], mr[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) m[e] = k == 0 ? fabsf(m0[e]) + eps : ck[k == 0 ? 0 : k - 1][e];
      for (int f = t0; f < t; ++f) sinkhorn_step(m, eps);
      sinkhorn_step(m, eps, r, mr, c);
      sinkhorn_step_bwd(d, m, r, mr, c);
    }
  }
}

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }

}  // namespace mhc

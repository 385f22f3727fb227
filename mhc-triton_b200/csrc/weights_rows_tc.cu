// Dynamic weights for many rows (per-token use: x [rows, K] fp32) on the fifth-generation tensor
// cores: the projection x * phi runs as tcgen05.mma kind::tf32 with the accumulator in tensor
// memory, x and phi tiles arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle), and the whole
// finish of a row (RMS norm, scale + bias, sigmoids, register Sinkhorn) is the kernel's epilogue,
// so one kernel goes from x to (H_pre, H_post, H_res, saved).
//
// fp32 parity needs more than one TF32 product: x = hi + lo and phi = hi + lo (each half rounded to
// TF32), and x * phi = hi*hi + hi*lo + lo*hi (+ lo*lo, which comes for free here).  The tensor core reads its B operand from shared
// memory and its A operand from shared OR tensor memory; splitting x inside shared memory would
// triple the shared-memory traffic of an HBM-bound kernel, so the rows take the tensor-memory road:
//
//   warp 4 (two lanes)  TMA producers: x tiles [128 rows x 32 k] through a ring of five stages (a stage is
//                       free again as soon as the row threads hold it in registers) and the pre-split
//                       phi^T tiles (hi, lo) [32 outputs x 32 k] through a ring of three (free when their
//                       MMAs are done).
//   warps 0-3           thread t owns row t: reads its 128 bytes of the x tile from shared memory,
//                       splits them into hi / lo in registers, adds up x^2, and writes both halves to
//                       tensor memory (tcgen05.st), lane t, as the A operand [128 x 32].
//   warp 5 (one lane)   issues 4 k-steps x 2 products of tcgen05.mma (M 128, N 64, K 8) per tile: x_hi and
//                       x_lo, each against [phi_hi | phi_lo] side by side, into one of two accumulators
//                       [128 x 64] in tensor memory (the two halves are added when drained), then tcgen05.commit.
//   warps 0-3 again     drain the accumulator of the previous tile (tcgen05.ld) into fp32 registers:
//                       the tensor core starts every 32-deep tile from zero and the running sums are
//                       ordinary round-to-nearest fp32 adds, which keeps its truncating adds out of
//                       the long sum over K.
//
// phi^T (hi, lo), padded to 32 outputs and to a multiple of 32 in K, is produced once per call by a
// small kernel into caller scratch.  Every mbarrier wait is bounded (about a second); a wait that
// runs out sets the status word in the scratch, the affected rows are filled with NaN, tensor
// memory is released and the kernel returns.  No TMA multicast, no clusters, this GPU's memory only.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "launch.h"

// Build with -DMHC_TC_TIMING to make one thread of each role of CTA 0 add up the cycles it spends in each phase
// of its loop into the scratch header (ints 8.. of the status block); a development aid, off by default.
#ifdef MHC_TC_TIMING
#define TC_TIMING_DECL(n) long long tc_t_[n] = {}; long long tc_last_ = clock64(); const bool tc_on_ = blockIdx.x == 0 && blockIdx.y == 0
#define TC_T(i) do { if (tc_on_) { const long long now_ = clock64(); tc_t_[i] += now_ - tc_last_; tc_last_ = now_; } } while (0)
#define TC_TIMING_FLUSH(status, off, n) do { if (tc_on_) for (int i_ = 0; i_ < (n); ++i_) (status)[8 + (off) + i_] = (int)(tc_t_[i_] >> 4); } while (0)
#else
#define TC_TIMING_DECL(n)
#define TC_T(i)
#define TC_TIMING_FLUSH(status, off, n)
#endif

// L2 promotion of the x tensor maps.  The backward's x loads gain 3.6 % from 256-byte promotion (813 -> 785 us at
// 32768 x 16384); the forward's do not change (426 / 424 / 427 us for 128 bytes / 256 bytes / none).
#ifndef MHC_TC_FWD_X_PROMO
#define MHC_TC_FWD_X_PROMO CU_TENSOR_MAP_L2_PROMOTION_L2_128B
#endif
#ifndef MHC_TC_BWD_X_PROMO
#define MHC_TC_BWD_X_PROMO CU_TENSOR_MAP_L2_PROMOTION_L2_256B
#endif

namespace mhc {
namespace tc {

constexpr int kBM = 128;   // rows per CTA = lanes of tensor memory
constexpr int kBK = 32;    // k per tile: 128 bytes of fp32, one swizzle span
constexpr int kBN = 32;    // the 24 outputs, padded
// Two rings of shared-memory stages: x tiles (free again as soon as the row threads hold them in
// registers) and phi tiles (free when their MMAs are done).  A TMA load takes 3000-4000 cycles to land, so
// what counts is the x in flight per SM: 2 CTAs x 5 stages x 16 KiB.
constexpr int kXStages = 5, kPStages = 3;
constexpr uint32_t kXBytes = kBM * kBK * 4;          // 16 KiB
constexpr uint32_t kPBytes = kBN * kBK * 4;          // 4 KiB
constexpr uint32_t kPStageBytes = 2 * kPBytes;       // phi_hi, phi_lo back to back
constexpr uint32_t kOffP = kXStages * kXBytes;
constexpr uint32_t kTmemCols = 256;                  // A: 2 buffers x (32 hi + 32 lo); D: 2 x 64  (two CTAs per SM)
constexpr uint32_t kColA = 0, kColD = 128;
constexpr int kDCols = 64;                           // an accumulator holds A * [phi_hi | phi_lo]
constexpr int kThreads = 192;
constexpr size_t kSmemBytes = 1024 + kXStages * kXBytes + kPStages * kPStageBytes + 256;
constexpr long long kWaitCycles = 2000000000LL;      // about one second

// status word values (first int of the scratch): which wait ran out
enum { kOk = 0, kErrFull = 1001, kErrAReady = 1002, kErrStageFree = 1003, kErrDFull = 1004, kErrDEmpty = 1005, kErrXReleased = 1006,
       kErrPFull = 1007 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One arrival per WARP (barriers that count warps are initialised with the number of warps): the
// lanes' earlier writes and tensor-memory operations are ordered before lane 0's arrive by the warp
// barrier.  128 single-thread arrivals per tile on one shared-memory word cost more than the tile's math.
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the barrier did not complete within kWaitCycles (the status
// word and the CTA's abort flag are then set) or when another thread of the CTA has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 31u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// The same for a whole warp waiting on one barrier: the answer is made warp-uniform, so that the lanes of a
// warp never part ways at a wait that ran out (they arrive on barriers together, see mbar_arrive_warp).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  const bool ok = mbar_wait(bar, parity, abort_flag, status, code);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[128 x N] (+)= A[128 x 8] (tensor memory) * B[N x 8]^T (shared memory, K-major), TF32 inputs, fp32 sums.
// One such instruction occupies the tensor core for roughly 85 cycles whether N is 32 or 64 (measured),
// so the kernels below concatenate the hi and lo halves of B along N and issue two products per k-step
// instead of three.
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (32 fp32) under the
// 128-byte swizzle: 8-row groups are 1024 bytes apart; the leading-dimension offset is not used in
// this mode.  Bits: [0,14) address >> 4, [16,30) leading offset >> 4, [32,46) stride offset >> 4,
// [46,48) descriptor version 1, [61,64) layout 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor: fp32 accumulator (bits [4,6) = 1), A and B TF32 (bits [7,10) = [10,13) = 2),
// both K-major (bits 15, 16 = 0), N >> 3 in bits [17,23), M >> 4 in bits [24,29).
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
constexpr uint32_t kIdescN64 = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

#define MHC_R32(a) a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], a[9], a[10], a[11], a[12], a[13], a[14], a[15], \
                   a[16], a[17], a[18], a[19], a[20], a[21], a[22], a[23], a[24], a[25], a[26], a[27], a[28], a[29], a[30], a[31]

// 32 consecutive columns of this thread's lane: registers -> tensor memory.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
// tensor memory -> registers, same shape.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Round-to-nearest split of an fp32 value into two TF32 values: v ~ hi + lo.
__device__ __forceinline__ uint32_t tf32_rn(float v) { return (__float_as_uint(v) + 0x1000u) & 0xFFFFE000u; }

// phiT_hi / phiT_lo [32, Kp] from phi [K, 24]: rows 24..31 and columns K..Kp-1 are zero.  Also clears
// the status word.
__global__ void __launch_bounds__(256)
k_phi_split_t(const float* __restrict__ phi, float* __restrict__ hi, float* __restrict__ lo, int64_t K, int64_t Kp,
              int* __restrict__ status) {
  pdl_prologue();
  if (blockIdx.x == 0 && threadIdx.x == 0) *status = kOk;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // index into [32, Kp]
  if (i >= 32 * Kp) return;
  const int64_t j = i / Kp, k = i - j * Kp;
  float h = 0.f, l = 0.f;
  if (j < 24 && k < K) {
    const float v = __ldg(phi + k * 24 + j);
    h = __uint_as_float(tf32_rn(v));
    l = __uint_as_float(tf32_rn(v - h));
  }
  hi[i] = h;
  lo[i] = l;
}

struct RowsFinish {
  BiasPtrs bias;
  const float *alpha_pre, *alpha_post, *alpha_res;
  float *H_pre, *H_post, *H_res, *saved;
  int iters;
  float eps;
};

__global__ void __launch_bounds__(kThreads, 2)
k_dw_rows_fwd_tc(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_phi_hi,
                 const __grid_constant__ CUtensorMap map_phi_lo, RowsFinish fin, int64_t rows, int64_t K, int* status) {
  pdl_prologue();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // tiles need 1024-byte alignment for the swizzle
  const uint32_t bars = base + kOffP + kPStages * kPStageBytes;
  // barriers: x_full[X] x_free[X] p_full[P] p_free[P] a_ready[2] d_full[2] d_empty[2]
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_xfree = [&](int s) { return bars + 8u * (kXStages + s); };
  auto bar_pfull = [&](int s) { return bars + 8u * (2 * kXStages + s); };
  auto bar_free = [&](int s) { return bars + 8u * (2 * kXStages + kPStages + s); };
  auto bar_aready = [&](int a) { return bars + 8u * (2 * kXStages + 2 * kPStages + a); };
  auto bar_dfull = [&](int d) { return bars + 8u * (2 * kXStages + 2 * kPStages + 2 + d); };
  auto bar_dempty = [&](int d) { return bars + 8u * (2 * kXStages + 2 * kPStages + 4 + d); };
  const uint32_t holder = bars + 8u * (2 * kXStages + 2 * kPStages + 6);
  __shared__ int s_abort;
  volatile int* abort_flag = &s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row0 = (int64_t)blockIdx.x * kBM;
  const int nk = (int)((K + kBK - 1) / kBK);

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kXStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_xfree(s), kBM / 32);
    }
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(bar_pfull(s), 1);
      mbar_init(bar_free(s), 1);
    }
    for (int d = 0; d < 2; ++d) {
      mbar_init(bar_aready(d), kBM / 32);
      mbar_init(bar_dfull(d), 1);
      mbar_init(bar_dempty(d), kBM / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) tmem_alloc(holder, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(holder) : "memory");

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producers: lane 0 x, lane 1 phi
    if (lane == 0) {
      TC_TIMING_DECL(3);
      for (int i = 0; i < nk; ++i) {
        const int s = i % kXStages;
        if (i >= kXStages && !mbar_wait(bar_xfree(s), ((i / kXStages) - 1) & 1, abort_flag, status, kErrXReleased)) break;
        TC_T(0);
        mbar_expect_tx(bar_full(s), kXBytes);
        tma_load_2d(base + s * kXBytes, &map_x, i * kBK, (int)row0, bar_full(s));
        TC_T(2);
      }
      TC_TIMING_FLUSH(status, 0, 3);
    } else if (lane == 1) {
      for (int i = 0; i < nk; ++i) {
        const int s = i % kPStages;
        if (i >= kPStages && !mbar_wait(bar_free(s), ((i / kPStages) - 1) & 1, abort_flag, status, kErrStageFree)) break;
        const uint32_t dst = base + kOffP + s * kPStageBytes;
        mbar_expect_tx(bar_pfull(s), kPStageBytes);
        tma_load_2d(dst, &map_phi_hi, i * kBK, 0, bar_pfull(s));
        tma_load_2d(dst + kPBytes, &map_phi_lo, i * kBK, 0, bar_pfull(s));
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      TC_TIMING_DECL(4);
      for (int i = 0; i < nk; ++i) {
        const int s = i % kPStages, d = i & 1;   // d: the A buffer and the accumulator of this tile
        if (!mbar_wait(bar_pfull(s), (i / kPStages) & 1, abort_flag, status, kErrPFull)) break;
        TC_T(0);
        if (!mbar_wait(bar_aready(d), (i >> 1) & 1, abort_flag, status, kErrAReady)) break;
        TC_T(1);
        if (i >= 2 && !mbar_wait(bar_dempty(d), ((i >> 1) - 1) & 1, abort_flag, status, kErrDEmpty)) break;
        TC_T(2);
        tc_fence_after();
        // phi_hi (32 rows) and phi_lo (32 rows) lie back to back: one K-major tile of 64 rows
        const uint64_t b_cat = make_kmajor_sw128_desc(base + kOffP + s * kPStageBytes);
        const uint32_t a_hi = tmem_base + kColA + d * 64, a_lo = a_hi + 32, dd = tmem_base + kColD + d * kDCols;
#pragma unroll
        for (int j = 0; j < kBK / 8; ++j) {   // a k-step of 8 is 32 bytes of a swizzled row: descriptor address + 2
          mma_tf32_ts(dd, a_hi + 8 * j, b_cat + 2 * j, kIdescN64, j > 0);   // columns 0..31: hi*hi, 32..63: hi*lo
          mma_tf32_ts(dd, a_lo + 8 * j, b_cat + 2 * j, kIdescN64, 1);       //                lo*hi,          lo*lo
        }
        tc_commit(bar_free(s));    // the phi tiles of stage s may be overwritten
        tc_commit(bar_dfull(d));   // accumulator d holds this tile's sums (and A buffer d has been read)
        TC_T(3);
      }
      TC_TIMING_FLUSH(status, 4, 4);
    }
  } else {
    // ------------------------------------------------------------------ rows: split, accumulate, finish
    const int t = threadIdx.x;                   // row within the tile = lane of tensor memory
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float acc[24];
#pragma unroll
    for (int j = 0; j < 24; ++j) acc[j] = 0.f;
    float q = 0.f;
    bool ok = true;
    TC_TIMING_DECL(8);
    auto drain = [&](int i) {   // add tile i's accumulator to the running sums
      const int d = i & 1;
      if (!mbar_wait_warp(bar_dfull(d), (i >> 1) & 1, abort_flag, status, kErrDFull)) return false;
      TC_T(4);
      tc_fence_after();
      uint32_t v[32], w[32];
      tmem_ld32(tmem_base + lane_addr + kColD + d * kDCols, v);          // the x * phi_hi terms
      tmem_ld32(tmem_base + lane_addr + kColD + d * kDCols + 32, w);     // the x * phi_lo terms
      tmem_wait_ld();
      TC_T(5);
#pragma unroll
      for (int j = 0; j < 24; ++j) acc[j] += __uint_as_float(v[j]) + __uint_as_float(w[j]);
      tc_fence_before();
      mbar_arrive_warp(bar_dempty(d));
      TC_T(6);
      return true;
    };
    for (int i = 0; i < nk && ok; ++i) {
      const int s = i % kXStages;
      if (!mbar_wait_warp(bar_full(s), (i / kXStages) & 1, abort_flag, status, kErrFull)) { ok = false; break; }
      TC_T(0);
      const uint32_t rowp = base + s * kXBytes + (uint32_t)t * 128u;
      uint32_t hi[32], lo[32];
      float qt = 0.f;
      float4 xr[8];
#pragma unroll
      for (int c = 0; c < 8; ++c)   // 16-byte chunk c of row t sits at chunk position c ^ (t & 7); all loads first
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(xr[c].x), "=f"(xr[c].y), "=f"(xr[c].z), "=f"(xr[c].w)
                     : "r"(rowp + (uint32_t)((c ^ (t & 7)) << 4))
                     : "memory");
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float e[4] = {xr[c].x, xr[c].y, xr[c].z, xr[c].w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t h = tf32_rn(e[u]);
          hi[4 * c + u] = h;
          lo[4 * c + u] = tf32_rn(e[u] - __uint_as_float(h));
          qt = fmaf(e[u], e[u], qt);
        }
      }
      q += qt;
      TC_T(1);
      mbar_arrive_warp(bar_xfree(s));   // the tile is in registers
      // A buffer i & 1 was last read by the MMAs of tile i - 2, whose accumulator this thread has already drained
      const uint32_t a_hi = tmem_base + lane_addr + kColA + (i & 1) * 64;
      tmem_st32(a_hi, hi);
      tmem_st32(a_hi + 32, lo);
      tmem_wait_st();
      TC_T(2);
      tc_fence_before();
      mbar_arrive_warp(bar_aready(i & 1));
      TC_T(3);
      // (collecting tile i - 1's sums before the stores above was tried: the products then start later and
      // the wait here only grows)
      if (i >= 1) ok = drain(i - 1);
    }
    if (ok && nk > 0) ok = drain(nk - 1);
    TC_TIMING_FLUSH(status, 8, 7);
    const int64_t row = row0 + t;
    if (row < rows) {
      const float nanv = __int_as_float(0x7fc00000);
      if (!ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) { fin.H_pre[row * 4 + j] = nanv; fin.H_post[row * 4 + j] = nanv; }
#pragma unroll
        for (int j = 0; j < 16; ++j) fin.H_res[row * 16 + j] = nanv;
      } else {
        // the finish of one row, thread-resident (same formulas and orders as the warp-per-row finish)
        const float eps = fin.eps;
        const float inv_rms = 1.f / sqrtf(q / (float)K + eps);
        const float a_pre = __ldg(fin.alpha_pre), a_post = __ldg(fin.alpha_post), a_res = __ldg(fin.alpha_res);
        float sc[24];
#pragma unroll
        for (int j = 0; j < 24; ++j) {
          const float al = j < 4 ? a_pre : (j < 8 ? a_post : a_res);
          const float b = j < 4 ? __ldg(fin.bias.pre + j) : (j < 8 ? __ldg(fin.bias.post + j - 4) : __ldg(fin.bias.res + j - 8));
          sc[j] = (inv_rms * al) * acc[j] + b;
        }
        if (fin.saved) {
          float* sv = fin.saved + row * kSavedStride;
#pragma unroll
          for (int j = 0; j < 24; ++j) sv[j] = acc[j];
          sv[24] = q;
          sv[25] = inv_rms;
        }
        float sg[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) sg[j] = sigmoidf_(sc[j]);
        const float ssum = (((sg[0] + sg[1]) + sg[2]) + sg[3]) + eps;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          fin.H_pre[row * 4 + j] = sg[j] / ssum;
          fin.H_post[row * 4 + j] = 2.f * sg[4 + j];
        }
        float m[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) m[j] = fabsf(sc[8 + j]) + eps;
        for (int it = 0; it < fin.iters; ++it) sinkhorn_step(m, eps);
#pragma unroll
        for (int j = 0; j < 16; ++j) fin.H_res[row * 16 + j] = m[j];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ======================================================================================
// Backward pass over x:  grad_x[r,k] = sum_j d_raw[r,j] phi[k,j] + coef[r] x[r,k]   and the per-group
// partial sums of  grad_phi[k,j] = sum_r x[r,k] d_raw[r,j],  reading x once.
//
// One CTA owns a slab of 128 k and walks a group of rows in sub-tiles of 128 rows.  Both products
// run on tcgen05 with 3xTF32 splits:
//   product 1 (grad_x):   A = d_raw hi/lo [128 rows x 32 j] in tensor memory, B = the slab of phi hi/lo
//                         [128 k x 32 j] in shared memory (loaded once per CTA), D1 [128 rows x 128 k].
//   product 2 (grad_phi): A = x^T hi/lo [128 k x 64 rows] per half sub-tile in tensor memory (thread t of
//                         warps 4-7 owns k = t: it reads its column of the x tile from shared memory,
//                         splits it and writes lane t), B = [d_raw^T hi | d_raw^T lo] (N = 64) written to
//                         shared memory by the row threads in the swizzled K-major layout, D2 [128 k x 64]
//                         per sub-tile (two products per k-step instead of three), drained into fp32
//                         registers after every sub-tile.
//   warps 0-3 (row threads)     d_raw of their row (fetched one sub-tile ahead) -> A of product 1 and B of product 2.
//   warps 4-7 (column threads)  x^T halves -> tensor memory; running sums of grad_phi.
//   warps 10-13 (epilogue)      thread = row: D1 + coef * x written over the x tile in place.
//   warp 8 (one lane)           TMA: phi slab once, x sub-tiles (two stages of 64 KiB), and the stores of the
//                               finished grad_x tiles; a stage is reloaded as soon as its store has read it.
//   warp 9 (one lane)           all tcgen05.mma and tcgen05.commit.
// Tensor memory: A1 64 + D1 128 + A2 2 x 128 + D2 64 = 512 columns (one CTA per SM).
// ======================================================================================
namespace bw {
constexpr int kSlab = 128;                         // k per CTA
constexpr uint32_t kXStage = 4 * kXBytes;          // 64 KiB: four [128 rows x 32 k] tiles
constexpr uint32_t kOffB1 = 2 * kXStage;           // phi slab hi, lo: 2 x 16 KiB
constexpr uint32_t kB1Bytes = kSlab * 32 * 4;
constexpr uint32_t kOffB2 = kOffB1 + 2 * kB1Bytes; // d_raw^T: 4 blocks (32 rows of x each) of [hi 32 j-rows | lo 32 j-rows] x 128 bytes
constexpr uint32_t kB2Bytes = 32 * 128 * 4;
constexpr uint32_t kOffBars = kOffB2 + 2 * kB2Bytes;
constexpr size_t kSmem = 1024 + kOffBars + 512;
constexpr int kThreadsBwd = 448;
constexpr uint32_t kColA1 = 0, kColD1 = 64, kColA2 = 192, kColD2 = 448;   // A2 half h at kColA2 + 128 h (hi 64, lo 64); D2 64
constexpr uint32_t kIdescN128 = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
enum { kErrPhi = 2001, kErrXFull = 2002, kErrStore = 2003, kErrXRead = 2004, kErrA1 = 2005, kErrAbFree = 2006,
       kErrA2Ready = 2007, kErrA2Free = 2008, kErrD1Full = 2009, kErrD1Empty = 2010, kErrD2Full = 2011, kErrD2Empty = 2012,
       kErrB2 = 2013 };
}  // namespace bw

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// phi_hi / phi_lo [Kp, 32] from phi [K, 24] (columns 24..31 and rows K..Kp-1 zero); clears the status word.
__global__ void __launch_bounds__(256)
k_phi_split_rows(const float* __restrict__ phi, float* __restrict__ hi, float* __restrict__ lo, int64_t K, int64_t Kp,
                 int* __restrict__ status) {
  pdl_prologue();
  if (blockIdx.x == 0 && threadIdx.x == 0) *status = kOk;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 32 * Kp) return;
  const int64_t k = i >> 5;
  const int j = (int)(i & 31);
  float h = 0.f, l = 0.f;
  if (j < 24 && k < K) {
    const float v = __ldg(phi + k * 24 + j);
    h = __uint_as_float(tf32_rn(v));
    l = __uint_as_float(tf32_rn(v - h));
  }
  hi[i] = h;
  lo[i] = l;
}

__global__ void __launch_bounds__(bw::kThreadsBwd, 1)
k_dw_rows_bwd_tc(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_gx,
                 const __grid_constant__ CUtensorMap map_phi_hi, const __grid_constant__ CUtensorMap map_phi_lo,
                 const float* __restrict__ buf, float* __restrict__ phi_part, int64_t rows, int64_t K,
                 int64_t rows_per_group, int* status) {
  using namespace bw;
  pdl_prologue();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + kOffBars;
  // barriers (8 bytes each).  The x tile of a sub-tile is four quarters [128 rows x 32 k] of 16 KiB, each with
  // its own load / read / store barriers (buffer q = 4 * (sub-tile & 1) + quarter), so that loading, splitting,
  // the epilogue and the store of different quarters overlap.
  const uint32_t b_phi = bars;
  auto b_xfull = [&](int q) { return bars + 8u * (1 + q); };     // TMA has filled quarter buffer q
  auto b_store = [&](int q) { return bars + 8u * (9 + q); };     // the epilogue warps (4) have written grad_x over it
  auto b_xread = [&](int q) { return bars + 8u * (17 + q); };    // the column warp of this quarter has read it
  const uint32_t b_a1 = bars + 8u * 25, b_b2free = bars + 8u * 26;   // A1 written / the products have read d_raw^T
  auto b_a2ready = [&](int h) { return bars + 8u * (27 + h); };
  auto b_a2free = [&](int h) { return bars + 8u * (29 + h); };
  const uint32_t b_d1full = bars + 8u * 31, b_d1empty = bars + 8u * 32;
  const uint32_t b_d2full = bars + 8u * 33, b_d2empty = bars + 8u * 34;
  const uint32_t b_a1free = bars + 8u * 35, b_b2 = bars + 8u * 36;   // product 1 has read A1 / d_raw^T written
  const uint32_t holder = bars + 8u * 38;
  __shared__ int s_abort;
  volatile int* abort_flag = &s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t k0 = (int64_t)blockIdx.x * kSlab;
  const int64_t g0 = (int64_t)blockIdx.y * rows_per_group;
  const int64_t g1 = min(g0 + rows_per_group, rows);
  const int nsub = (int)((g1 - g0 + kBM - 1) / kBM);

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(b_phi, 1);
    for (int q = 0; q < 8; ++q) {
      mbar_init(b_xfull(q), 1);
      mbar_init(b_store(q), 4);
      mbar_init(b_xread(q), 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(b_a2ready(h), 4);
      mbar_init(b_a2free(h), 1);
    }
    mbar_init(b_a1, 4);
    mbar_init(b_b2, 4);
    mbar_init(b_a1free, 1);
    mbar_init(b_b2free, 1);
    mbar_init(b_d1full, 1);
    mbar_init(b_d1empty, 4);
    mbar_init(b_d2full, 1);
    mbar_init(b_d2empty, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) tmem_alloc(holder, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(holder) : "memory");

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA: loads, and the stores of grad_x
    if (lane == 0) {
      TC_TIMING_DECL(4);
      auto load_q = [&](int it, int kk) {
        const int q = 4 * (it & 1) + kk;
        mbar_expect_tx(b_xfull(q), kXBytes);
        tma_load_2d(base + q * kXBytes, &map_x, (int)k0 + 32 * kk, (int)(g0 + (int64_t)it * kBM), b_xfull(q));
      };
      mbar_expect_tx(b_phi, 2 * kB1Bytes);
      tma_load_2d(base + kOffB1, &map_phi_hi, 0, (int)k0, b_phi);
      tma_load_2d(base + kOffB1 + kB1Bytes, &map_phi_lo, 0, (int)k0, b_phi);
      for (int it = 0; it < 2 && it < nsub; ++it)
        for (int kk = 0; kk < 4; ++kk) load_q(it, kk);
      int prev_it = -1, prev_kk = 0;
      bool ok = true;
      for (int it = 0; it < nsub && ok; ++it) {
        for (int kk = 0; kk < 4; ++kk) {
          const int q = 4 * (it & 1) + kk;
          TC_T(3);
          if (!mbar_wait(b_store(q), (it >> 1) & 1, abort_flag, status, kErrStore)) { ok = false; break; }
          TC_T(0);
          tma_store_2d(&map_gx, (int)k0 + 32 * kk, (int)(g0 + (int64_t)it * kBM), base + q * kXBytes);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          TC_T(1);
          // the quarter stored one step earlier has been read out by now (all groups but the newest): refill it
          if (prev_it >= 0 && prev_it + 2 < nsub) {
            asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            load_q(prev_it + 2, prev_kk);
          }
          prev_it = it;
          prev_kk = kk;
          TC_T(2);
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      TC_TIMING_FLUSH(status, 24, 4);
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      TC_TIMING_DECL(8);
      bool ok = mbar_wait(b_phi, 0, abort_flag, status, kErrPhi);
      const uint64_t b1_hi = make_kmajor_sw128_desc(base + kOffB1), b1_lo = make_kmajor_sw128_desc(base + kOffB1 + kB1Bytes);
      for (int it = 0; it < nsub && ok; ++it) {
        const uint32_t ph = it & 1;
        TC_T(7);
        if (!mbar_wait(b_a1, ph, abort_flag, status, kErrA1)) break;
        TC_T(0);
        if (it >= 1 && !mbar_wait(b_d1empty, (it - 1) & 1, abort_flag, status, kErrD1Empty)) break;
        TC_T(1);
        tc_fence_after();
        const uint32_t a1_hi = tmem_base + kColA1, a1_lo = a1_hi + 32, d1 = tmem_base + kColD1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {   // product 1: K = 32 (24 used) in steps of 8
          mma_tf32_ts(d1, a1_hi + 8 * j, b1_hi + 2 * j, kIdescN128, j > 0);
          mma_tf32_ts(d1, a1_hi + 8 * j, b1_lo + 2 * j, kIdescN128, 1);
          mma_tf32_ts(d1, a1_lo + 8 * j, b1_hi + 2 * j, kIdescN128, 1);
        }
        tc_commit(b_d1full);
        tc_commit(b_a1free);       // the row threads may write the next sub-tile's A1 while product 2 runs
        TC_T(2);
        if (!mbar_wait(b_b2, ph, abort_flag, status, kErrB2)) break;
        const uint32_t d2 = tmem_base + kColD2;
        for (int h = 0; h < 2 && ok; ++h) {
          if (!mbar_wait(b_a2ready(h), ph, abort_flag, status, kErrA2Ready)) { ok = false; break; }
          TC_T(3);
          if (h == 0 && it >= 1 && !mbar_wait(b_d2empty, (it - 1) & 1, abort_flag, status, kErrD2Empty)) { ok = false; break; }
          TC_T(4);
          tc_fence_after();
          const uint32_t a2_hi = tmem_base + kColA2 + 128 * h, a2_lo = a2_hi + 64;
#pragma unroll
          for (int j = 0; j < 8; ++j) {   // product 2: K = 64 rows of this half in steps of 8, B = [d_hi | d_lo] (N = 64)
            const int r = 64 * h + 8 * j;                         // first row of the step
            const uint64_t b2 = make_kmajor_sw128_desc(base + kOffB2 + (uint32_t)(r >> 5) * 8192u + (uint32_t)(r & 31) * 4u);
            mma_tf32_ts(d2, a2_hi + 8 * j, b2, kIdescN64, (h | j) > 0);
            mma_tf32_ts(d2, a2_lo + 8 * j, b2, kIdescN64, 1);
          }
          tc_commit(b_a2free(h));
          TC_T(5);
        }
        if (ok) {
          tc_commit(b_d2full);
          tc_commit(b_b2free);
        }
        TC_T(6);
      }
      TC_TIMING_FLUSH(status, 0, 8);
    }
  } else if (warp < 4) {
    // ---------------------------------------------------------------- row threads: operands from d_raw
    const int t = threadIdx.x;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    // rows j = 24..31 of both halves of d_raw^T stay zero for the whole kernel
    for (uint32_t i = t; i < 2 * kB2Bytes / 16; i += 128)
      asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(base + kOffB2 + i * 16), "r"(0u) : "memory");
    asm volatile("bar.sync 1, 128;" ::: "memory");
    TC_TIMING_DECL(8);
    // this row's d_raw (24 values), fetched one sub-tile ahead
    float4 dq[6];
    auto fetch = [&](int it) {
      const int64_t row = g0 + (int64_t)it * kBM + t;
      if (it < nsub && row < g1) {
        const float* q = buf + row * 56 + 24;   // 16-byte aligned: rows are 224 bytes, the offset 96
#pragma unroll
        for (int i = 0; i < 6; ++i) dq[i] = __ldg(reinterpret_cast<const float4*>(q) + i);
      } else {
#pragma unroll
        for (int i = 0; i < 6; ++i) dq[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    };
    fetch(0);
    bool good = true;
    for (int it = 0; it < nsub && good; ++it) {
      TC_T(7);
      if (it >= 1 && !mbar_wait_warp(b_a1free, (it - 1) & 1, abort_flag, status, kErrAbFree)) break;
      TC_T(0);
      uint32_t hi[32], lo[32];
#pragma unroll
      for (int i = 0; i < 6; ++i) {
        const float e[4] = {dq[i].x, dq[i].y, dq[i].z, dq[i].w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          hi[4 * i + u] = tf32_rn(e[u]);
          lo[4 * i + u] = tf32_rn(e[u] - __uint_as_float(hi[4 * i + u]));
        }
      }
#pragma unroll
      for (int j = 24; j < 32; ++j) { hi[j] = 0u; lo[j] = 0u; }
      tmem_st32(tmem_base + lane_addr + kColA1, hi);
      tmem_st32(tmem_base + lane_addr + kColA1 + 32, lo);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(b_a1);
      TC_T(6);
      // d_raw^T is still being read by product 2 of the previous sub-tile
      if (it >= 1 && !mbar_wait_warp(b_b2free, (it - 1) & 1, abort_flag, status, kErrAbFree)) break;
      TC_T(2);
      {
        // element (j, r = t) of block t / 32 = [hi: 32 j-rows x 128 bytes][lo: the same], 128-byte swizzle
        // (16-byte chunk index ^ (j & 7)): one K-major tile of 64 rows per block of 32 rows of x
        const uint32_t blk = base + kOffB2 + (uint32_t)(t >> 5) * 8192u + (uint32_t)(t & 3) * 4u;
        const uint32_t chunk = (uint32_t)(t & 31) >> 2;
#pragma unroll
        for (int j = 0; j < 24; ++j) {
          const uint32_t a = blk + (uint32_t)j * 128u + ((chunk ^ (uint32_t)(j & 7)) << 4);
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(hi[j]) : "memory");
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(a + 4096u), "r"(lo[j]) : "memory");
        }
      }
      fence_async_smem();
      mbar_arrive_warp(b_b2);
      fetch(it + 1);   // in flight while the products of this sub-tile run
      TC_T(1);
    }
    if (t == 0) TC_TIMING_FLUSH(status, 8, 8);
  } else if (warp >= 10) {
    // ---------------------------------------------------------------- epilogue threads (warps 10-13)
    // grad_x = D1 + coef * x, written over the x tile in place; the TMA warp stores it.  A warp reaches the
    // lanes 32 * (warp % 4) .. + 31 of tensor memory, and the lane is the row.
    const int t = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    TC_TIMING_DECL(8);
    auto coef_of = [&](int it) {
      const int64_t row = g0 + (int64_t)it * kBM + t;
      return (it < nsub && row < g1) ? __ldg(buf + row * 56 + 48) : 0.f;
    };
    float coef_next = coef_of(0);
    for (int it = 0; it < nsub; ++it) {
      const int s = it & 1;
      const float coef = coef_next;
      coef_next = coef_of(it + 1);
      TC_T(7);
      if (!mbar_wait_warp(b_d1full, it & 1, abort_flag, status, kErrD1Full)) break;
      TC_T(4);
      tc_fence_after();
      uint32_t v[2][32];
      tmem_ld32(tmem_base + lane_addr + kColD1, v[0]);
      bool good = true;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int q = 4 * s + kk;
        // the quarter is loaded and its column warp has finished reading it
        good = good && mbar_wait_warp(b_xfull(q), (it >> 1) & 1, abort_flag, status, kErrXFull) &&
               mbar_wait_warp(b_xread(q), (it >> 1) & 1, abort_flag, status, kErrXRead);
        if (!good) break;
        TC_T(3);
        tmem_wait_ld();
        if (kk + 1 < 4) tmem_ld32(tmem_base + lane_addr + kColD1 + 32 * (kk + 1), v[(kk + 1) & 1]);   // next quarter in flight
        const uint32_t rowp = base + q * kXBytes + (uint32_t)t * 128u;
        float4 xv[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)   // all loads first, then the arithmetic, then the stores
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(xv[c].x), "=f"(xv[c].y), "=f"(xv[c].z), "=f"(xv[c].w)
                       : "r"(rowp + (uint32_t)((c ^ (t & 7)) << 4))
                       : "memory");
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          xv[c].x = fmaf(coef, xv[c].x, __uint_as_float(v[kk & 1][4 * c]));
          xv[c].y = fmaf(coef, xv[c].y, __uint_as_float(v[kk & 1][4 * c + 1]));
          xv[c].z = fmaf(coef, xv[c].z, __uint_as_float(v[kk & 1][4 * c + 2]));
          xv[c].w = fmaf(coef, xv[c].w, __uint_as_float(v[kk & 1][4 * c + 3]));
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};"
                       ::"r"(rowp + (uint32_t)((c ^ (t & 7)) << 4)), "f"(xv[c].x), "f"(xv[c].y), "f"(xv[c].z), "f"(xv[c].w)
                       : "memory");
        if (kk == 3) {   // all of D1 is in registers: product 1 of the next sub-tile may overwrite it
          tc_fence_before();
          mbar_arrive_warp(b_d1empty);
        }
        fence_async_smem();
        mbar_arrive_warp(b_store(q));   // the TMA lane stores this quarter
        TC_T(5);
      }
      if (!good) break;
    }
    if (t == 0) TC_TIMING_FLUSH(status, 28, 8);
  } else if (warp < 8) {
    // ---------------------------------------------------------------- column threads (warps 4-7)
    const int t = threadIdx.x - 128;           // k within the slab = lane of tensor memory
    const int kk = t >> 5, c = t & 31;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t colp = (uint32_t)kk * kXBytes + (uint32_t)(c & 3) * 4u;
    const uint32_t chunk = (uint32_t)c >> 2;
    float acc[24];
#pragma unroll
    for (int j = 0; j < 24; ++j) acc[j] = 0.f;
    bool ok = true;
    TC_TIMING_DECL(6);
    // grad_phi sums of sub-tile `it` -> fp32 registers (columns 0..31: the d_hi terms, 32..63: the d_lo terms)
    auto drain = [&](int it) {
      if (!mbar_wait_warp(b_d2full, it & 1, abort_flag, status, kErrD2Full)) return false;
      TC_T(3);
      tc_fence_after();
      uint32_t v[32], w[32];
      tmem_ld32(tmem_base + lane_addr + kColD2, v);
      tmem_ld32(tmem_base + lane_addr + kColD2 + 32, w);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 24; ++j) acc[j] += __uint_as_float(v[j]) + __uint_as_float(w[j]);
      tc_fence_before();
      mbar_arrive_warp(b_d2empty);
      TC_T(4);
      return true;
    };
    for (int it = 0; it < nsub && ok; ++it) {
      const int q = 4 * (it & 1) + kk;          // this warp's quarter of the sub-tile
      if (!mbar_wait_warp(b_xfull(q), (it >> 1) & 1, abort_flag, status, kErrXFull)) { ok = false; break; }
      TC_T(0);
      const uint32_t tile = base + (it & 1) * kXStage + colp;
      for (int h = 0; h < 2 && ok; ++h) {
        if (it >= 1 && !mbar_wait_warp(b_a2free(h), (it - 1) & 1, abort_flag, status, kErrA2Free)) { ok = false; break; }
        TC_T(1);
#pragma unroll 1
        for (int rq = 0; rq < 2; ++rq) {         // 32 rows at a time
          uint32_t hi[32], lo[32];
          float xc[32];
#pragma unroll
          for (int u = 0; u < 32; ++u) {   // all loads first
            const uint32_t r = (uint32_t)(64 * h + 32 * rq + u);
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(xc[u]) : "r"(tile + r * 128u + ((chunk ^ (r & 7u)) << 4)) : "memory");
          }
#pragma unroll
          for (int u = 0; u < 32; ++u) {
            hi[u] = tf32_rn(xc[u]);
            lo[u] = tf32_rn(xc[u] - __uint_as_float(hi[u]));
          }
          const uint32_t a2 = tmem_base + lane_addr + kColA2 + 128 * h + 32 * rq;
          tmem_st32(a2, hi);
          tmem_st32(a2 + 64, lo);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive_warp(b_a2ready(h));
        TC_T(2);
        // The previous sub-tile's sums are collected here, after the first half of this one is on its way: the
        // tensor core needs a while to finish them, and the first product of this sub-tile cannot start before
        // they are out of the accumulator anyway.
        if (h == 0 && it >= 1) ok = drain(it - 1);
      }
      if (!ok) break;
      mbar_arrive_warp(b_xread(q));              // this warp no longer reads its quarter of the x tile
    }
    if (ok && nsub > 0) ok = drain(nsub - 1);
    if (t == 0) TC_TIMING_FLUSH(status, 16, 5);
    const int64_t k = k0 + t;
    if (k < K) {
      float* o = phi_part + ((int64_t)blockIdx.y * K + k) * 24;
      const float nanv = __int_as_float(0x7fc00000);
#pragma unroll
      for (int j = 0; j < 24; ++j) o[j] = ok ? acc[j] : nanv;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static const EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      p = nullptr;
    }
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// A [rows, cols] fp32 row-major tensor (row pitch cols * 4 bytes) cut into [box_rows x 32] tiles under
// the 128-byte swizzle; out-of-range elements read as zero.
static bool make_map_2d(CUtensorMap* m, const float* ptr, int64_t rows, int64_t cols, int box_rows,
                        CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool enabled() {
  static const bool on = [] {
    const char* e = std::getenv("MHC_ROWS_TC");
    return !(e && std::strcmp(e, "0") == 0);
  }();
  return on;
}

}  // namespace tc

static inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// Scratch of the tensor-core forward: a 256-byte header (status word) + phi^T hi and lo [32, Kp].
int64_t rows_tc_fwd_scratch_bytes(int64_t K) { return 256 + 2 * 32 * round_up(K, tc::kBK) * (int64_t)sizeof(float); }

// The tensor-core path needs TMA-compatible x rows (16-byte aligned base and pitch); MHC_ROWS_TC=0 in
// the environment turns it off (the mma.sync kernels then run).
bool rows_tc_usable(const float* x, int64_t batch, int64_t K) {
  return tc::enabled() && batch >= kManyRows && K % 4 == 0 && K >= 4 && is_aligned16(x) && batch < (1LL << 31) &&
         K < (1LL << 31) && tc::encode_fn() != nullptr;
}

// Scratch of the tensor-core backward, in floats: a 256-byte header (status word) + phi hi and lo [Kp, 32]
// with Kp = K rounded up to the slab of 128.
int64_t rows_tc_bwd_scratch_floats(int64_t K) { return 64 + 2 * 32 * round_up(K, tc::bw::kSlab); }

// The pass over x of the many-rows backward on tcgen05.  Row groups (one set of grad_phi partial sums each)
// are multiples of 128 rows so that no two CTAs ever store to the same rows of grad_x; *groups_used tells
// the caller how many sets to add up.
int rows_bwd_tc_launch(const float* x, const float* phi, const float* buf, float* phi_part, float* grad_x,
                       float* scratch, int64_t batch, int64_t K, int max_groups, cudaStream_t st, int* groups_used) {
  using namespace tc;
  if (!is_aligned16(scratch) || !is_aligned16(grad_x))
    return fail(MHC_ERR_MISALIGNED, "dynamic_weights_bwd: scratch and grad_x must be 16-byte aligned");
  const int64_t Kp = round_up(K, bw::kSlab);
  int* status = (int*)scratch;
  float* phi_hi = scratch + 64;
  float* phi_lo = phi_hi + 32 * Kp;
  if (max_groups < 1) max_groups = 1;
  const int64_t rows_per_group = round_up((batch + max_groups - 1) / max_groups, kBM);
  const int64_t groups = (batch + rows_per_group - 1) / rows_per_group;
  CUtensorMap mx, mg, mh, ml;
  if (!make_map_2d(&mx, x, batch, K, kBM, MHC_TC_BWD_X_PROMO) || !make_map_2d(&mg, grad_x, batch, K, kBM) ||
      !make_map_2d(&mh, phi_hi, Kp, 32, bw::kSlab) || !make_map_2d(&ml, phi_lo, Kp, 32, bw::kSlab))
    return fail(MHC_ERR_CUDA, "dynamic_weights_bwd: cuTensorMapEncodeTiled failed");
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(k_dw_rows_bwd_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bw::kSmem) != cudaSuccess)
      return check_launch("dynamic_weights_bwd(tc attribute)");
    attr_set = true;
  }
  {
    ProfScope ps("k_phi_split_rows", st);
    launch_k(k_phi_split_rows, (unsigned)((32 * Kp + 255) / 256), 256, 0, st, phi, phi_hi, phi_lo, K, Kp, status);
  }
  if (int e = check_launch("dynamic_weights_bwd(phi split)")) return e;
  {
    ProfScope ps("k_dw_rows_bwd_tc", st);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(Kp / bw::kSlab), (unsigned)groups);
    cfg.blockDim = dim3(bw::kThreadsBwd);
    cfg.dynamicSmemBytes = bw::kSmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, k_dw_rows_bwd_tc, mx, mg, mh, ml, buf, phi_part, batch, K, rows_per_group, status);
  }
  *groups_used = (int)groups;
  return check_launch("dynamic_weights_bwd(tc)");
}

int rows_fwd_tc_launch(const float* x, const float* phi, BiasPtrs bias, const float* alpha_pre, const float* alpha_post,
                       const float* alpha_res, float* H_pre, float* H_post, float* H_res, float* saved, void* scratch,
                       int64_t batch, int64_t K, int iters, float eps, cudaStream_t st) {
  using namespace tc;
  if (!is_aligned16(scratch)) return fail(MHC_ERR_MISALIGNED, "dynamic_weights_fwd: scratch must be 16-byte aligned");
  const int64_t Kp = round_up(K, kBK);
  int* status = (int*)scratch;
  float* phi_hi = (float*)((char*)scratch + 256);
  float* phi_lo = phi_hi + 32 * Kp;
  CUtensorMap mx, mh, ml;
  if (!make_map_2d(&mx, x, batch, K, kBM, MHC_TC_FWD_X_PROMO) || !make_map_2d(&mh, phi_hi, 32, Kp, kBN) ||
      !make_map_2d(&ml, phi_lo, 32, Kp, kBN))
    return fail(MHC_ERR_CUDA, "dynamic_weights_fwd: cuTensorMapEncodeTiled failed");
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(k_dw_rows_fwd_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess)
      return check_launch("dynamic_weights_fwd(tc attribute)");
    attr_set = true;
  }
  {
    ProfScope ps("k_phi_split_t", st);
    launch_k(k_phi_split_t, (unsigned)((32 * Kp + 255) / 256), 256, 0, st, phi, phi_hi, phi_lo, K, Kp, status);
  }
  if (int e = check_launch("dynamic_weights_fwd(phi split)")) return e;
  const RowsFinish fin{bias, alpha_pre, alpha_post, alpha_res, H_pre, H_post, H_res, saved, iters, eps};
  {
    ProfScope ps("k_dw_rows_fwd_tc", st);
    launch_k(k_dw_rows_fwd_tc, (unsigned)((batch + kBM - 1) / kBM), kThreads, kSmemBytes, st, mx, mh, ml, fin, batch, K, status);
  }
  return check_launch("dynamic_weights_fwd(tc)");
}

}  // namespace mhc

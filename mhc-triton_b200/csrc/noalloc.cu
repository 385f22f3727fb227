// Allocation-free variant of the add-residual backward.
//
// Some hosts that bind this library have no device allocator to hand: a plain C or C++ service
// without PyTorch's caching allocator, whose steady-state loop may not call cudaMalloc (it
// synchronises the whole device and can fail under a fixed memory budget), or a plugin that is
// handed input and output buffers by its framework and nothing else.  mhc_add_residual_bwd needs a
// small scratch area for its per-CTA partial sums; here that area is a fixed array inside the
// library image instead, so the caller passes only inputs and outputs.
#include <mutex>

#include "common.cuh"
#include "launch.h"

namespace mhc {

// Every GPU that loads the library holds this array (1 MiB) until the process exits.
constexpr int64_t kStaticScratchFloats = 262144;
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
static std::mutex g_addr_mu;
static float* g_addr[kMaxDevices] = {};

// Device address of g_static_scratch on the current device.  In host code the array's name is only
// a handle for the runtime, not an address a kernel can use, so the address is asked for once per
// device (with that device current) and cached.
static int static_scratch_ptr(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(MHC_ERR_CUDA, "add_residual_bwd_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  }
  if (dev < 0 || dev >= kMaxDevices) return fail(MHC_ERR_BAD_ARGUMENT, "add_residual_bwd_noalloc: device %d unsupported", dev);
  std::lock_guard<std::mutex> lk(g_addr_mu);
  if (!g_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return fail(MHC_ERR_CUDA, "add_residual_bwd_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    }
    g_addr[dev] = static_cast<float*>(p);
  }
  *out = g_addr[dev];
  return MHC_OK;
}

}  // namespace mhc

using namespace mhc;

extern "C" int64_t mhc_add_residual_bwd_noalloc_max_bytes(void) { return kStaticScratchFloats * (int64_t)sizeof(float); }

extern "C" int mhc_add_residual_bwd_noalloc(const void* dH_new, const void* branch_output, const float* H_post,
                                            void* d_branch_output, float* dH_post, int64_t B, int64_t S, int64_t D,
                                            int dtype, mhc_stream_t stream) {
  if (int e = check_bsd_pub("add_residual_bwd_noalloc", B, S, D, dtype)) return e;
  const int64_t need = add_residual_bwd_need_bytes(dH_new, branch_output, d_branch_output, B, S, D, dtype);
  if (need > mhc_add_residual_bwd_noalloc_max_bytes())
    return fail(MHC_ERR_SCRATCH_TOO_SMALL,
                "add_residual_bwd_noalloc: B=%lld S=%lld D=%lld needs %lld bytes of partial sums, the built-in area "
                "holds %lld; use mhc_add_residual_bwd with caller scratch",
                (long long)B, (long long)S, (long long)D, (long long)need,
                (long long)mhc_add_residual_bwd_noalloc_max_bytes());
  float* scratch = nullptr;
  if (int e = static_scratch_ptr(&scratch)) return e;
  // Every partial-sum slot the finish kernel reads is written by the main kernel of the same call,
  // so nothing in the area has to be cleared between calls.
  return mhc_add_residual_bwd(dH_new, branch_output, H_post, d_branch_output, dH_post, scratch,
                              mhc_add_residual_bwd_noalloc_max_bytes(), nullptr, B, S, D, dtype, stream);
}

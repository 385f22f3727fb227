// Status reporting for the C ABI: per-thread last-error text, CUDA launch checks, version.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "launch.h"

namespace mhc {

static thread_local char g_last_error[512] = "";
static std::atomic<long long> g_launches{0};

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return MHC_OK;
  }
  return fail(MHC_ERR_CUDA, "%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
}

}  // namespace mhc

extern "C" int mhc_version(void) { return MHC_B200_VERSION; }

extern "C" int64_t mhc_launch_count(void) { return (int64_t)mhc::g_launches.load(std::memory_order_relaxed); }

extern "C" const char* mhc_last_error_string(void) { return mhc::g_last_error; }

extern "C" const char* mhc_status_name(int status) {
  switch (status) {
    case MHC_OK: return "MHC_OK";
    case MHC_ERR_NULL_POINTER: return "MHC_ERR_NULL_POINTER";
    case MHC_ERR_BAD_SHAPE: return "MHC_ERR_BAD_SHAPE";
    case MHC_ERR_BAD_DTYPE: return "MHC_ERR_BAD_DTYPE";
    case MHC_ERR_BAD_ARGUMENT: return "MHC_ERR_BAD_ARGUMENT";
    case MHC_ERR_SCRATCH_TOO_SMALL: return "MHC_ERR_SCRATCH_TOO_SMALL";
    case MHC_ERR_MISALIGNED: return "MHC_ERR_MISALIGNED";
    case MHC_ERR_CUDA: return "MHC_ERR_CUDA";
  }
  return "MHC_ERR_UNKNOWN";
}

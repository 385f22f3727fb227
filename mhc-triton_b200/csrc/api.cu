// Status reporting for the C ABI: per-thread last-error text, CUDA launch checks, version.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

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

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("MHC_PDL");
    return !(e && std::strcmp(e, "0") == 0);
  }();
  return on;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return MHC_OK;
  }
  return fail(MHC_ERR_CUDA, "%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
}

// ---- optional per-kernel timing: CUDA events around each launch, on the launching stream ----
struct ProfRec { const char* name; cudaEvent_t a, b; };
static std::atomic<int> g_prof_on{0};
static std::mutex g_prof_mu;
static std::vector<ProfRec> g_prof;
static char g_prof_only[64] = "";  // when non-empty, only this kernel is timed

ProfScope::ProfScope(const char* name, cudaStream_t s) : slot(-1), st(s) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  if (g_prof_only[0] && std::strcmp(g_prof_only, name) != 0) return;
  ProfRec r{name, nullptr, nullptr};
  if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) {
    (void)cudaGetLastError();
    return;
  }
  cudaEventRecord(r.a, st);
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_prof.push_back(r);
  slot = (int)g_prof.size() - 1;
}

ProfScope::~ProfScope() {
  if (slot < 0) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (slot < (int)g_prof.size()) cudaEventRecord(g_prof[slot].b, st);
}

static void prof_clear() {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (auto& r : g_prof) {
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  g_prof.clear();
}

}  // namespace mhc

extern "C" int mhc_profile_enable(int on) {
  if (on == 1) mhc::prof_clear();   // 2 = resume, keeping the records
  mhc::g_prof_on.store(on ? 1 : 0);
  return MHC_OK;
}

extern "C" int mhc_profile_select(const char* kernel_name) {
  std::lock_guard<std::mutex> lk(mhc::g_prof_mu);
  std::snprintf(mhc::g_prof_only, sizeof(mhc::g_prof_only), "%s", kernel_name ? kernel_name : "");
  return MHC_OK;
}

extern "C" int64_t mhc_profile_count(void) {
  std::lock_guard<std::mutex> lk(mhc::g_prof_mu);
  return (int64_t)mhc::g_prof.size();
}

extern "C" int mhc_profile_get(int64_t index, const char** name, float* milliseconds) {
  std::lock_guard<std::mutex> lk(mhc::g_prof_mu);
  if (index < 0 || index >= (int64_t)mhc::g_prof.size() || !name || !milliseconds)
    return mhc::fail(MHC_ERR_BAD_ARGUMENT, "profile_get: bad index or null pointer");
  const mhc::ProfRec& r = mhc::g_prof[(size_t)index];
  *name = r.name;
  const cudaError_t e = cudaEventElapsedTime(milliseconds, r.a, r.b);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return mhc::fail(MHC_ERR_CUDA, "profile_get: %s (synchronize the device first)", cudaGetErrorString(e));
  }
  return MHC_OK;
}

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

// Host-side helpers shared by the C-ABI translation units: status reporting, launch checks,
// and the geometry (tokens per chunk, columns per CTA) of the streaming kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <initializer_list>

#include "../../include/mhc_b200.h"
#include "common.cuh"

namespace mhc {

constexpr int64_t kMaxGridItems = 0x7fffffffLL;  // gridDim.x limit

int fail(int status, const char* fmt, ...);  // records the message for mhc_last_error_string
int check_launch(const char* what);          // cudaGetLastError -> status

inline bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Geometry of a streaming kernel over [B, S, 4, D].
//   vec   : elements per pack (1 = scalar path for odd D or unaligned pointers)
//   pool  : the mean-pool kernel (long chunks, sub-groups inside the CTA)
Geo make_geo(int64_t S, int64_t D, int vec, bool pool);
inline int geo_block(const Geo& g) { return g.cols * g.sub; }
inline int64_t geo_slots(const Geo& g) { return (int64_t)g.nchunk * g.CG; }  // partial rows per batch element

// Pack width usable for a row length D of `dtype` given the pointers involved.
int pick_vec(int dtype, int64_t D, std::initializer_list<const void*> ptrs);

int64_t weights_fwd_scratch_bytes(int64_t batch, int64_t K);
int64_t weights_bwd_scratch_bytes(int64_t batch, int64_t K);

}  // namespace mhc

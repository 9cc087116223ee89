// Shared helpers for the cueq_b200 kernels: error reporting, dtype-generic loads, atomics.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/cueq_b200.h"

namespace cueq {

// thread-local message returned by cueq_b200_last_error()
char* error_buffer();
int fail(const char* fmt, ...);

#define CUEQ_CUDA_OK(expr)                                                        \
  do {                                                                            \
    cudaError_t e__ = (expr);                                                     \
    if (e__ != cudaSuccess)                                                       \
      return ::cueq::fail("%s failed: %s", #expr, cudaGetErrorString(e__));       \
  } while (0)

static inline int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// One flag per device ordinal.  Function attributes such as the dynamic shared-memory limit
// belong to the device that was current when they were set, so a launcher that has configured
// its kernel on one GPU still has to do it on the next GPU the same process uses.
struct PerDeviceFlag {
  static constexpr int kMax = 64;
  bool done[kMax] = {};
  static int current() {
    int d = -1;
    return cudaGetDevice(&d) == cudaSuccess ? d : -1;
  }
  bool get() const {
    const int d = current();
    return d >= 0 && d < kMax && done[d];
  }
  void set() {
    const int d = current();
    if (d >= 0 && d < kMax) done[d] = true;
  }
};

// Load one element of a buffer whose element type is only known at run time.
template <typename M>
__device__ __forceinline__ M load_as(const void* p, int dtype, int64_t i) {
  switch (dtype) {
    case CUEQ_F32: return (M)__ldg(reinterpret_cast<const float*>(p) + i);
    case CUEQ_F64: return (M)__ldg(reinterpret_cast<const double*>(p) + i);
    case CUEQ_BF16: return (M)__bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    default: return (M)__half2float(reinterpret_cast<const __half*>(p)[i]);
  }
}

__device__ __forceinline__ int64_t load_index(const void* idx, int is64, int64_t z) {
  return is64 ? __ldg(reinterpret_cast<const long long*>(idx) + z)
              : (int64_t)__ldg(reinterpret_cast<const int*>(idx) + z);
}

template <typename M>
__device__ __forceinline__ M warp_sum(M v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace cueq

// Self-test of the bounded waits used by the tensor-core kernels: one thread waits on an mbarrier
// that nothing ever arrives on.  The wait must give up after its cycle budget (about half a
// second), record status 2 and return, leaving the context usable - the behaviour every pipeline
// in gemm_tc.cu, fctp_fused.cu and gemm_f32x3.cu relies on when a producer or a copy never shows up.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

__global__ void bounded_wait_selftest_kernel(int* status, long long* waited_cycles) {
  __shared__ unsigned long long bar;
  if (threadIdx.x == 0) {
    cueq_tc::bar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    const long long t0 = clock64();
    const bool ok = cueq_tc::bar_wait(&bar, 0, status);   // nothing arrives: must come back false
    if (waited_cycles) *waited_cycles = ok ? -1 : clock64() - t0;
  }
}

// Debug aid standing in for a memory checker: flags gather / scatter indices that point outside their
// buffer (status 3) instead of letting the launch that uses them read or write out of bounds.
template <typename I>
__global__ void index_range_kernel(const I* __restrict__ idx, int64_t n, int64_t rows, int* status) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t v = (int64_t)idx[i];
    if (v < 0 || v >= rows) atomicExch(status, 3);
  }
}

// Measures what the float32 multiply-add pipes deliver: every thread runs 16 independent chains of dependent
// FMAs held in registers, no memory traffic.  The host times the launch; work = 2 * threads * 16 * iters flop.
__global__ void __launch_bounds__(256) fma_peak_kernel(float* __restrict__ sink, int iters, float a, float b) {
  float acc[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) acc[k] = (float)(threadIdx.x + k);
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int k = 0; k < 16; ++k) acc[k] = fmaf(acc[k], a, b);
  }
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 16; ++k) s += acc[k];
  if (s == 12345.678f) sink[0] = s;   // keeps the chains alive without a store in practice
}

// The same measurement with the packed instruction of sm_100 (fma.rn.f32x2: two float32 multiply-adds per
// thread and instruction): eight chains of float2 per thread, work = 2 * threads * 16 * iters flop as above.
__global__ void __launch_bounds__(256) fma2_peak_kernel(float* __restrict__ sink, int iters, float a, float b) {
  float2 acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = make_float2((float)(threadIdx.x + k), (float)k);
  const float2 a2 = make_float2(a, a), b2 = make_float2(b, b);
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = __ffma2_rn(acc[k], a2, b2);
  }
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += acc[k].x + acc[k].y;
  if (s == 12345.678f) sink[0] = s;
}

}  // namespace

extern "C" int cueq_b200_selftest_fma2_peak(void* sink, int32_t blocks, int32_t iters, void* stream) {
  if (!sink || blocks <= 0 || iters <= 0) return cueq::fail("fma peak: invalid arguments");
  fma2_peak_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<float*>(sink), iters, 0.999f, 0.001f);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int cueq_b200_selftest_fma_peak(void* sink, int32_t blocks, int32_t iters, void* stream) {
  if (!sink || blocks <= 0 || iters <= 0) return cueq::fail("fma peak: invalid arguments");
  fma_peak_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<float*>(sink), iters, 0.999f, 0.001f);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int cueq_b200_check_index_range(const void* index, int64_t n, int64_t rows, int32_t index_is_64, void* status, void* stream) {
  if (!status) return cueq::fail("index check: the status word is required");
  if (n <= 0) return 0;
  if (!index) return cueq::fail("index check: null index");
  const unsigned grid = (unsigned)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (index_is_64) index_range_kernel<long long><<<grid, 256, 0, st>>>(reinterpret_cast<const long long*>(index), n, rows, reinterpret_cast<int*>(status));
  else index_range_kernel<int><<<grid, 256, 0, st>>>(reinterpret_cast<const int*>(index), n, rows, reinterpret_cast<int*>(status));
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int cueq_b200_selftest_bounded_wait(void* status, void* waited_cycles, void* stream) {
  if (!status) return cueq::fail("selftest: the status word is required");
  bounded_wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<int*>(status),
                                                                                   reinterpret_cast<long long*>(waited_cycles));
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

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

}  // namespace

extern "C" int cueq_b200_selftest_bounded_wait(void* status, void* waited_cycles, void* stream) {
  if (!status) return cueq::fail("selftest: the status word is required");
  bounded_wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<int*>(status),
                                                                                   reinterpret_cast<long long*>(waited_cycles));
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

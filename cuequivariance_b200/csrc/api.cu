// C ABI housekeeping: version, thread-local error text.
#include "common.cuh"

namespace cueq {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return 1;
}

}  // namespace cueq

extern "C" int cueq_b200_abi_version(void) { return CUEQ_B200_ABI_VERSION; }

// One asynchronous copy between device pointers on `stream`; either side may be another GPU's memory
// mapped into this process.  The driver serves it with a copy engine, so no SM is taken from the kernels
// that run meanwhile.
// Lets copies and kernels of the current device reach memory of `peer_device` directly (over NVLink where the
// GPUs are linked).  Without it a copy between two devices is staged through host memory.  Idempotent.
extern "C" int cueq_b200_enable_peer_access(int peer_device) {
  int dev = -1, can = 0;
  CUEQ_CUDA_OK(cudaGetDevice(&dev));
  if (dev == peer_device) return 0;
  CUEQ_CUDA_OK(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  if (!can) return cueq::fail("device %d cannot access device %d directly", dev, peer_device);
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();   // clear the sticky-free error state
    return 0;
  }
  if (e != cudaSuccess) return cueq::fail("cudaDeviceEnablePeerAccess(%d) failed: %s", peer_device, cudaGetErrorString(e));
  return 0;
}

extern "C" int cueq_b200_copy_async(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return 0;
  if (!dst || !src) return cueq::fail("copy: null pointer");
  CUEQ_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, reinterpret_cast<cudaStream_t>(stream)));
  return 0;
}
extern "C" const char* cueq_b200_last_error(void) { return cueq::error_buffer(); }
extern "C" int64_t cueq_b200_sizeof(int which) {
  switch (which) {
    case 0: return sizeof(cueq_u1d_desc);
    case 1: return sizeof(cueq_buffer);
    case 2: return sizeof(cueq_cw_args);
    case 3: return sizeof(cueq_cw_noalloc_args);
    case 4: return sizeof(cueq_gemm_args);
    case 5: return sizeof(cueq_fctp_args);
    case 6: return sizeof(cueq_fctp_fused_args);
    case 7: return sizeof(cueq_fctp_fused_task);
    case 8: return sizeof(cueq_fctp_fused_gx_args);
    case 9: return sizeof(cueq_fctp_fused_unit);
    case 10: return sizeof(cueq_fctp_fused_gw_args);
    case 11: return sizeof(cueq_fctp_fused_wunit);
    case 12: return sizeof(cueq_gemm_f32x3_args);
    case 13: return sizeof(cueq_gemm_f32x3_tn_args);
    case 14: return sizeof(cueq_sh_args);
    default: return -1;
  }
}

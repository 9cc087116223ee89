// Row exchange between the GPUs of one node with plain stores into peer-mapped memory.
//
// The receiver-sharded channelwise product moves node rows between ranks twice per step (node features
// out, their gradients back).  A copy-engine transfer into memory that another process exported through
// CUDA IPC turned out to block the issuing host thread until the copy had run (measured: 1.3 ms per call,
// the host fell behind the device), so the rows are pushed by a small kernel instead: up to eight
// (destination, source, size) pieces per launch, a handful of thread blocks per piece, 16-byte loads from
// local memory and 16-byte stores to the peer over NVLink.  A launch never blocks the host, and it takes
// a few dozen thread-block slots for the duration of the transfer instead of the SMs a collective uses.
// Stores only (a read from the peer ran at 24 GB/s, a write at 650 GB/s on this system); no multicast, no
// TMA, no flag: completion is ordered by the stream, and ranks agree on it with a one-element all-reduce.
#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace {

typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

GetAddressRangeFn address_range_fn() {
  static GetAddressRangeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<GetAddressRangeFn>(p);
  }
  return fn;
}

__global__ void __launch_bounds__(256) push_kernel(const __grid_constant__ cueq_push_args a) {
  const int piece = blockIdx.y;
  const uint4* __restrict__ src = reinterpret_cast<const uint4*>(a.src[piece]);
  uint4* __restrict__ dst = reinterpret_cast<uint4*>(a.dst[piece]);
  const int64_t n = a.bytes[piece] / 16;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  // four independent 16-byte transfers in flight per thread
  for (; i + 3 * stride < n; i += 4 * stride) {
    const uint4 v0 = src[i], v1 = src[i + stride], v2 = src[i + 2 * stride], v3 = src[i + 3 * stride];
    dst[i] = v0; dst[i + stride] = v1; dst[i + 2 * stride] = v2; dst[i + 3 * stride] = v3;
  }
  for (; i < n; i += stride) dst[i] = src[i];
}

}  // namespace

// ---- sharing a buffer with the other processes of the node -----------------------------------------
//
// export: the IPC handle of the allocation that contains `ptr`, and the offset of `ptr` inside it.
// open  : maps that allocation into the CURRENT device's address space (with peer access to the exporting
//         GPU), which is what lets kernels and copies of this device reach it.  Opening the handle while the
//         exporting GPU's ordinal is current - what a generic tensor hand-over between processes does - yields
//         a mapping that belongs to that other device: a kernel of this device faults on it and a copy is
//         staged by the driver (measured: host-synchronous and slow).
extern "C" int cueq_b200_ipc_export(const void* ptr, void* handle64, int64_t* offset) {
  if (!ptr || !handle64 || !offset) return cueq::fail("ipc export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  GetAddressRangeFn range = address_range_fn();
  if (!range) return cueq::fail("ipc export: cuMemGetAddressRange is not available from the driver");
  CUdeviceptr base = 0;
  size_t size = 0;
  if (range(&base, &size, (CUdeviceptr)(uintptr_t)ptr) != CUDA_SUCCESS) return cueq::fail("ipc export: not a device allocation");
  CUEQ_CUDA_OK(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), reinterpret_cast<void*>((uintptr_t)base)));
  *offset = (int64_t)((uintptr_t)ptr - (uintptr_t)base);
  return 0;
}

extern "C" int cueq_b200_ipc_open(const void* handle64, void** base) {
  if (!handle64 || !base) return cueq::fail("ipc open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  CUEQ_CUDA_OK(cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}

extern "C" int cueq_b200_ipc_close(void* base) {
  if (!base) return 0;
  CUEQ_CUDA_OK(cudaIpcCloseMemHandle(base));
  return 0;
}

extern "C" int cueq_b200_push(const cueq_push_args* a, void* stream) {
  if (!a) return cueq::fail("push: null arguments");
  if (a->num_pieces < 0 || a->num_pieces > 8) return cueq::fail("push: 0..8 pieces per launch, got %d", a->num_pieces);
  if (a->num_pieces == 0) return 0;
  for (int k = 0; k < a->num_pieces; ++k) {
    if (!a->dst[k] || !a->src[k]) return cueq::fail("push: null pointer in piece %d", k);
    if (((uintptr_t)a->dst[k] | (uintptr_t)a->src[k] | (uintptr_t)a->bytes[k]) & 15) return cueq::fail("push: pieces must be 16-byte aligned and sized");
  }
  const int blocks = a->blocks_per_piece > 0 ? a->blocks_per_piece : 4;
  push_kernel<<<dim3(blocks, a->num_pieces), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

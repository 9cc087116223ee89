// Device and host helpers shared by the tensor-core kernels (gemm_tc.cu, fctp_fused.cu): mbarrier
// and TMA wrappers with bounded waits, shared-memory matrix descriptors for 128-byte-swizzled
// tiles, tcgen05.mma / tcgen05.commit wrappers, and the driver entry point that encodes tensor maps.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace cueq_tc {

constexpr long long kMaxWaitCycles = 1ll << 30;   // bound of every barrier wait, in SM clock cycles

__device__ __forceinline__ unsigned s32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(unsigned long long* b, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(s32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(unsigned long long* b, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(unsigned long long* b, unsigned parity) {
  // try_wait parks the thread in hardware until the phase completes or a short system time
  // limit passes, so a waiter wakes within nanoseconds of the arrival (a test_wait + nanosleep
  // loop was measured to add microseconds per hand-over)
  unsigned ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(s32(b)), "r"(parity) : "memory");
  return ok != 0;
}
// returns false (and records it) if the barrier did not flip within about half a second
__device__ __forceinline__ bool bar_wait(unsigned long long* b, unsigned parity, int* status) {
  if (bar_try(b, parity)) return true;
  const long long t0 = clock64();
  while (clock64() - t0 < kMaxWaitCycles) {
    if (bar_try(b, parity)) return true;
  }
  if (status) {
    atomicExch(status, 2);
    __threadfence();  // visible to the epilogue threads before anything this thread signals next
  }
  return false;
}
// True while no bounded wait has run out on this device since the host last cleared the word.
// Every epilogue asks this after its own wait and before its first global store: a role of
// the same CTA that gave up has stored 2 (and fenced) before it released the epilogue, so a
// partial accumulator never reaches caller-owned memory; the host learns of it from the word.
__device__ __forceinline__ bool status_clean(const int* status) {
  return !status || *reinterpret_cast<const volatile int*>(status) == 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, unsigned long long* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(s32(dst)), "l"(map), "r"(s32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ unsigned long long smem_desc(const void* p) {
  // K-major, 128-byte swizzle: 8-row groups are 1024 bytes apart; version 1 (Blackwell)
  const unsigned long long addr = (s32(p) & 0x3FFFFu) >> 4;
  return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ unsigned long long smem_desc_mn(const void* p) {
  // MN-major, 128-byte swizzle: the tile is stored as blocks of [64 K-rows][64 elements along M/N]
  // (8 KiB each, rows of 128 bytes); groups of 8 K-rows are 1024 bytes apart (stride offset),
  // consecutive 64-element blocks along M/N are 8192 bytes apart (leading offset)
  const unsigned long long addr = (s32(p) & 0x3FFFFu) >> 4;
  return addr | ((8192ull >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_c, unsigned long long da, unsigned long long db, unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
               ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(s32(bar)) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}


}  // namespace cueq_tc

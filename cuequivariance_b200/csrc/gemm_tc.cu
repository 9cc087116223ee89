// Tensor-core GEMM for the dense ("uvw") contractions: C[M,N] (+)= A[M,K] * B[N,K]^T with
// bf16 operands (both K-major) and float32 accumulation, written directly against the
// Blackwell tensor-core interface:
//   * operand tiles are brought into 128-byte-swizzled shared memory by TMA
//     (cp.async.bulk.tensor.2d) and their arrival is signalled on mbarriers;
//   * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, 128 x 64 x 16 per
//     instruction) with the accumulator in tensor memory (TMEM); tcgen05.commit releases a
//     pipeline stage when the MMAs that read it have finished;
//   * four epilogue warps read the accumulator back with tcgen05.ld and store the rows.
// Takes the place of the closed FusedTensorProductOp4 kernel's dense contraction
// (cuequivariance_torch/primitives/segmented_polynomial_fused_tp.py:51-72) once the coupled
// operand has been formed.  Every wait is bounded: on timeout the kernel records a status
// word, still frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

using namespace cueq_tc;

constexpr int BM = 128, BN = 64, BK = 64;       // tile; BK bf16 = 128 bytes = one swizzle row
constexpr int kStagesTc = 4;
constexpr int kTileA = BM * BK * 2, kTileB = BN * BK * 2;
constexpr int kStageBytes = kTileA + kTileB;
constexpr int kThreads = 192;                   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue

struct GemmParams {
  void* C;
  int64_t ldc;          // elements between consecutive rows of one group
  int64_t group_stride; // elements between consecutive groups of rows
  int rows_per_group;   // row r lives at (r / rows_per_group) * group_stride + (r % rows_per_group) * ldc
  int M, N, K;
  int accumulate;
  int out_bf16;         // 1: C is bf16 (no accumulation), 0: float32
  int a_mn_major, b_mn_major;  // 1: the operand is stored [K][M or N] (M/N contiguous) instead of [M or N][K]
  int kb_per_split;     // K blocks handled by one CTA (split-K over blockIdx.z; partial sums are added atomically)
  int* status;
};

__global__ void __launch_bounds__(kThreads) gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_b,
                                                               const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned long long* full = reinterpret_cast<unsigned long long*>(smem + kStagesTc * kStageBytes);
  unsigned long long* empty = full + kStagesTc;
  unsigned long long* acc_ready = empty + kStagesTc;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_ready + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int num_kb = min(p.kb_per_split, p.K / BK - kb_begin);
  const bool split = gridDim.z > 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesTc; ++s) { bar_init(full + s, 1); bar_init(empty + s, 1); }
    bar_init(acc_ready, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {  // TMEM: 64 columns x 128 lanes of float32 accumulator
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(tmem_slot)), "r"(64u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStagesTc;
        if (!bar_wait(empty + s, ((kb / kStagesTc) & 1) ^ 1, p.status)) break;
        bar_expect_tx(full + s, kStageBytes);
        unsigned char* a = smem + s * kStageBytes;
        if (p.a_mn_major) {
          tma_load_2d(a, &map_a, m0, (kb_begin + kb) * BK, full + s);
          tma_load_2d(a + 8192, &map_a, m0 + 64, (kb_begin + kb) * BK, full + s);
        } else {
          tma_load_2d(a, &map_a, (kb_begin + kb) * BK, m0, full + s);
        }
        if (p.b_mn_major) tma_load_2d(a + kTileA, &map_b, n0, (kb_begin + kb) * BK, full + s);
        else tma_load_2d(a + kTileA, &map_b, (kb_begin + kb) * BK, n0, full + s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: D = f32, A = B = bf16, both K-major, N = 64, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24) |
                             (p.a_mn_major ? (1u << 15) : 0u) | (p.b_mn_major ? (1u << 16) : 0u);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % kStagesTc;
        ok = bar_wait(full + s, (kb / kStagesTc) & 1, p.status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned long long da = p.a_mn_major ? smem_desc_mn(smem + s * kStageBytes) : smem_desc(smem + s * kStageBytes);
        const unsigned long long db = p.b_mn_major ? smem_desc_mn(smem + s * kStageBytes + kTileA) : smem_desc(smem + s * kStageBytes + kTileA);
        // one instruction covers 16 elements of K: 32 bytes along a K-major row (2 descriptor
        // units), or 16 rows of 128 bytes of an MN-major block (128 units)
        const unsigned long long sa = p.a_mn_major ? 128 : 2, sb = p.b_mn_major ? 128 : 2;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk)
          umma_bf16(tmem_base, da + sa * kk, db + sb * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
        umma_commit(empty + s);  // frees the stage once these MMAs have read it
      }
      umma_commit(acc_ready);
    }
  } else {
    // epilogue: warp w may touch TMEM lanes 32*(w%4) .. 32*(w%4)+31
    const int q = warp & 3;
    const bool ok = bar_wait(acc_ready, 0, p.status);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const int row = m0 + q * 32 + lane;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      unsigned v[32];
      const unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + half * 32;
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                   "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                   "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                     "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                     "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                     "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                   : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      if (ok && status_clean(p.status) && row < p.M) {
        const int64_t roff = (int64_t)(row / p.rows_per_group) * p.group_stride + (int64_t)(row % p.rows_per_group) * p.ldc + n0 + half * 32;
        if (p.out_bf16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + roff;
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) h[t] = __floats2bfloat162_rn(__uint_as_float(v[c + 2 * t]), __uint_as_float(v[c + 2 * t + 1]));
            *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<uint4*>(h);
          }
        } else {
          float* dst = reinterpret_cast<float*>(p.C) + roff;
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            float4 o = make_float4(__uint_as_float(v[c]), __uint_as_float(v[c + 1]), __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
            if (split) {
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(dst + c), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
              continue;
            }
            if (p.accumulate) {
              const float4 old = *reinterpret_cast<const float4*>(dst + c);
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *reinterpret_cast<float4*>(dst + c) = o;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(64u) : "memory");
  }
}

// K-major operand: global [rows][cols = K] with `ld` elements between rows; box = 64 K x box_rows.
// MN-major operand: global [K][cols = M or N]; box = 64 (M/N) x 64 (K).
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return cueq::fail("gemm: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cueq::fail("gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

}  // namespace

extern "C" int cueq_b200_gemm_bf16(const cueq_gemm_args* g, void* stream) {
  if (!g || !g->A || !g->B || !g->C) return cueq::fail("gemm: null operand");
  const int64_t M = g->M, N = g->N, K = g->K;
  if (M <= 0 || N <= 0 || K <= 0) return cueq::fail("gemm: empty problem");
  if (N % BN || K % BK) return cueq::fail("gemm: N must be a multiple of %d and K of %d (got N=%lld K=%lld)", BN, BK, (long long)N, (long long)K);
  if (g->a_mn_major && (M % BM)) return cueq::fail("gemm: an MN-major A needs M to be a multiple of %d", BM);
  if ((g->lda % 8) || (g->ldb % 8) || (g->ldc % 4)) return cueq::fail("gemm: leading dimensions must keep rows 16-byte aligned");
  if (((uintptr_t)g->A | (uintptr_t)g->B | (uintptr_t)g->C) & 15) return cueq::fail("gemm: operands must be 16-byte aligned");
  if (M > 2147483647LL || K > 2147483647LL) return cueq::fail("gemm: dimension too large");
  if (g->out_bf16 && g->accumulate) return cueq::fail("gemm: accumulation needs a float32 output");
  const int rpg = g->rows_per_group > 0 ? g->rows_per_group : 1;
  if ((g->group_stride % 4) != 0) return cueq::fail("gemm: group stride must be a multiple of 4 elements");
  CUtensorMap ma, mb;
  // K-major: rows = M (or N), cols = K.  MN-major: rows = K, cols = M (or N).
  if (int rc = g->a_mn_major ? make_map(&ma, g->A, K, M, g->lda, 64) : make_map(&ma, g->A, M, K, g->lda, BM)) return rc;
  if (int rc = g->b_mn_major ? make_map(&mb, g->B, K, N, g->ldb, 64) : make_map(&mb, g->B, N, K, g->ldb, BN)) return rc;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.C = g->C; p.ldc = g->ldc; p.rows_per_group = rpg; p.group_stride = g->group_stride > 0 ? g->group_stride : (int64_t)rpg * g->ldc;
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.accumulate = g->accumulate; p.out_bf16 = g->out_bf16;
  p.a_mn_major = g->a_mn_major; p.b_mn_major = g->b_mn_major; p.status = reinterpret_cast<int*>(g->status);
  const size_t smem = kStagesTc * kStageBytes + 1024 + 256;
  static cueq::PerDeviceFlag configured;
  if (!configured.get()) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(gemm_bf16_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set();
  }
  // split K when the tile grid alone cannot fill the GPU (partial sums then need a float32 C that
  // the caller zeroed or wants accumulated into)
  const int64_t tiles = ((M + BM - 1) / BM) * (N / BN);
  const int total_kb = (int)(K / BK);
  int splits = 1;
  if (!g->out_bf16 && (g->accumulate || g->c_is_zero) && tiles < 296 && total_kb >= 16) {
    splits = (int)((592 + tiles - 1) / tiles);
    if (splits > total_kb / 4) splits = total_kb / 4;
    if (splits < 1) splits = 1;
  }
  p.kb_per_split = (total_kb + splits - 1) / splits;
  splits = (total_kb + p.kb_per_split - 1) / p.kb_per_split;
  dim3 grid((unsigned)((M + BM - 1) / BM), (unsigned)(N / BN), (unsigned)splits);
  gemm_bf16_tn_kernel<<<grid, kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(ma, mb, p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int cueq_b200_gemm_bf16_tn(const void* A, const void* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                                      int64_t ldb, int64_t ldc, int32_t accumulate, void* status, void* stream) {
  cueq_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.A = A; g.B = B; g.C = C; g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb; g.ldc = ldc;
  g.accumulate = accumulate; g.status = status; g.rows_per_group = 1; g.c_is_zero = 0;
  return cueq_b200_gemm_bf16(&g, stream);
}

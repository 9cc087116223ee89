// Fully connected ("uvw") tensor product with the coupled operand built on chip.
//
// For a path (l1, l2, l3) of ``uvw,iu,jv,kw+ijk`` (descriptor:
// cuequivariance/group_theory/descriptors/irreps_tp.py:22-91; executor call site:
// cuequivariance_torch/primitives/segmented_polynomial_fused_tp.py:51-72) with coupling C[i,j,k]:
//
//   out[z,k,w] = sum_paths sum_(u,v) Z[z,k,(u,v)] * W[(u,v),w],   Z[z,k,(u,v)] = sum_ij C[i,j,k] x1[z,i,u] x2[z,j,v]
//
// Z has 64 x 64 columns per (sample, component); writing it to memory costs 2.4 GB per pass at
// 32,768 samples.  Here it never leaves the SM: producer warps compute one [128 samples x 64 (u
// fixed, all v)] slice at a time directly into 128-byte-swizzled shared memory in the layout
// tcgen05.mma expects for a K-major A operand, the matching [64 x 64] slice of W arrives by TMA,
// two threads issue the MMAs of alternate slices into two TMEM accumulators, and four epilogue warps
// add them and write the finished [128 x 64] block of the output.  One CTA owns (output irrep, component k, 128 samples) and runs
// over all paths that end in that irrep, so every output element is written exactly once.
//
// Warp roles: 0 = TMA (W slices), 1 and 14 = MMA issue (1 owns TMEM), 2-5 = epilogue, 6-13 = producers.
// Every wait is bounded; a wait that runs out records status 2, the thread stops waiting and
// working but keeps arriving on barriers, so the CTA always reaches its end and frees its TMEM.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

using namespace cueq_tc;

constexpr int FM = 128;                 // samples per CTA (MMA M)
constexpr int FN = 64;                  // w extent (MMA N)
constexpr int FK = 64;                  // K per stage: one u, all 64 v
constexpr int kStagesF = 6;             // A ring: tiles written by the producer warps (short latency)
constexpr int kStagesB = 8;             // B ring: W slices fetched by TMA (L2 latency: needs the deeper lookahead)
constexpr int kTileAF = FM * FK * 2;    // 16 KiB
constexpr int kTileBF = FK * FN * 2;    // 8 KiB
constexpr int kStageF = kTileAF;
constexpr int kProducers = 256;
constexpr int kThreadsF = 64 + 128 + kProducers;
constexpr int kIssuers = 2;              // threads issuing tcgen05.mma in the forward kernel
constexpr int kThreadsFwd = kThreadsF + 32 * (kIssuers - 1);
constexpr int kFwdTmemCols = kIssuers * FN <= 64 ? 64 : kIssuers * FN <= 128 ? 128 : 256;   // allocations are powers of two

struct FwdParams {
  const __nv_bfloat16* x1;
  const __nv_bfloat16* x2;
  void* out;
  int64_t ld1, ld2, ldo, batch;
  int out_bf16;
  int* status;
  cueq_fctp_fused_task tasks[CUEQ_FCTP_FUSED_MAX_TASKS];
};

__device__ __forceinline__ void producers_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kProducers) : "memory"); }
__device__ __forceinline__ void bar_arrive(unsigned long long* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(s32(b)) : "memory");
}
__device__ __forceinline__ float bf16_lo(unsigned w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(unsigned w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ unsigned hfma2_bits(unsigned a, unsigned b, unsigned c) {
  unsigned d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ unsigned hmul2_bits(unsigned a, unsigned b) {
  unsigned d;
  asm("mul.rn.bf16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ unsigned pack_same(float t) {
  unsigned d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %1;\n" : "=r"(d) : "f"(t));
  return d;
}

__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                 "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                 "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
               : "r"(taddr));
}

// The 64 stage items (u = 0..63) of one path for this CTA's component k.  `ptid` in [0, 256): a
// warp covers 16 sample rows; the 2 lanes of a row each own 32 of the 64 v (four 16-byte chunks)
// and keep that part of x2[z, j, v] in registers for the whole path (only the NJ columns j for
// which C[:, j, k] is not all zero), so the only shared-memory traffic of an item is the A tile
// itself.  The 2 lanes take turns computing T[j] = sum_i C[i,j,k] x1[z,i,u] for 2 consecutive u
// and exchange the values with shuffles.  `coef[i * 5 + jj]` holds C[i, active[jj], k].
template <int D1, int NJ>
__device__ __forceinline__ void produce_items(const FwdParams& p, const cueq_fctp_fused_path& path, unsigned char* stages,
                                              const float* coef, const int* active, unsigned long long* full,
                                              unsigned long long* empty, int item0, bool& dead, int64_t z0, int ptid) {
  const int lane = ptid & 31;
  const int row = (ptid >> 5) * 16 + (lane >> 1), half = lane & 1;
  const int64_t z = z0 + row;
  const bool valid = z < p.batch;
  const unsigned short* x1row = reinterpret_cast<const unsigned short*>(p.x1 + (valid ? z : 0) * p.ld1 + path.off1);
  uint4 x2r[4][NJ];
#pragma unroll
  for (int jj = 0; jj < NJ; ++jj) {
    const uint4* src = reinterpret_cast<const uint4*>(p.x2 + (valid ? z : 0) * p.ld2 + path.off2 + active[jj] * 64) + half * 4;
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) x2r[cc][jj] = valid ? __ldg(src + cc) : make_uint4(0, 0, 0, 0);
  }
  float cf[D1][NJ];
#pragma unroll
  for (int i = 0; i < D1; ++i)
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) cf[i][jj] = coef[i * 5 + jj];
  const int swz = row & 7;
  unsigned short xn[D1];
#pragma unroll
  for (int i = 0; i < D1; ++i) xn[i] = valid ? __ldg(x1row + i * 64 + half) : (unsigned short)0;
  for (int u0 = 0; u0 < FK; u0 += 2) {
    unsigned tmine[NJ];
    {
      float xf[D1];
#pragma unroll
      for (int i = 0; i < D1; ++i) xf[i] = bf16_lo(xn[i]);
      if (u0 + 2 < FK) {
#pragma unroll
        for (int i = 0; i < D1; ++i) xn[i] = valid ? __ldg(x1row + i * 64 + u0 + 2 + half) : (unsigned short)0;
      }
#pragma unroll
      for (int jj = 0; jj < NJ; ++jj) {
        float t = cf[0][jj] * xf[0];
#pragma unroll
        for (int i = 1; i < D1; ++i) t = fmaf(cf[i][jj], xf[i], t);
        tmine[jj] = pack_same(t);
      }
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      unsigned t2[NJ];
#pragma unroll
      for (int jj = 0; jj < NJ; ++jj) t2[jj] = __shfl_sync(0xffffffffu, tmine[jj], (lane & ~1) + q);
      const int item = item0 + u0 + q;
      const int s = item % kStagesF;
      if (!dead) dead = !bar_wait(empty + s, ((item / kStagesF) & 1) ^ 1, p.status);
      if (!dead) {
        unsigned char* arow = stages + s * kStageF + row * 128;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint4 acc;
          acc.x = hmul2_bits(t2[0], x2r[cc][0].x);
          acc.y = hmul2_bits(t2[0], x2r[cc][0].y);
          acc.z = hmul2_bits(t2[0], x2r[cc][0].z);
          acc.w = hmul2_bits(t2[0], x2r[cc][0].w);
#pragma unroll
          for (int jj = 1; jj < NJ; ++jj) {
            acc.x = hfma2_bits(t2[jj], x2r[cc][jj].x, acc.x);
            acc.y = hfma2_bits(t2[jj], x2r[cc][jj].y, acc.y);
            acc.z = hfma2_bits(t2[jj], x2r[cc][jj].z, acc.z);
            acc.w = hfma2_bits(t2[jj], x2r[cc][jj].w, acc.w);
          }
          *reinterpret_cast<uint4*>(arow + (((half * 4 + cc) ^ swz) << 4)) = acc;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy writes -> visible to the MMA's reads
      __syncwarp();
      if (lane == 0) bar_arrive(full + s);
    }
  }
}

// Compacts the path's coupling columns (thread 0), then runs the item loop specialised on the
// number of active columns.
template <int D1>
__device__ __forceinline__ void produce_path(const FwdParams& p, const cueq_fctp_fused_path& path, unsigned char* stages,
                                             float* coef, int* active, unsigned long long* full, unsigned long long* empty,
                                             int item0, bool& dead, int64_t z0, int ptid) {
  producers_sync();  // every producer has finished with the previous path's tables
  if (ptid == 0) {
    int nj = 0;
    for (int j = 0; j < path.d2; ++j) {
      bool any = false;
      for (int i = 0; i < D1; ++i) any |= path.c[i * 5 + j] != 0.f;
      if (any || (j == path.d2 - 1 && nj == 0)) {
        for (int i = 0; i < D1; ++i) coef[i * 5 + nj] = path.c[i * 5 + j];
        active[nj++] = j;
      }
    }
    active[7] = nj;
  }
  producers_sync();
  switch (active[7]) {
    case 1: produce_items<D1, 1>(p, path, stages, coef, active, full, empty, item0, dead, z0, ptid); break;
    case 2: produce_items<D1, 2>(p, path, stages, coef, active, full, empty, item0, dead, z0, ptid); break;
    case 3: produce_items<D1, 3>(p, path, stages, coef, active, full, empty, item0, dead, z0, ptid); break;
    case 4: produce_items<D1, 4>(p, path, stages, coef, active, full, empty, item0, dead, z0, ptid); break;
    default: produce_items<D1, 5>(p, path, stages, coef, active, full, empty, item0, dead, z0, ptid); break;
  }
}

__global__ void __launch_bounds__(kThreadsFwd, 1) fctp_fused_forward_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                         const __grid_constant__ FwdParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ringB = smem + kStagesF * kStageF;
  float* coef = reinterpret_cast<float*>(ringB + kStagesB * kTileBF);
  int* active = reinterpret_cast<int*>(coef + 32);   // active[0..4]: column ids, active[7]: their count
  unsigned long long* full = reinterpret_cast<unsigned long long*>(active + 8);
  unsigned long long* empty = full + kStagesF;
  unsigned long long* fullB = empty + kStagesF;
  unsigned long long* emptyB = fullB + kStagesB;
  unsigned long long* acc_ready = emptyB + kStagesB;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_ready + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const cueq_fctp_fused_task& task = p.tasks[blockIdx.y];
  const int64_t z0 = (int64_t)blockIdx.x * FM;
  const int total_items = task.num_paths * (FK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesF; ++s) { bar_init(full + s, kProducers / 32); bar_init(empty + s, 1); }
    for (int s = 0; s < kStagesB; ++s) { bar_init(fullB + s, 1); bar_init(emptyB + s, 1); }
    bar_init(acc_ready, kIssuers);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(tmem_slot)), "r"((unsigned)kFwdTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int item = 0; item < total_items; ++item) {
        const int s = item % kStagesB;
        if (!bar_wait(emptyB + s, ((item / kStagesB) & 1) ^ 1, p.status)) break;
        bar_expect_tx(fullB + s, kTileBF);
        const int row0 = task.paths[item / FK].w_row0 + (item % FK) * FK;
        tma_load_2d(ringB + s * kTileBF, &map_w, 0, row0, fullB + s);
      }
    }
  } else if (warp == 1 || warp >= 6 + kProducers / 32) {
    // MMA issue.  Consecutive tcgen05.mma of one thread were measured to start about 110 ns apart
    // whatever their shape, while two issuing threads overlap, so the items are dealt round-robin
    // to kIssuers threads, each with its own accumulator; the epilogue adds the accumulators.
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1 + (warp - (6 + kProducers / 32));
      // D = f32, A = B = bf16, A K-major, B MN-major ([K = (u,v)][N = w], w contiguous), N = 64, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(FN >> 3) << 17) | ((unsigned)(FM >> 4) << 24);
      for (int item = me; item < total_items; item += kIssuers) {
        const int s = item % kStagesF, sb = item % kStagesB;
        if (!bar_wait(fullB + sb, (item / kStagesB) & 1, p.status)) break;
        if (!bar_wait(full + s, (item / kStagesF) & 1, p.status)) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned long long da = smem_desc(smem + s * kStageF);
        const unsigned long long db = smem_desc_mn(ringB + sb * kTileBF);
#pragma unroll
        for (int kk = 0; kk < FK / 16; ++kk) umma_bf16(tmem_base + me * FN, da + 2ull * kk, db + 128ull * kk, idesc, (item >= kIssuers || kk != 0) ? 1u : 0u);
        umma_commit(empty + s);
        umma_commit(emptyB + sb);
      }
      umma_commit(acc_ready);
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    const bool ok = bar_wait(acc_ready, 0, p.status);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const int64_t z = z0 + q * 32 + lane;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      unsigned v[32];
      tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + half * 32, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
      for (int r = 1; r < kIssuers; ++r) {
        {
          unsigned v2[32];
          tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + r * FN + half * 32, v2);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) + __uint_as_float(v2[c]));
        }
      }
      if (ok && status_clean(p.status) && z < p.batch) {
        const int64_t off = z * p.ldo + task.out_off + half * 32;
        if (p.out_bf16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + off;
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) h[t] = __floats2bfloat162_rn(__uint_as_float(v[c + 2 * t]), __uint_as_float(v[c + 2 * t + 1]));
            *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<uint4*>(h);
          }
        } else {
          float* dst = reinterpret_cast<float*>(p.out) + off;
#pragma unroll
          for (int c = 0; c < 32; c += 4)
            *reinterpret_cast<float4*>(dst + c) = make_float4(__uint_as_float(v[c]), __uint_as_float(v[c + 1]), __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
        }
      }
    }
  } else {
    const int ptid = threadIdx.x - 192;
    bool dead = false;
    for (int pi = 0; pi < task.num_paths; ++pi) {
      const int item = pi * FK;
      const cueq_fctp_fused_path& path = task.paths[pi];
      switch (path.d1) {
        case 1: produce_path<1>(p, path, smem, coef, active, full, empty, item, dead, z0, ptid); break;
        case 3: produce_path<3>(p, path, smem, coef, active, full, empty, item, dead, z0, ptid); break;
        case 5: produce_path<5>(p, path, smem, coef, active, full, empty, item, dead, z0, ptid); break;
        default: break;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((unsigned)kFwdTmemCols) : "memory");
  }
}

// W as a 2-D bf16 array [rows = (path, u, v)][64 w]; one box = 64 rows x 64 columns.
int make_w_map(CUtensorMap* map, const void* base, int64_t rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return cueq::fail("fctp fused: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)FN, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)FN * 2};
  cuuint32_t box[2] = {(cuuint32_t)FN, (cuuint32_t)FK};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cueq::fail("fctp fused: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

int check_tasks(const cueq_fctp_fused_args* a) {
  if (a->num_tasks < 1 || a->num_tasks > CUEQ_FCTP_FUSED_MAX_TASKS) return cueq::fail("fctp fused: between 1 and %d tasks", CUEQ_FCTP_FUSED_MAX_TASKS);
  for (int t = 0; t < a->num_tasks; ++t) {
    const cueq_fctp_fused_task& task = a->tasks[t];
    if (task.num_paths < 1 || task.num_paths > CUEQ_FCTP_FUSED_MAX_PATHS) return cueq::fail("fctp fused: task %d has %d paths (1..%d)", t, task.num_paths, CUEQ_FCTP_FUSED_MAX_PATHS);
    if (task.out_off < 0 || (task.out_off % 8)) return cueq::fail("fctp fused: output offsets must be multiples of 8 elements");
    for (int q = 0; q < task.num_paths; ++q) {
      const cueq_fctp_fused_path& path = task.paths[q];
      const bool okd = (path.d1 == 1 || path.d1 == 3 || path.d1 == 5) && (path.d2 == 1 || path.d2 == 3 || path.d2 == 5);
      if (!okd) return cueq::fail("fctp fused: irrep dimensions must be 1, 3 or 5 (task %d path %d: %d, %d)", t, q, path.d1, path.d2);
      if ((path.off1 % 8) || (path.off2 % 8) || path.off1 < 0 || path.off2 < 0) return cueq::fail("fctp fused: segment offsets must be multiples of 8 elements");
      if (path.w_row0 < 0 || (int64_t)path.w_row0 + FK * FK > a->w_rows) return cueq::fail("fctp fused: weight block of task %d path %d is outside the weight array", t, q);
    }
  }
  return 0;
}


// ---- gradient with respect to one of the two data operands -------------------------------------
//
//   gXa[z, ia, a] += sum_k sum_jb C[ia, jb, k] * sum_b gZ[z, k, (a, b)] * xb[z, jb, b],
//   gZ[z, k, (a, b)] = sum_w gout[z, k, w] * W[(a, b), w]
//
// ("a" = the operand being differentiated, "b" = the other one; for x2 the caller passes a copy
// of W with rows ordered (v, u) and the transposed coupling table).  gZ is a [128 samples x 256
// (4 a, 64 b)] tile of a GEMM with K = 64: gout tile (K-major A, TMA) x W rows (K-major B, TMA),
// accumulated in TMEM (two 256-column buffers, so that the next tile's MMAs overlap the reduction
// of the current one).  Consumer warps read the tile back with tcgen05.ld and fold it against xb
// (held in shared memory) on the CUDA cores; gZ never exists in memory.
// One CTA owns (path, up to two components k, 128 samples).
// Warp roles: 0 = TMA, 1 = MMA issue + TMEM owner, 2-9 = consumers (lane quadrant = warp % 4,
// a-pair = (warp - 2) / 4).
constexpr int GN = 256;                       // columns per tile: 4 a x 64 b
constexpr int kStagesG = 3;                   // W-row ring (32 KiB each)
constexpr int kTileBG = GN * 64 * 2;          // 32 KiB
constexpr int kMaxKG = 2;                     // components per CTA
constexpr int kConsumers = 256;
constexpr int kThreadsG = 64 + kConsumers;
constexpr int kXPitch = 5 * 128 + 16;
constexpr int kXTile = FM * kXPitch;

struct GxParams {
  const __nv_bfloat16* xb;
  float* gxa;
  int64_t ldb, lda, batch;
  int* status;
  cueq_fctp_fused_unit units[CUEQ_FCTP_FUSED_MAX_UNITS];
};

__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 2, %0;\n" ::"n"(kConsumers) : "memory"); }

// Folds one [row, 2 a, 64 b] strip of a gZ tile against the NJ active rows of xb:
// r[a2][jj] = sum_b gZ[a2, b] * xb[act[jj], b].
template <int NJ>
__device__ __forceinline__ void fold_tile(unsigned tcol, const unsigned char* xrow, const int* act, float (&r)[2][5]) {
#pragma unroll
  for (int a2 = 0; a2 < 2; ++a2)
#pragma unroll
    for (int jj = 0; jj < 5; ++jj) r[a2][jj] = 0.f;
#pragma unroll
  for (int vh = 0; vh < 2; ++vh) {
    unsigned g0[32], g1[32];
    tmem_ld32(tcol + vh * 32, g0);
    tmem_ld32(tcol + 64 + vh * 32, g1);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
#pragma unroll
      for (int jj = 0; jj < NJ; ++jj) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xrow + act[jj] * 128 + (vh * 4 + c4) * 16);
        const unsigned wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = bf16_lo(wds[e]), hi = bf16_hi(wds[e]);
          r[0][jj] = fmaf(__uint_as_float(g0[c4 * 8 + 2 * e]), lo, r[0][jj]);
          r[0][jj] = fmaf(__uint_as_float(g0[c4 * 8 + 2 * e + 1]), hi, r[0][jj]);
          r[1][jj] = fmaf(__uint_as_float(g1[c4 * 8 + 2 * e]), lo, r[1][jj]);
          r[1][jj] = fmaf(__uint_as_float(g1[c4 * 8 + 2 * e + 1]), hi, r[1][jj]);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(kThreadsG, 1) fctp_fused_gx_kernel(const __grid_constant__ CUtensorMap map_g,
                                                                    const __grid_constant__ CUtensorMap map_w,
                                                                    const __grid_constant__ GxParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* tilesA = smem;                                 // kMaxKG gout tiles, 16 KiB each
  unsigned char* ringB = tilesA + kMaxKG * kTileAF;             // W rows
  unsigned char* xtile = ringB + kStagesG * kTileBG;            // xb rows of the 128 samples, bf16, padded pitch
  float* coef = reinterpret_cast<float*>(xtile + kXTile);       // [kMaxKG][25] compacted: coef[k][ia * 5 + jj]
  int* act = reinterpret_cast<int*>(coef + kMaxKG * 25 + 2);    // [kMaxKG][8]: active jb ids, [7] = their count
  unsigned long long* fullA = reinterpret_cast<unsigned long long*>(act + kMaxKG * 8);
  unsigned long long* fullB = fullA + 1;
  unsigned long long* emptyB = fullB + kStagesG;
  unsigned long long* accfull = emptyB + kStagesG;
  unsigned long long* accempty = accfull + 2;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(accempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const cueq_fctp_fused_unit& unit = p.units[blockIdx.y];
  const int64_t z0 = (int64_t)blockIdx.x * FM;
  const int nk = unit.nk;
  constexpr int kGroups = 16;   // 64 a in groups of 4

  if (threadIdx.x == 0) {
    bar_init(fullA, 1);
    for (int s = 0; s < kStagesG; ++s) { bar_init(fullB + s, 1); bar_init(emptyB + s, 1); }
    for (int b = 0; b < 2; ++b) { bar_init(accfull + b, 1); bar_init(accempty + b, kConsumers / 32); }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    // compact the coupling columns of every component of this CTA
    for (int t = 0; t < kMaxKG * 25; ++t) coef[t] = 0.f;
    for (int k = 0; k < nk; ++k) {
      int nj = 0;
      for (int j = 0; j < unit.db; ++j) {
        bool any = false;
        for (int i = 0; i < unit.da; ++i) any |= unit.c[k][i * 5 + j] != 0.f;
        if (any || (j == unit.db - 1 && nj == 0)) {
          for (int i = 0; i < 5; ++i) coef[k * 25 + i * 5 + nj] = i < unit.da ? unit.c[k][i * 5 + j] : 0.f;
          act[k * 8 + nj++] = j;
        }
      }
      act[k * 8 + 7] = nj;
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      bar_expect_tx(fullA, nk * kTileAF);
      for (int k = 0; k < nk; ++k) tma_load_2d(tilesA + k * kTileAF, &map_g, unit.goff[k], (int)z0, fullA);
      for (int g = 0; g < kGroups; ++g) {
        const int s = g % kStagesG;
        if (!bar_wait(emptyB + s, ((g / kStagesG) & 1) ^ 1, p.status)) break;
        bar_expect_tx(fullB + s, kTileBG);
        tma_load_2d(ringB + s * kTileBG, &map_w, 0, unit.w_row0 + g * GN, fullB + s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // D = f32, A = B = bf16, both K-major, N = 256, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(GN >> 3) << 17) | ((unsigned)(FM >> 4) << 24);
      bool ok = bar_wait(fullA, 0, p.status);
      int t = 0;
      for (int g = 0; g < kGroups && ok; ++g) {
        const int s = g % kStagesG;
        ok = bar_wait(fullB + s, (g / kStagesG) & 1, p.status);
        for (int k = 0; k < nk && ok; ++k, ++t) {
          const int buf = t & 1;
          ok = bar_wait(accempty + buf, ((t >> 1) & 1) ^ 1, p.status);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned long long da = smem_desc(tilesA + k * kTileAF);
          const unsigned long long db = smem_desc(ringB + s * kTileBG);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem_base + buf * GN, da + 2ull * kk, db + 2ull * kk, idesc, kk != 0 ? 1u : 0u);
          umma_commit(accfull + buf);
        }
        umma_commit(emptyB + s);
      }
    }
  } else {
    const int ctid = threadIdx.x - 64;
    const int q = warp & 3, ah = (warp - 2) >> 2;          // lane quadrant, which pair of the group's 4 a
    const int row = q * 32 + lane;
    const int64_t z = z0 + row;
    const bool valid = z < p.batch;
    const int pitch = unit.db * 128 + 16;
    for (int idx = ctid; idx < FM * unit.db * 8; idx += kConsumers) {
      const int r = idx / (unit.db * 8), c = idx % (unit.db * 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (z0 + r < p.batch) v = __ldg(reinterpret_cast<const uint4*>(p.xb + (z0 + r) * p.ldb + unit.offb) + c);
      *reinterpret_cast<uint4*>(xtile + r * pitch + c * 16) = v;
    }
    consumers_sync();
    const unsigned char* xrow = xtile + row * pitch;
    bool dead = false;
    int t = 0;
    for (int g = 0; g < kGroups; ++g) {
      float gacc[5][2];
#pragma unroll
      for (int i = 0; i < 5; ++i) gacc[i][0] = gacc[i][1] = 0.f;
      for (int k = 0; k < nk; ++k, ++t) {
        const int buf = t & 1;
        if (!dead) dead = !bar_wait(accfull + buf, (t >> 1) & 1, p.status);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        float r[2][5];
        const unsigned tcol = tmem_base + ((unsigned)(q * 32) << 16) + buf * GN + ah * 128;
        const int* actk = act + k * 8;
        switch (actk[7]) {
          case 1: fold_tile<1>(tcol, xrow, actk, r); break;
          case 2: fold_tile<2>(tcol, xrow, actk, r); break;
          case 3: fold_tile<3>(tcol, xrow, actk, r); break;
          case 4: fold_tile<4>(tcol, xrow, actk, r); break;
          default: fold_tile<5>(tcol, xrow, actk, r); break;
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) bar_arrive(accempty + buf);
        const float* ck = coef + k * 25;
#pragma unroll
        for (int i = 0; i < 5; ++i)
#pragma unroll
          for (int jj = 0; jj < 5; ++jj) {
            const float cij = ck[i * 5 + jj];   // zero beyond the active columns / rows
            gacc[i][0] = fmaf(cij, r[0][jj], gacc[i][0]);
            gacc[i][1] = fmaf(cij, r[1][jj], gacc[i][1]);
          }
      }
      if (valid && !dead && status_clean(p.status)) {
        float* dst = p.gxa + z * p.lda + unit.offa + g * 4 + ah * 2;
#pragma unroll
        for (int i = 0; i < 5; ++i)
          if (i < unit.da)
            asm volatile("red.global.add.v2.f32 [%0], {%1, %2};\n" ::"l"(dst + i * 64), "f"(gacc[i][0]), "f"(gacc[i][1]) : "memory");
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}


// ---- gradient with respect to the weights ------------------------------------------------------
//
//   gW[(u, v), w] += sum_z sum_k Z[z, k, (u, v)] * gout[z, k, w]
//
// A GEMM with K = samples: A = Z^T is built by the producer warps as an MN-major operand (rows =
// samples, 128 consecutive (u, v) = 2 u per tile), B = a [64 samples x 64 w] block of the cotangent
// (MN-major, TMA).  One CTA owns (path, component k, 16 u, a range of samples) and keeps eight [128 x 64]
// accumulators in TMEM (all 512 columns), so that x2 values, the cotangent block and the T
// products of a (component, 64-sample block) are shared by eight MMA groups.  The partial sums
// of the sample ranges are combined with red.global.add.
// Warp roles: 0 = TMA, 1 and 14 = MMA issue (1 owns TMEM), 2-5 = epilogue, 6-13 = producers.
constexpr int WK = 64;                         // samples per item (MMA K, 4 instructions)
constexpr int kStagesWA = 6;                   // A ring (16 KiB: 2 blocks of [64 samples][64 (u,v)])
constexpr int kStagesWB = 4;                   // cotangent blocks (8 KiB)
constexpr int kTilesW = 8;                     // accumulators per CTA (2 u each)

struct GwParams {
  const __nv_bfloat16* x1;
  const __nv_bfloat16* x2;
  float* gw;
  int64_t ld1, ld2, batch;
  int blocks_per_split;    // 64-sample blocks handled by one CTA
  int* status;
  cueq_fctp_fused_wunit units[CUEQ_FCTP_FUSED_MAX_WUNITS];
};

// All items of the CTA's (path, component): for every 64-sample block, 8 tiles of 2 u.
// Thread = (sample row, u within the tile, half of v); lanes 8 apart hold the two halves.
template <int D1, int NJ>
__device__ __forceinline__ void produce_gw(const GwParams& p, const cueq_fctp_fused_wunit& unit, unsigned char* ringA,
                                           const float* coef, const int* active, unsigned long long* fullA,
                                           unsigned long long* emptyA, int item, bool& dead, int64_t zb0, int nblocks,
                                           int u0, int ptid) {
  const int lane = ptid & 31;
  const int row = (ptid >> 5) * 8 + (lane & 7), ul = (lane >> 4) & 1, vh = (lane >> 3) & 1;
  float cf[D1][NJ];
#pragma unroll
  for (int i = 0; i < D1; ++i)
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) cf[i][jj] = coef[i * 5 + jj];
  const int swz = row & 7;
  for (int b = 0; b < nblocks; ++b) {
    const int64_t z = (zb0 + b) * WK + row;
    const bool valid = z < p.batch;
    uint4 x2r[4][NJ];
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) {
      const uint4* src = reinterpret_cast<const uint4*>(p.x2 + (valid ? z : 0) * p.ld2 + unit.off2 + active[jj] * 64) + vh * 4;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) x2r[cc][jj] = valid ? __ldg(src + cc) : make_uint4(0, 0, 0, 0);
    }
    const unsigned short* x1row = reinterpret_cast<const unsigned short*>(p.x1 + (valid ? z : 0) * p.ld1 + unit.off1) + u0 + ul;
    for (int t2i = 0; t2i < kTilesW; t2i += 2) {
      // the two v-halves of a (row, u) compute T for tiles t2i and t2i + 1 and exchange them
      unsigned tmine[NJ];
      {
        const int u = (t2i + vh) * 2;
        float xf[D1];
#pragma unroll
        for (int i = 0; i < D1; ++i) xf[i] = valid ? bf16_lo(__ldg(x1row + i * 64 + u)) : 0.f;
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) {
          float t = cf[0][jj] * xf[0];
#pragma unroll
          for (int i = 1; i < D1; ++i) t = fmaf(cf[i][jj], xf[i], t);
          tmine[jj] = pack_same(t);
        }
      }
#pragma unroll
      for (int q = 0; q < 2; ++q, ++item) {
        unsigned t2[NJ];
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) t2[jj] = __shfl_sync(0xffffffffu, tmine[jj], (lane & ~8) | (q << 3));
        const int s = item % kStagesWA;
        if (!dead) dead = !bar_wait(emptyA + s, ((item / kStagesWA) & 1) ^ 1, p.status);
        if (!dead) {
          unsigned char* arow = ringA + s * kTileAF + ul * 8192 + row * 128;
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            uint4 acc;
            acc.x = hmul2_bits(t2[0], x2r[cc][0].x);
            acc.y = hmul2_bits(t2[0], x2r[cc][0].y);
            acc.z = hmul2_bits(t2[0], x2r[cc][0].z);
            acc.w = hmul2_bits(t2[0], x2r[cc][0].w);
#pragma unroll
            for (int jj = 1; jj < NJ; ++jj) {
              acc.x = hfma2_bits(t2[jj], x2r[cc][jj].x, acc.x);
              acc.y = hfma2_bits(t2[jj], x2r[cc][jj].y, acc.y);
              acc.z = hfma2_bits(t2[jj], x2r[cc][jj].z, acc.z);
              acc.w = hfma2_bits(t2[jj], x2r[cc][jj].w, acc.w);
            }
            *reinterpret_cast<uint4*>(arow + (((vh * 4 + cc) ^ swz) << 4)) = acc;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) bar_arrive(fullA + s);
      }
    }
  }
}

template <int D1>
__device__ __forceinline__ void produce_gw_k(const GwParams& p, const cueq_fctp_fused_wunit& unit, unsigned char* ringA,
                                             float* coef, int* active, unsigned long long* fullA, unsigned long long* emptyA,
                                             int item, bool& dead, int64_t zb0, int nblocks, int u0, int ptid) {
  producers_sync();
  if (ptid == 0) {
    int nj = 0;
    for (int j = 0; j < unit.d2; ++j) {
      bool any = false;
      for (int i = 0; i < D1; ++i) any |= unit.c[i * 5 + j] != 0.f;
      if (any || (j == unit.d2 - 1 && nj == 0)) {
        for (int i = 0; i < D1; ++i) coef[i * 5 + nj] = unit.c[i * 5 + j];
        active[nj++] = j;
      }
    }
    active[7] = nj;
  }
  producers_sync();
  switch (active[7]) {
    case 1: produce_gw<D1, 1>(p, unit, ringA, coef, active, fullA, emptyA, item, dead, zb0, nblocks, u0, ptid); break;
    case 2: produce_gw<D1, 2>(p, unit, ringA, coef, active, fullA, emptyA, item, dead, zb0, nblocks, u0, ptid); break;
    case 3: produce_gw<D1, 3>(p, unit, ringA, coef, active, fullA, emptyA, item, dead, zb0, nblocks, u0, ptid); break;
    case 4: produce_gw<D1, 4>(p, unit, ringA, coef, active, fullA, emptyA, item, dead, zb0, nblocks, u0, ptid); break;
    default: produce_gw<D1, 5>(p, unit, ringA, coef, active, fullA, emptyA, item, dead, zb0, nblocks, u0, ptid); break;
  }
}

__global__ void __launch_bounds__(kThreadsFwd, 1) fctp_fused_gw_kernel(const __grid_constant__ CUtensorMap map_g,
                                                                    const __grid_constant__ GwParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ringA = smem;
  unsigned char* ringB = ringA + kStagesWA * kTileAF;
  float* coef = reinterpret_cast<float*>(ringB + kStagesWB * kTileBF);
  int* active = reinterpret_cast<int*>(coef + 32);
  unsigned long long* fullA = reinterpret_cast<unsigned long long*>(active + 8);
  unsigned long long* emptyA = fullA + kStagesWA;
  unsigned long long* fullB = emptyA + kStagesWA;
  unsigned long long* emptyB = fullB + kStagesWB;
  unsigned long long* acc_ready = emptyB + kStagesWB;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_ready + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const cueq_fctp_fused_wunit& unit = p.units[blockIdx.y];
  const int u0 = blockIdx.z * (2 * kTilesW);
  const int total_blocks = (int)((p.batch + WK - 1) / WK);
  const int64_t zb0 = (int64_t)blockIdx.x * p.blocks_per_split;
  const int nblocks = min(p.blocks_per_split, total_blocks - (int)zb0);
  const int ngroups = nblocks;                 // one cotangent block per 64 samples

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesWA; ++s) { bar_init(fullA + s, kProducers / 32); bar_init(emptyA + s, 1); }
    for (int s = 0; s < kStagesWB; ++s) { bar_init(fullB + s, 1); bar_init(emptyB + s, kIssuers); }
    bar_init(acc_ready, kIssuers);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int g = 0; g < ngroups; ++g) {
        const int s = g % kStagesWB;
        if (!bar_wait(emptyB + s, ((g / kStagesWB) & 1) ^ 1, p.status)) break;
        bar_expect_tx(fullB + s, kTileBF);
        tma_load_2d(ringB + s * kTileBF, &map_g, unit.goff, (int)((zb0 + g) * WK), fullB + s);
      }
    }
  } else if (warp == 1 || warp >= 6 + kProducers / 32) {
    // kIssuers threads issue the MMAs (see the forward kernel): issuer r owns tiles t = r, r + kIssuers, ...
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1 + (warp - (6 + kProducers / 32));
      // D = f32, A = B = bf16, both MN-major, N = 64, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((unsigned)(FN >> 3) << 17) | ((unsigned)(FM >> 4) << 24);
      bool ok = true;
      for (int g = 0; g < ngroups && ok; ++g) {
        const int sb = g % kStagesWB;
        ok = bar_wait(fullB + sb, (g / kStagesWB) & 1, p.status);
        const unsigned long long db = smem_desc_mn(ringB + sb * kTileBF);
        for (int t = me; t < kTilesW && ok; t += kIssuers) {
          const int item = g * kTilesW + t;
          const int s = item % kStagesWA;
          ok = bar_wait(fullA + s, (item / kStagesWA) & 1, p.status);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned long long da = smem_desc_mn(ringA + s * kTileAF);
#pragma unroll
          for (int kk = 0; kk < WK / 16; ++kk) umma_bf16(tmem_base + t * FN, da + 128ull * kk, db + 128ull * kk, idesc, (g | kk) != 0 ? 1u : 0u);
          umma_commit(emptyA + s);
        }
        umma_commit(emptyB + sb);
      }
      umma_commit(acc_ready);
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    const bool ok = bar_wait(acc_ready, 0, p.status);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const int m = q * 32 + lane;       // row of the tile: (u within the pair) * 64 + v
    for (int t = 0; t < kTilesW; ++t) {
      float* dst = p.gw + ((int64_t)unit.w_row0 + (int64_t)(u0 + 2 * t) * 64 + m) * 64;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        unsigned v[32];
        tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + t * FN + half * 32, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (ok && status_clean(p.status) && ngroups > 0) {
#pragma unroll
          for (int c = 0; c < 32; c += 4)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(dst + half * 32 + c), "f"(__uint_as_float(v[c])),
                         "f"(__uint_as_float(v[c + 1])), "f"(__uint_as_float(v[c + 2])), "f"(__uint_as_float(v[c + 3])) : "memory");
        }
      }
    }
  } else {
    const int ptid = threadIdx.x - 192;
    bool dead = false;
    switch (unit.d1) {
      case 1: produce_gw_k<1>(p, unit, ringA, coef, active, fullA, emptyA, 0, dead, zb0, nblocks, u0, ptid); break;
      case 3: produce_gw_k<3>(p, unit, ringA, coef, active, fullA, emptyA, 0, dead, zb0, nblocks, u0, ptid); break;
      case 5: produce_gw_k<5>(p, unit, ringA, coef, active, fullA, emptyA, 0, dead, zb0, nblocks, u0, ptid); break;
      default: break;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

int make_map_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return cueq::fail("fctp fused: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cueq::fail("fctp fused: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

}  // namespace

extern "C" int cueq_b200_fctp_fused_forward(const cueq_fctp_fused_args* a, void* stream) {
  if (!a || !a->x1 || !a->x2 || !a->w || !a->out || !a->tasks) return cueq::fail("fctp fused: null argument");
  if (a->batch <= 0) return 0;
  if (int rc = check_tasks(a)) return rc;
  if ((a->ld1 % 8) || (a->ld2 % 8) || (a->ldo % 8)) return cueq::fail("fctp fused: row pitches must be multiples of 8 elements");
  if (((uintptr_t)a->x1 | (uintptr_t)a->x2 | (uintptr_t)a->w | (uintptr_t)a->out) & 15) return cueq::fail("fctp fused: operands must be 16-byte aligned");
  if (a->out_dtype != CUEQ_F32 && a->out_dtype != CUEQ_BF16) return cueq::fail("fctp fused: output must be float32 or bfloat16");
  CUtensorMap mw;
  if (int rc = make_w_map(&mw, a->w, a->w_rows)) return rc;
  FwdParams p;
  std::memset(&p, 0, sizeof(p));
  p.x1 = reinterpret_cast<const __nv_bfloat16*>(a->x1);
  p.x2 = reinterpret_cast<const __nv_bfloat16*>(a->x2);
  p.out = a->out;
  p.ld1 = a->ld1; p.ld2 = a->ld2; p.ldo = a->ldo; p.batch = a->batch;
  p.out_bf16 = a->out_dtype == CUEQ_BF16;
  p.status = reinterpret_cast<int*>(a->status);
  std::memcpy(p.tasks, a->tasks, sizeof(cueq_fctp_fused_task) * a->num_tasks);
  const size_t smem = kStagesF * kStageF + kStagesB * kTileBF + 160 + 40 * 8 + 1024;
  static cueq::PerDeviceFlag configured;
  if (!configured.get()) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(fctp_fused_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set();
  }
  dim3 grid((unsigned)((a->batch + FM - 1) / FM), (unsigned)a->num_tasks);
  fctp_fused_forward_kernel<<<grid, kThreadsFwd, smem, reinterpret_cast<cudaStream_t>(stream)>>>(mw, p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}


extern "C" int cueq_b200_fctp_fused_gx(const cueq_fctp_fused_gx_args* a, void* stream) {
  if (!a || !a->xb || !a->gout || !a->w || !a->gxa || !a->units) return cueq::fail("fctp fused gx: null argument");
  if (a->batch <= 0) return 0;
  if (a->num_units < 1 || a->num_units > CUEQ_FCTP_FUSED_MAX_UNITS) return cueq::fail("fctp fused gx: between 1 and %d units", CUEQ_FCTP_FUSED_MAX_UNITS);
  for (int t = 0; t < a->num_units; ++t) {
    const cueq_fctp_fused_unit& u = a->units[t];
    const bool okd = (u.da == 1 || u.da == 3 || u.da == 5) && (u.db == 1 || u.db == 3 || u.db == 5);
    if (!okd) return cueq::fail("fctp fused gx: irrep dimensions must be 1, 3 or 5 (unit %d: %d, %d)", t, u.da, u.db);
    if (u.nk < 1 || u.nk > 2) return cueq::fail("fctp fused gx: a unit covers 1 or 2 components (unit %d: %d)", t, u.nk);
    if (u.offa < 0 || u.offb < 0 || (u.offa % 8) || (u.offb % 8)) return cueq::fail("fctp fused gx: segment offsets must be non-negative multiples of 8 elements");
    if (u.offa + u.da * 64 > a->lda || u.offb + u.db * 64 > a->ldb) return cueq::fail("fctp fused gx: segment of unit %d exceeds the row", t);
    for (int k = 0; k < u.nk; ++k)
      if (u.goff[k] < 0 || (u.goff[k] % 8) || u.goff[k] + 64 > a->ldg) return cueq::fail("fctp fused gx: cotangent block of unit %d is outside the row", t);
    if (u.w_row0 < 0 || (int64_t)u.w_row0 + 4096 > a->w_rows) return cueq::fail("fctp fused gx: weight block of unit %d is outside the weight array", t);
  }
  if ((a->lda % 2) || (a->ldb % 8) || (a->ldg % 8)) return cueq::fail("fctp fused gx: row pitches must keep rows aligned (xb, gout: 8 elements; gxa: 2)");
  if (((uintptr_t)a->xb | (uintptr_t)a->gout | (uintptr_t)a->w) & 15) return cueq::fail("fctp fused gx: operands must be 16-byte aligned");
  if ((uintptr_t)a->gxa & 7) return cueq::fail("fctp fused gx: the gradient must be 8-byte aligned");
  if (a->batch > 2147483647LL) return cueq::fail("fctp fused gx: batch too large");
  CUtensorMap mg, mw;
  if (int rc = make_map_2d(&mg, a->gout, a->batch, a->ldg, a->ldg, 64, FM)) return rc;
  if (int rc = make_map_2d(&mw, a->w, a->w_rows, 64, 64, 64, GN)) return rc;
  GxParams p;
  std::memset(&p, 0, sizeof(p));
  p.xb = reinterpret_cast<const __nv_bfloat16*>(a->xb);
  p.gxa = reinterpret_cast<float*>(a->gxa);
  p.ldb = a->ldb; p.lda = a->lda; p.batch = a->batch;
  p.status = reinterpret_cast<int*>(a->status);
  std::memcpy(p.units, a->units, sizeof(cueq_fctp_fused_unit) * a->num_units);
  const size_t smem = kMaxKG * kTileAF + kStagesG * kTileBG + kXTile + 512 + 1024;
  static cueq::PerDeviceFlag configured;
  if (!configured.get()) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(fctp_fused_gx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set();
  }
  dim3 grid((unsigned)((a->batch + FM - 1) / FM), (unsigned)a->num_units);
  fctp_fused_gx_kernel<<<grid, kThreadsG, smem, reinterpret_cast<cudaStream_t>(stream)>>>(mg, mw, p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}


extern "C" int cueq_b200_fctp_fused_gw(const cueq_fctp_fused_gw_args* a, void* stream) {
  if (!a || !a->x1 || !a->x2 || !a->gout || !a->gw || !a->units) return cueq::fail("fctp fused gw: null argument");
  if (a->batch <= 0) return 0;
  if (a->num_units < 1 || a->num_units > CUEQ_FCTP_FUSED_MAX_WUNITS) return cueq::fail("fctp fused gw: between 1 and %d units", CUEQ_FCTP_FUSED_MAX_WUNITS);
  for (int t = 0; t < a->num_units; ++t) {
    const cueq_fctp_fused_wunit& u = a->units[t];
    const bool okd = (u.d1 == 1 || u.d1 == 3 || u.d1 == 5) && (u.d2 == 1 || u.d2 == 3 || u.d2 == 5);
    if (!okd) return cueq::fail("fctp fused gw: irrep dimensions must be 1, 3 or 5 (unit %d)", t);
    if (u.off1 < 0 || u.off2 < 0 || (u.off1 % 8) || (u.off2 % 8)) return cueq::fail("fctp fused gw: segment offsets must be non-negative multiples of 8 elements");
    if (u.off1 + u.d1 * 64 > a->ld1 || u.off2 + u.d2 * 64 > a->ld2) return cueq::fail("fctp fused gw: segment of unit %d exceeds the row", t);
    if (u.goff < 0 || (u.goff % 8) || u.goff + 64 > a->ldg) return cueq::fail("fctp fused gw: cotangent block of unit %d is outside the row", t);
    if (u.w_row0 < 0 || (int64_t)u.w_row0 + 4096 > a->w_rows) return cueq::fail("fctp fused gw: weight block of unit %d is outside the weight array", t);
  }
  if ((a->ld1 % 8) || (a->ld2 % 8) || (a->ldg % 8)) return cueq::fail("fctp fused gw: row pitches must be multiples of 8 elements");
  if (((uintptr_t)a->x1 | (uintptr_t)a->x2 | (uintptr_t)a->gout | (uintptr_t)a->gw) & 15) return cueq::fail("fctp fused gw: operands must be 16-byte aligned");
  if (a->batch > 2147483647LL - 64) return cueq::fail("fctp fused gw: batch too large");
  CUtensorMap mg;
  if (int rc = make_map_2d(&mg, a->gout, a->batch, a->ldg, a->ldg, 64, WK)) return rc;
  GwParams p;
  std::memset(&p, 0, sizeof(p));
  p.x1 = reinterpret_cast<const __nv_bfloat16*>(a->x1);
  p.x2 = reinterpret_cast<const __nv_bfloat16*>(a->x2);
  p.gw = reinterpret_cast<float*>(a->gw);
  p.ld1 = a->ld1; p.ld2 = a->ld2; p.batch = a->batch;
  p.status = reinterpret_cast<int*>(a->status);
  std::memcpy(p.units, a->units, sizeof(cueq_fctp_fused_wunit) * a->num_units);
  // sample ranges: enough CTAs to fill the GPU about four times over, at least 8 blocks each
  const int total_blocks = (int)((a->batch + WK - 1) / WK);
  int splits = (592 + a->num_units * 4 - 1) / (a->num_units * 4);
  if (splits > total_blocks / 8) splits = total_blocks / 8;
  if (splits < 1) splits = 1;
  p.blocks_per_split = (total_blocks + splits - 1) / splits;
  splits = (total_blocks + p.blocks_per_split - 1) / p.blocks_per_split;
  const size_t smem = kStagesWA * kTileAF + kStagesWB * kTileBF + 512 + 1024;
  static cueq::PerDeviceFlag configured;
  if (!configured.get()) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(fctp_fused_gw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set();
  }
  dim3 grid((unsigned)splits, (unsigned)a->num_units, 64 / (2 * kTilesW));
  fctp_fused_gw_kernel<<<grid, kThreadsFwd, smem, reinterpret_cast<cudaStream_t>(stream)>>>(mg, p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

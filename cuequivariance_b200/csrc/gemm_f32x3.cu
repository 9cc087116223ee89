// float32-accurate GEMM on the tensor cores: C[M,N] = A[M,K] * B[N,K]^T (+ bias[N]), K a multiple of 32.
//
// The dense layer that turns per-edge radial features into the per-edge weights of a channelwise
// tensor product (h[E,64] x W[2944,64]^T -> w[E,2944]; the pattern of
// cuequivariance_torch/layers/tp_conv_fully_connected.py:145-152,219-238) is too large for the
// CUDA cores to be cheap (0.39 TFLOP at 1M edges) and must keep float32 accuracy, which one TF32
// pass (10 mantissa bits) does not.  Each operand is therefore split into two TF32-exact halves,
// x = hi + lo with hi = x rounded to TF32 (19 bits) and lo = (x - hi) rounded likewise, and three
// tcgen05.mma kind::tf32 passes accumulate hi*hi + hi*lo + lo*hi in float32 in TMEM; the dropped
// lo*lo term and the rounding of lo are below 2^-21 relative.
//
// One CTA owns 128 rows of A: the tile arrives by TMA and is split in place by four warps (the
// operation is element-wise, so it does not care about the 128-byte swizzle); B arrives already
// split (two float32 arrays prepared once by the caller) in 128-row tiles; two threads issue the
// MMAs for alternate column tiles out of a ring of B blocks, each with its own pair of TMEM
// accumulators, and eight epilogue warps add the bias and send the rows out through shared memory
// and TMA stores (whole 128-byte lines).
// Warp roles: 0 = TMA, 1 and 10 = MMA issue (1 owns TMEM), 2-5 and 11-14 = epilogue, 6-9 = split.
// Every wait is bounded (status word 2 on timeout; the CTA still reaches its end and frees TMEM).
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

using namespace cueq_tc;

constexpr int XM = 128, XN = 128, XKB = 32;            // tile; XKB float32 = 128 bytes = one swizzle row
constexpr int kBlkA = XM * XKB * 4;                     // 16 KiB per K block of A
constexpr int kBlkB = XN * XKB * 4;                     // 16 KiB per K block of a B tile
constexpr int kMaxKB = 2;                               // K <= 64
constexpr int kThreadsX = 11 * 32;
constexpr int kThreadsRes = 15 * 32;                    // the resident-A kernel has four more epilogue warps

struct XParams {
  float* C;
  const float* bias;
  int64_t ldc;
  int M, N, nkb;
  int* status;
};

__device__ __forceinline__ void umma_tf32(unsigned tmem_c, unsigned long long da, unsigned long long db, unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
               ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// float32 bits rounded to TF32 (10 mantissa bits, ties away from zero; the low 13 bits come out zero)
__device__ __forceinline__ unsigned rna_tf32(unsigned bits) {
  unsigned r;
  asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(__uint_as_float(bits)));
  return r;
}
__device__ __forceinline__ void tmem_ld32x(unsigned taddr, unsigned (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                 "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                 "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void bar_arrive1(unsigned long long* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(s32(b)) : "memory");
}

__global__ void __launch_bounds__(kThreadsRes, 1) gemm_f32x3_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                  const __grid_constant__ CUtensorMap map_bhi,
                                                                  const __grid_constant__ CUtensorMap map_blo,
                                                                  const __grid_constant__ CUtensorMap map_c,
                                                                  const XParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* a_hi = smem;                                  // [nkb][128 rows][128 B]
  unsigned char* a_lo = a_hi + kMaxKB * kBlkA;
  unsigned char* b_st = a_lo + kMaxKB * kBlkA;                 // kBStages x (hi + lo) of one K block of one column tile
  constexpr int kStageB = 2 * kBlkB;
  // four stages: with items dealt tile by tile to two issuers, stage s is then always consumed by the same
  // issuer, so every waiter sees consecutive phases of its barriers (with two stages an issuer would skip a
  // phase and the parity test would alias)
  constexpr int kBStages = 4;
  unsigned char* stage_c = b_st + kBStages * kStageB;          // per epilogue warp: [32 rows][128 B], swizzled
  unsigned long long* fullA = reinterpret_cast<unsigned long long*>(stage_c + 8 * 4096);
  unsigned long long* readyA = fullA + 1;
  unsigned long long* fullB = readyA + 1;      // [4]
  unsigned long long* emptyB = fullB + 4;      // [4]
  unsigned long long* accfull = emptyB + 4;    // [4]
  unsigned long long* accempty = accfull + 4;  // [4]
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(accempty + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * XM;
  const int ntiles = (p.N + XN - 1) / XN;
  const int nkb = p.nkb;

  if (threadIdx.x == 0) {
    bar_init(fullA, 1);
    bar_init(readyA, 4);
    for (int s = 0; s < kBStages; ++s) { bar_init(fullB + s, 1); bar_init(emptyB + s, 1); }
    for (int b = 0; b < 4; ++b) { bar_init(accfull + b, 1); bar_init(accempty + b, 8); }
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
      bar_expect_tx(fullA, nkb * kBlkA);
      for (int kb = 0; kb < nkb; ++kb) tma_load_2d(a_hi + kb * kBlkA, &map_a, kb * XKB, m0, fullA);
      // items = (column tile, K block) in order; the ring runs up to four items ahead of the MMAs,
      // which hides the L2 latency of the loads
      for (int item = 0; item < ntiles * nkb; ++item) {
        const int s = item % kBStages;
        const int t = item / nkb, kb = item % nkb;
        if (!bar_wait(emptyB + s, ((item / kBStages) & 1) ^ 1, p.status)) break;
        bar_expect_tx(fullB + s, kStageB);
        unsigned char* st = b_st + s * kStageB;
        tma_load_2d(st, &map_bhi, kb * XKB, t * XN, fullB + s);
        tma_load_2d(st + kBlkB, &map_blo, kb * XKB, t * XN, fullB + s);
      }
    }
  } else if (warp == 1 || warp == 10) {
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1;
      // D = f32, A = B = tf32, both K-major, N = 128, M = 128
      const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(XN >> 3) << 17) | ((unsigned)(XM >> 4) << 24);
      bool ok = bar_wait(readyA, 0, p.status);
      for (int t = me; t < ntiles && ok; t += 2) {
        const int n = t >> 1;                 // this issuer's n-th tile
        const int buf = me * 2 + (n & 1);
        ok = bar_wait(accempty + buf, ((n >> 1) & 1) ^ 1, p.status);
        unsigned acc = 0;
        for (int kb = 0; kb < nkb && ok; ++kb) {
          const int item = t * nkb + kb, s = item % kBStages;
          ok = bar_wait(fullB + s, (item / kBStages) & 1, p.status);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned char* st = b_st + s * kStageB;
          const unsigned long long dah = smem_desc(a_hi + kb * kBlkA), dal = smem_desc(a_lo + kb * kBlkA);
          const unsigned long long dbh = smem_desc(st), dbl = smem_desc(st + kBlkB);
#pragma unroll
          for (int kk = 0; kk < XKB / 8; ++kk) {   // one instruction covers 8 float32 of K = 32 bytes = 2 descriptor units
            umma_tf32(tmem_base + buf * XN, dal + 2ull * kk, dbh + 2ull * kk, idesc, acc);
            acc = 1;
            umma_tf32(tmem_base + buf * XN, dah + 2ull * kk, dbl + 2ull * kk, idesc, 1u);
            umma_tf32(tmem_base + buf * XN, dah + 2ull * kk, dbh + 2ull * kk, idesc, 1u);
          }
          umma_commit(emptyB + s);
        }
        if (!ok) break;
        umma_commit(accfull + buf);
      }
    }
  } else if (warp < 6 || warp > 10) {
    // eight epilogue warps: lane quadrant = warp % 4; warps 2-5 take columns 0-63 of a tile, warps 11-14 columns 64-127
    const int q = warp & 3, ph = warp > 10 ? 1 : 0, ew = ph * 4 + q;
    bool dead = false;
    for (int t = 0; t < ntiles; ++t) {
      const int me = t & 1, n = t >> 1;
      const int buf = me * 2 + (n & 1);
      if (!dead) dead = !bar_wait(accfull + buf, (n >> 1) & 1, p.status);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
      for (int pp = 0; pp < 2; ++pp) {
        const int part = ph * 2 + pp;
        unsigned v[32];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                     "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                     "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                       "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                       "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                       "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                     : "r"(tmem_base + ((unsigned)(q * 32) << 16) + buf * XN + part * 32));
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        const int col0 = t * XN + part * 32;
        // rows leave through shared memory and a TMA store, so that global writes are whole 128-byte
        // lines (a lane-per-row store would touch 32 rows per instruction)
        unsigned char* mine = stage_c + ew * 4096;
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");   // the previous store has read the buffer
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          float4 o = make_float4(__uint_as_float(v[c]), __uint_as_float(v[c + 1]), __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
          if (p.bias && col0 + c < p.N) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + c));
            o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
          }
          *reinterpret_cast<float4*>(mine + lane * 128 + (((c >> 2) ^ (lane & 7)) << 4)) = o;
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (!dead && status_clean(p.status) && col0 < p.N && m0 + q * 32 < p.M)
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n"
                         ::"l"(&map_c), "r"(s32(mine)), "r"(col0), "r"(m0 + q * 32) : "memory");
          asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive1(accempty + buf);
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
  } else if (warp < 10) {
    // split the A tile: hi overwrites the raw values, lo goes to the twin buffer at the same offset
    const int tid = threadIdx.x - 6 * 32;
    const bool ok = bar_wait(fullA, 0, p.status);
    if (ok) {
      uint4* hi = reinterpret_cast<uint4*>(a_hi);
      uint4* lo = reinterpret_cast<uint4*>(a_lo);
      for (int idx = tid; idx < nkb * kBlkA / 16; idx += 128) {
        uint4 x = hi[idx], h, l;
        h.x = rna_tf32(x.x); h.y = rna_tf32(x.y); h.z = rna_tf32(x.z); h.w = rna_tf32(x.w);
        l.x = rna_tf32(__float_as_uint(__uint_as_float(x.x) - __uint_as_float(h.x)));
        l.y = rna_tf32(__float_as_uint(__uint_as_float(x.y) - __uint_as_float(h.y)));
        l.z = rna_tf32(__float_as_uint(__uint_as_float(x.z) - __uint_as_float(h.z)));
        l.w = rna_tf32(__float_as_uint(__uint_as_float(x.w) - __uint_as_float(h.w)));
        hi[idx] = h;
        lo[idx] = l;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) bar_arrive1(readyA);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- the same product for any K (a multiple of 32): both operands stream through a ring -----------
//
// Used when K is large (the input gradient of the layer above: gout[E,2944] x W[2944,64]).  Per
// 32-wide K block a stage holds the raw A block (split in place by four warps into hi / lo twins)
// and the matching pre-split B blocks; two threads issue the MMAs of alternate K blocks, dealt
// round-robin to several accumulators, which the epilogue adds.  Warp roles as above.
template <int NT>
struct StreamCfg {
  static constexpr int kBlkBn = NT * XKB * 4;
  static constexpr int kStage = 2 * kBlkA + 2 * kBlkBn;
  static constexpr int kStages = NT == 128 ? 3 : 4;
  // The tensor core's float32 accumulation is not round-to-nearest: along one accumulator the error
  // grew linearly with the number of instructions (3e-4 at K = 2944 against 1.4e-5 for a CUDA-core
  // float32 GEMM).  K blocks are therefore dealt round-robin to kAcc accumulators (all 512 TMEM
  // columns), which the epilogue adds on the CUDA cores.
  static constexpr int kAcc = 512 / NT;
};

template <int NT>
__global__ void __launch_bounds__(kThreadsX, 1) gemm_f32x3_stream_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                         const __grid_constant__ CUtensorMap map_bhi,
                                                                         const __grid_constant__ CUtensorMap map_blo,
                                                                         const __grid_constant__ CUtensorMap map_c,
                                                                         const XParams p) {
  using Cfg = StreamCfg<NT>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* stage_c = smem + Cfg::kStages * Cfg::kStage;     // per epilogue warp: 2 x [32 rows][128 B], swizzled
  unsigned long long* fullraw = reinterpret_cast<unsigned long long*>(stage_c + 4 * 2 * 4096);
  unsigned long long* ready = fullraw + Cfg::kStages;
  unsigned long long* empty = ready + Cfg::kStages;
  unsigned long long* acc_ready = empty + Cfg::kStages;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_ready + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * XM, n0 = blockIdx.y * NT;
  const int nkb = p.nkb;
  constexpr unsigned kCols = 512;      // Cfg::kAcc accumulators

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) { bar_init(fullraw + s, 1); bar_init(ready + s, 4); bar_init(empty + s, 1); }
    bar_init(acc_ready, 2);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(tmem_slot)), "r"(kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % Cfg::kStages;
        if (!bar_wait(empty + s, ((kb / Cfg::kStages) & 1) ^ 1, p.status)) break;
        unsigned char* st = smem + s * Cfg::kStage;
        bar_expect_tx(fullraw + s, kBlkA + 2 * Cfg::kBlkBn);
        tma_load_2d(st, &map_a, kb * XKB, m0, fullraw + s);
        tma_load_2d(st + 2 * kBlkA, &map_bhi, kb * XKB, n0, fullraw + s);
        tma_load_2d(st + 2 * kBlkA + Cfg::kBlkBn, &map_blo, kb * XKB, n0, fullraw + s);
      }
    }
  } else if (warp == 1 || warp == 10) {
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1;
      const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(NT >> 3) << 17) | ((unsigned)(XM >> 4) << 24);
      for (int kb = me; kb < nkb; kb += 2) {
        const int s = kb % Cfg::kStages;
        if (!bar_wait(ready + s, (kb / Cfg::kStages) & 1, p.status)) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned char* st = smem + s * Cfg::kStage;
        const unsigned long long dah = smem_desc(st), dal = smem_desc(st + kBlkA);
        const unsigned long long dbh = smem_desc(st + 2 * kBlkA), dbl = smem_desc(st + 2 * kBlkA + Cfg::kBlkBn);
        const unsigned tacc = tmem_base + (kb % Cfg::kAcc) * NT;
        unsigned acc = kb >= Cfg::kAcc ? 1u : 0u;   // first block of this accumulator overwrites
#pragma unroll
        for (int kk = 0; kk < XKB / 8; ++kk) {
          umma_tf32(tacc, dal + 2ull * kk, dbh + 2ull * kk, idesc, acc);
          acc = 1;
          umma_tf32(tacc, dah + 2ull * kk, dbl + 2ull * kk, idesc, 1u);
          umma_tf32(tacc, dah + 2ull * kk, dbh + 2ull * kk, idesc, 1u);
        }
        umma_commit(empty + s);
      }
      umma_commit(acc_ready);
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    const bool ok = bar_wait(acc_ready, 0, p.status);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
    for (int part = 0; part < NT / 32; ++part) {
      unsigned v[32];
      tmem_ld32x(tmem_base + ((unsigned)(q * 32) << 16) + part * 32, v);
      for (int a = 1; a < Cfg::kAcc && a < nkb; ++a) {   // accumulators that received at least one K block
        unsigned v2[32];
        tmem_ld32x(tmem_base + ((unsigned)(q * 32) << 16) + a * NT + part * 32, v2);
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) + __uint_as_float(v2[c]));
      }
      const int col0 = n0 + part * 32;
      unsigned char* mine = stage_c + (q * 2 + (part & 1)) * 4096;
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        float4 o = make_float4(__uint_as_float(v[c]), __uint_as_float(v[c + 1]), __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
        if (p.bias && col0 + c < p.N) {
          const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + c));
          o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
        }
        *reinterpret_cast<float4*>(mine + lane * 128 + (((c >> 2) ^ (lane & 7)) << 4)) = o;
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (ok && status_clean(p.status) && col0 < p.N && m0 + q * 32 < p.M)
          asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n"
                       ::"l"(&map_c), "r"(s32(mine)), "r"(col0), "r"(m0 + q * 32) : "memory");
        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
  } else if (warp < 10) {
    const int tid = threadIdx.x - 6 * 32;
    bool dead = false;
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % Cfg::kStages;
      if (!dead) dead = !bar_wait(fullraw + s, (kb / Cfg::kStages) & 1, p.status);
      if (!dead) {
        uint4* hi = reinterpret_cast<uint4*>(smem + s * Cfg::kStage);
        uint4* lo = reinterpret_cast<uint4*>(smem + s * Cfg::kStage + kBlkA);
#pragma unroll 4
        for (int idx = tid; idx < kBlkA / 16; idx += 128) {
          uint4 x = hi[idx], h, l;
          h.x = rna_tf32(x.x); h.y = rna_tf32(x.y); h.z = rna_tf32(x.z); h.w = rna_tf32(x.w);
          l.x = rna_tf32(__float_as_uint(__uint_as_float(x.x) - __uint_as_float(h.x)));
          l.y = rna_tf32(__float_as_uint(__uint_as_float(x.y) - __uint_as_float(h.y)));
          l.z = rna_tf32(__float_as_uint(__uint_as_float(x.z) - __uint_as_float(h.z)));
          l.w = rna_tf32(__float_as_uint(__uint_as_float(x.w) - __uint_as_float(h.w)));
          hi[idx] = h;
          lo[idx] = l;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive1(ready + s);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kCols) : "memory");
  }
}

// ---- reduction over rows: C[M,N] += sum_k A[k,M] * B[k,N]  (and colsum[M] += sum_k A[k,M]) --------
//
// The weight gradient of a dense layer (gout[E,2944]^T x h[E,64]) and its bias gradient.  Both
// operands are stored with the reduction index as the row, i.e. transposed with respect to what
// the K-major MMA wants: raw [32 x 128] / [32 x 64] blocks arrive by TMA without swizzle, and the
// eight split warps transpose them while they split them, writing K-major 128-byte-swizzled hi / lo
// tiles (a thread reads four consecutive k of one column and stores one 16-byte chunk, so reads
// and writes are both free of bank conflicts).  A constant extra row of B holding ones gives the
// column sums of A from the same MMAs.  The K range is cut into slices of kTnBlocks blocks per CTA
// (short accumulation chains, see StreamCfg) whose partial results are added with red.global.add.
constexpr int TN_N = 64;                       // columns of B per CTA
constexpr int TN_NB = 80;                      // rows of the B operand tile: 64 + ones row + padding to a multiple of 16
constexpr int kTnRawA = 32 * XM * 4;           // 16 KiB
constexpr int kTnRawB = 32 * TN_N * 4;         // 8 KiB
constexpr int kTnRaw = kTnRawA + kTnRawB;      // 24 KiB
constexpr int kTnRawStages = 3;
constexpr int kTnOpB = TN_NB * 128;            // 10 KiB
constexpr int kTnOp = 2 * kBlkA + 2 * kTnOpB + 3072;   // hi/lo of A and B, padded to a multiple of 1 KiB (55 KiB... 56 KiB)
constexpr int kTnOpStages = 2;
constexpr int kTnBlocks = 64;                  // K blocks (of 32 rows) per CTA

struct TnParams {
  float* C;
  float* colsum;
  int64_t ldc;
  int M, N, K;
  int* status;
};

__global__ void __launch_bounds__(kThreadsRes, 1) gemm_f32x3_tn_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                     const __grid_constant__ CUtensorMap map_b,
                                                                     const TnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ops = smem;                                   // kTnOpStages x [A_hi | A_lo | B_hi | B_lo]
  unsigned char* raws = ops + kTnOpStages * kTnOp;             // kTnRawStages x [raw A | raw B]
  unsigned long long* fullraw = reinterpret_cast<unsigned long long*>(raws + kTnRawStages * kTnRaw);
  unsigned long long* rawempty = fullraw + kTnRawStages;
  unsigned long long* opready = rawempty + kTnRawStages;
  unsigned long long* opempty = opready + kTnOpStages;
  unsigned long long* acc_ready = opempty + kTnOpStages;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_ready + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * XM, n0 = blockIdx.y * TN_N;
  const int total_kb = (p.K + XKB - 1) / XKB;
  const int kb0 = blockIdx.z * kTnBlocks;
  const int nkb = min(kTnBlocks, total_kb - kb0);
  const bool with_sum = p.colsum != nullptr && blockIdx.y == 0;
  constexpr int kAcc = 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTnRawStages; ++s) { bar_init(fullraw + s, 1); bar_init(rawempty + s, 8); }
    for (int s = 0; s < kTnOpStages; ++s) { bar_init(opready + s, 8); bar_init(opempty + s, 1); }
    bar_init(acc_ready, 2);
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
      for (int kb = 0; kb < nkb; ++kb) {
        const int r = kb % kTnRawStages;
        if (!bar_wait(rawempty + r, ((kb / kTnRawStages) & 1) ^ 1, p.status)) break;
        unsigned char* raw = raws + r * kTnRaw;
        bar_expect_tx(fullraw + r, kTnRaw);
        tma_load_2d(raw, &map_a, m0, (kb0 + kb) * XKB, fullraw + r);
        tma_load_2d(raw + kTnRawA, &map_b, n0, (kb0 + kb) * XKB, fullraw + r);
      }
    }
  } else if (warp == 1 || warp == 10) {
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1;
      const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(TN_NB >> 3) << 17) | ((unsigned)(XM >> 4) << 24);
      for (int kb = me; kb < nkb; kb += 2) {
        const int o = kb % kTnOpStages;
        if (!bar_wait(opready + o, (kb / kTnOpStages) & 1, p.status)) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned char* st = ops + o * kTnOp;
        const unsigned long long dah = smem_desc(st), dal = smem_desc(st + kBlkA);
        const unsigned long long dbh = smem_desc(st + 2 * kBlkA), dbl = smem_desc(st + 2 * kBlkA + kTnOpB);
        const unsigned tacc = tmem_base + (kb % kAcc) * 128;
        unsigned acc = kb >= kAcc ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < XKB / 8; ++kk) {
          umma_tf32(tacc, dal + 2ull * kk, dbh + 2ull * kk, idesc, acc);
          acc = 1;
          umma_tf32(tacc, dah + 2ull * kk, dbl + 2ull * kk, idesc, 1u);
          umma_tf32(tacc, dah + 2ull * kk, dbh + 2ull * kk, idesc, 1u);
        }
        umma_commit(opempty + o);
      }
      umma_commit(acc_ready);
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    const bool ok = bar_wait(acc_ready, 0, p.status);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const int m = m0 + q * 32 + lane;
#pragma unroll
    for (int part = 0; part < 3; ++part) {     // columns 0-31, 32-63, 64-95 (only column 64 of the last part is used)
      if (part == 2 && !with_sum) break;
      unsigned v[32];
      tmem_ld32x(tmem_base + ((unsigned)(q * 32) << 16) + part * 32, v);
      for (int a = 1; a < kAcc && a < nkb; ++a) {
        unsigned v2[32];
        tmem_ld32x(tmem_base + ((unsigned)(q * 32) << 16) + a * 128 + part * 32, v2);
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) + __uint_as_float(v2[c]));
      }
      if (ok && status_clean(p.status) && nkb > 0 && m < p.M) {
        if (part < 2) {
          float* dst = p.C + (int64_t)m * p.ldc + n0 + part * 32;
#pragma unroll
          for (int c = 0; c < 32; c += 4)
            if (n0 + part * 32 + c < p.N)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(dst + c), "f"(__uint_as_float(v[c])),
                           "f"(__uint_as_float(v[c + 1])), "f"(__uint_as_float(v[c + 2])), "f"(__uint_as_float(v[c + 3])) : "memory");
        } else {
          atomicAdd(p.colsum + m, __uint_as_float(v[0]));
        }
      }
    }
  } else {
    // eight split warps: 6-9 and 11-14
    const int tid = warp < 10 ? threadIdx.x - 6 * 32 : threadIdx.x - 11 * 32 + 128;
    // constant rows of the B operand tiles: row 64 = ones (hi) / zeros (lo), rows 65..79 zeros
    for (int o = 0; o < kTnOpStages; ++o) {
      float* bh = reinterpret_cast<float*>(ops + o * kTnOp + 2 * kBlkA);
      float* bl = reinterpret_cast<float*>(ops + o * kTnOp + 2 * kBlkA + kTnOpB);
      for (int idx = tid; idx < (TN_NB - TN_N) * 32; idx += 256) {
        bh[TN_N * 32 + idx] = idx < 32 ? 1.0f : 0.f;    // a row of identical values is unchanged by the swizzle
        bl[TN_N * 32 + idx] = 0.f;
      }
    }
    bool dead = false;
    for (int kb = 0; kb < nkb; ++kb) {
      const int r = kb % kTnRawStages, o = kb % kTnOpStages;
      if (!dead) dead = !bar_wait(fullraw + r, (kb / kTnRawStages) & 1, p.status);
      if (!dead) dead = !bar_wait(opempty + o, ((kb / kTnOpStages) & 1) ^ 1, p.status);
      if (!dead) {
        const float* rawA = reinterpret_cast<const float*>(raws + r * kTnRaw);
        const float* rawB = reinterpret_cast<const float*>(raws + r * kTnRaw + kTnRawA);
        unsigned char* st = ops + o * kTnOp;
        {  // A: thread = (column m of the raw block = row m of the operand tile, half of the k range)
          const int m = tid & 127, ga = (tid >> 7) * 4;
#pragma unroll
          for (int gg = 0; gg < 4; ++gg) {
            const int g = ga + gg;
            uint4 h, l;
            unsigned x[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = __float_as_uint(rawA[(4 * g + j) * XM + m]);
            h.x = rna_tf32(x[0]); h.y = rna_tf32(x[1]); h.z = rna_tf32(x[2]); h.w = rna_tf32(x[3]);
            l.x = rna_tf32(__float_as_uint(__uint_as_float(x[0]) - __uint_as_float(h.x)));
            l.y = rna_tf32(__float_as_uint(__uint_as_float(x[1]) - __uint_as_float(h.y)));
            l.z = rna_tf32(__float_as_uint(__uint_as_float(x[2]) - __uint_as_float(h.z)));
            l.w = rna_tf32(__float_as_uint(__uint_as_float(x[3]) - __uint_as_float(h.w)));
            const int off = m * 128 + ((g ^ (m & 7)) << 4);
            *reinterpret_cast<uint4*>(st + off) = h;
            *reinterpret_cast<uint4*>(st + kBlkA + off) = l;
          }
        }
        {  // B: 64 columns, four quarters of the k range
          const int n = tid & 63, g0 = (tid >> 6) * 2;
#pragma unroll
          for (int gg = 0; gg < 2; ++gg) {
            const int g = g0 + gg;
            uint4 h, l;
            unsigned x[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = __float_as_uint(rawB[(4 * g + j) * TN_N + n]);
            h.x = rna_tf32(x[0]); h.y = rna_tf32(x[1]); h.z = rna_tf32(x[2]); h.w = rna_tf32(x[3]);
            l.x = rna_tf32(__float_as_uint(__uint_as_float(x[0]) - __uint_as_float(h.x)));
            l.y = rna_tf32(__float_as_uint(__uint_as_float(x[1]) - __uint_as_float(h.y)));
            l.z = rna_tf32(__float_as_uint(__uint_as_float(x[2]) - __uint_as_float(h.z)));
            l.w = rna_tf32(__float_as_uint(__uint_as_float(x[3]) - __uint_as_float(h.w)));
            const int off = n * 128 + ((g ^ (n & 7)) << 4);
            *reinterpret_cast<uint4*>(st + 2 * kBlkA + off) = h;
            *reinterpret_cast<uint4*>(st + 2 * kBlkA + kTnOpB + off) = l;
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) { bar_arrive1(opready + o); bar_arrive1(rawempty + r); }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// float32 [rows][cols], no swizzle; box = box_cols x 32 rows
int make_map_f32_plain(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return cueq::fail("gemm f32x3: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, 32u};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cueq::fail("gemm f32x3: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

// float32 [rows][cols] with `ld` elements between rows; box = 32 columns (128 bytes) x box_rows
int make_map_f32(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return cueq::fail("gemm f32x3: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {(cuuint32_t)XKB, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cueq::fail("gemm f32x3: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

}  // namespace

extern "C" int cueq_b200_gemm_f32x3(const cueq_gemm_f32x3_args* g, void* stream) {
  if (!g || !g->A || !g->B_hi || !g->B_lo || !g->C) return cueq::fail("gemm f32x3: null operand");
  if (g->M <= 0 || g->N <= 0) return 0;
  if (g->K <= 0 || (g->K % 32)) return cueq::fail("gemm f32x3: K must be a positive multiple of 32 (got %lld)", (long long)g->K);
  if (g->N % 4) return cueq::fail("gemm f32x3: N must be a multiple of 4");
  if ((g->lda % 4) || (g->ldb % 4) || (g->ldc % 4)) return cueq::fail("gemm f32x3: leading dimensions must keep rows 16-byte aligned");
  if (((uintptr_t)g->A | (uintptr_t)g->B_hi | (uintptr_t)g->B_lo | (uintptr_t)g->C | (uintptr_t)g->bias) & 15)
    return cueq::fail("gemm f32x3: operands must be 16-byte aligned");
  if (g->M > 2147483647LL - XM || g->N > 2147483647LL - XN || g->K > 2147483647LL) return cueq::fail("gemm f32x3: dimension too large");
  const bool resident = g->K <= kMaxKB * XKB;          // A tile split once, reused for every column tile
  const int nt = resident ? XN : (g->N <= 64 ? 64 : 128);
  CUtensorMap ma, mh, ml, mc;
  if (int rc = make_map_f32(&ma, g->A, g->M, g->K, g->lda, XM)) return rc;
  if (int rc = make_map_f32(&mh, g->B_hi, g->N, g->K, g->ldb, nt)) return rc;
  if (int rc = make_map_f32(&ml, g->B_lo, g->N, g->K, g->ldb, nt)) return rc;
  if (int rc = make_map_f32(&mc, g->C, g->M, g->N, g->ldc, 32)) return rc;
  XParams p;
  std::memset(&p, 0, sizeof(p));
  p.C = reinterpret_cast<float*>(g->C);
  p.bias = reinterpret_cast<const float*>(g->bias);
  p.ldc = g->ldc; p.M = (int)g->M; p.N = (int)g->N; p.nkb = (int)(g->K / XKB);
  p.status = reinterpret_cast<int*>(g->status);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned mtiles = (unsigned)((g->M + XM - 1) / XM);
  if (resident) {
    const size_t smem = 2 * kMaxKB * kBlkA + 4 * 2 * kBlkB + 8 * 4096 + 256 + 1024;
    static cueq::PerDeviceFlag configured;
    if (!configured.get()) {
      CUEQ_CUDA_OK(cudaFuncSetAttribute(gemm_f32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured.set();
    }
    gemm_f32x3_kernel<<<dim3(mtiles), kThreadsRes, smem, st>>>(ma, mh, ml, mc, p);
  } else if (nt == 64) {
    using Cfg = StreamCfg<64>;
    const size_t smem = Cfg::kStages * Cfg::kStage + 4 * 2 * 4096 + 256 + 1024;
    static cueq::PerDeviceFlag configured;
    if (!configured.get()) {
      CUEQ_CUDA_OK(cudaFuncSetAttribute(gemm_f32x3_stream_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured.set();
    }
    gemm_f32x3_stream_kernel<64><<<dim3(mtiles, (unsigned)((g->N + 63) / 64)), kThreadsX, smem, st>>>(ma, mh, ml, mc, p);
  } else {
    using Cfg = StreamCfg<128>;
    const size_t smem = Cfg::kStages * Cfg::kStage + 4 * 2 * 4096 + 256 + 1024;
    static cueq::PerDeviceFlag configured;
    if (!configured.get()) {
      CUEQ_CUDA_OK(cudaFuncSetAttribute(gemm_f32x3_stream_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured.set();
    }
    gemm_f32x3_stream_kernel<128><<<dim3(mtiles, (unsigned)((g->N + 127) / 128)), kThreadsX, smem, st>>>(ma, mh, ml, mc, p);
  }
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int cueq_b200_gemm_f32x3_tn(const cueq_gemm_f32x3_tn_args* g, void* stream) {
  if (!g || !g->A || !g->B || !g->C) return cueq::fail("gemm f32x3 tn: null operand");
  if (g->M <= 0 || g->N <= 0 || g->K <= 0) return 0;
  if ((g->M % 4) || (g->N % 4)) return cueq::fail("gemm f32x3 tn: M and N must be multiples of 4");
  if ((g->lda % 4) || (g->ldb % 4) || (g->ldc % 4)) return cueq::fail("gemm f32x3 tn: leading dimensions must keep rows 16-byte aligned");
  if (((uintptr_t)g->A | (uintptr_t)g->B | (uintptr_t)g->C) & 15) return cueq::fail("gemm f32x3 tn: operands must be 16-byte aligned");
  if (g->M > 2147483647LL - XM || g->N > 2147483647LL - TN_N || g->K > 2147483647LL - XKB) return cueq::fail("gemm f32x3 tn: dimension too large");
  CUtensorMap ma, mb;
  if (int rc = make_map_f32_plain(&ma, g->A, g->K, g->M, g->lda, XM)) return rc;
  if (int rc = make_map_f32_plain(&mb, g->B, g->K, g->N, g->ldb, TN_N)) return rc;
  TnParams p;
  std::memset(&p, 0, sizeof(p));
  p.C = reinterpret_cast<float*>(g->C);
  p.colsum = reinterpret_cast<float*>(g->colsum);
  p.ldc = g->ldc; p.M = (int)g->M; p.N = (int)g->N; p.K = (int)g->K;
  p.status = reinterpret_cast<int*>(g->status);
  const size_t smem = kTnOpStages * kTnOp + kTnRawStages * kTnRaw + 256 + 1024;
  static cueq::PerDeviceFlag configured;
  if (!configured.get()) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(gemm_f32x3_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set();
  }
  const int64_t total_kb = (g->K + XKB - 1) / XKB;
  dim3 grid((unsigned)((g->M + XM - 1) / XM), (unsigned)((g->N + TN_N - 1) / TN_N), (unsigned)((total_kb + kTnBlocks - 1) / kTnBlocks));
  if (grid.z > 65535) return cueq::fail("gemm f32x3 tn: K too large for one launch");
  gemm_f32x3_tn_kernel<<<grid, kThreadsRes, smem, reinterpret_cast<cudaStream_t>(stream)>>>(ma, mb, p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

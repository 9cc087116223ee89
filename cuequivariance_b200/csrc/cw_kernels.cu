// Channelwise ("uvu") tensor product: fused gather * Clebsch-Gordan multiply-add * receiver
// reduction, forward and backward, one launch per group of paths that read the same irrep of
// the first operand.
//
// These kernels replace the reference's closed uniform-1d kernel on the hot polynomial
// ``uv,iu,jv,kuv+ijk`` (descriptor: cuequivariance/group_theory/descriptors/irreps_tp.py:232-321;
// module: cuequivariance_torch/operations/tp_channel_wise.py:186-258), including the layout
// transpositions the reference performs as separate passes (tp_channel_wise.py:221-222,258).
//
// Work decomposition
//   * edges are addressed through a CSR over receivers (rowptr, optional edge order), so the
//     reduction over the edges of a receiver happens in registers: every output row is
//     written exactly once, without atomics and without a prior memset;
//   * one warp owns one receiver at a time; a lane owns two (or four) consecutive channels (one
//     128-bit access per segment), so a warp covers 128 channels; wider operands use
//     blockIdx.y;
//   * per edge, the channel-independent matrices M[i,k] = sum_j C[i,j,k] x2[j] of all paths of
//     the group are computed once per warp into shared memory (a table-driven loop spread
//     over the lanes) and then read back as broadcasts by the straight-line generated code;
//   * the rows of the next edge (the gathered x1 block and one weight segment per path) are
//     prefetched with cp.async into a per-warp, lane-private double buffer, so HBM latency
//     overlaps the arithmetic of the current edge;
//   * backward: the cotangent row of the receiver is staged once per receiver; the gradient
//     of the gathered operand goes out as vectorised reductions (red.global.add.v4.f32) keyed
//     by sender, the weight gradient is streamed out, the gradient of x2 is reduced over the
//     channels with warp shuffles.
#include <cstdint>
#include <cstring>

#include "common.cuh"
#include "generated/cw_groups.cuh"

namespace {

constexpr int kMaxPaths = 8;
constexpr int kMaxTerms = 160;
#ifndef CW_WARPS
#define CW_WARPS 4
#endif
constexpr int kWarps = CW_WARPS;  // warps per CTA
#ifndef CW_MINBLOCKS
#define CW_MINBLOCKS 4
#endif

struct CwCoef {
  float c[kMaxTerms];
};

struct CwParams {
  const float* w;
  const float* x1;
  const float* x2;
  float* out;          // forward output / unused in backward
  const float* gout;   // backward: cotangent of out
  float* gw;
  float* gx1;
  float* gx2;
  const int* senders;  // [E] row of x1 for each edge (edge ids, not CSR positions); null: edge id
  const int* order;    // [E] CSR position -> edge id; null: identity
  const int* rowptr;   // [num_receivers + 1]
  const int* tab_start;  // [NPAIR + 1] term range of every (i,k) pair
  const int* tab_j;      // [NTERM] x2 element of the term
  const float* tab_c;    // [NTERM] coefficient of the term
  int64_t w_stride, x1_stride, x2_stride, out_stride;
  int num_receivers;
  int extent;
  int x1_off;               // element offset of the group's irrep block inside an x1 row
  int w_off[kMaxPaths];     // element offset of each path's weight segment inside a w row
  int out_off[kMaxPaths];   // element offset of each path's output block inside an out row
  int need_gw, need_gx1, need_gx2;
  int* status;              // nullable: set to 1 if a bounded wait on a bulk copy ran out
  int recv_mod;             // backward: CSR rows are (pass, receiver) pairs; the cotangent row is row % recv_mod (0: off)
};

template <int C> struct VecT;
template <> struct VecT<4> { using type = float4; };
template <> struct VecT<2> { using type = float2; };
template <int C> using Vec = typename VecT<C>::type;

__device__ __forceinline__ void to_array(const float4& v, float (&a)[4]) { a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w; }
__device__ __forceinline__ void to_array(const float2& v, float (&a)[2]) { a[0] = v.x; a[1] = v.y; }

template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem_dst, const void* gmem_src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  if constexpr (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
// L2 cache policies: per-edge operands are read once (evict first), the gathered node rows
// and the scattered node gradients are revisited by other edges (evict last)
__device__ __forceinline__ unsigned long long policy_evict_first() {
  unsigned long long p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(p));
  return p;
}
__device__ __forceinline__ unsigned long long policy_evict_last() {
  unsigned long long p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(p));
  return p;
}
template <int BYTES>
__device__ __forceinline__ void cp_async_hint(void* smem_dst, const void* gmem_src, unsigned long long policy) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  if constexpr (BYTES == 16)
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gmem_src), "l"(policy) : "memory");
  else
    asm volatile("cp.async.ca.shared.global.L2::cache_hint [%0], [%1], 8, %2;\n" ::"r"(d), "l"(gmem_src), "l"(policy) : "memory");
}
__device__ __forceinline__ void red_add_hint(float* addr, const float (&v)[4], unsigned long long policy) {
  asm volatile("red.global.add.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;\n" ::"l"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "l"(policy) : "memory");
}
__device__ __forceinline__ void red_add_hint(float* addr, const float (&v)[2], unsigned long long policy) {
  asm volatile("red.global.add.L2::cache_hint.v2.f32 [%0], {%1, %2}, %3;\n" ::"l"(addr), "f"(v[0]), "f"(v[1]), "l"(policy) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// ---- bulk-copy (TMA) staging ----------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~2^20 polls (each poll itself blocks for a hardware time slice),
// records the failure and lets the kernel run to its end instead of hanging the GPU.
__device__ __forceinline__ void mbar_wait(unsigned long long* bar, unsigned parity, int* status) {
  for (int spin = 0; spin < (1 << 20); ++spin)
    if (mbar_try_wait(bar, parity)) return;
  if (status) atomicExch(status, 1);
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
// One bulk reduction (float32 add) of `bytes` contiguous bytes from shared to global memory, issued by one thread
// and tracked by that thread's bulk async-group; both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_reduce_add(float* gmem_dst, const void* smem_src, unsigned bytes, unsigned long long pol) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.L2::cache_hint.add.f32 [%0], [%1], %2, %3;\n"
               ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes), "l"(pol) : "memory");
  asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
}
// the issuing thread waits until its bulk reductions have read their shared-memory source / have completed
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

__device__ __forceinline__ void red_add(float* addr, const float (&v)[4]) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
}
__device__ __forceinline__ void red_add(float* addr, const float (&v)[2]) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};\n" ::"l"(addr), "f"(v[0]), "f"(v[1]) : "memory");
}
__device__ __forceinline__ void st_stream(float* addr, const float (&v)[4]) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
}
__device__ __forceinline__ void st_stream(float* addr, const float (&v)[2]) {
  asm volatile("st.global.cs.v2.f32 [%0], {%1, %2};\n" ::"l"(addr), "f"(v[0]), "f"(v[1]) : "memory");
}

// shared memory carve-up, in floats.  C = channels per lane.  Everything is per warp.
template <class G, int C>
struct Smem {
  static constexpr int kM = G::NPAIR_PAD;                                   // per stage
  static constexpr int kX2 = 16;                                            // per stage: x2 row (<= 16 floats)
  static constexpr int kStage = (G::D1 + G::NPATH) * 32 * C;                // per stage: x1 block + weights
  static constexpr int kPerStage = kX2 + kStage;
  static constexpr int kPerWarpFwd = kM + 2 * kPerStage;
  static constexpr int kGrow = G::SUMD3 * 32 * C;                           // cotangent row of the receiver
  static constexpr int kPerWarpBwd = kPerWarpFwd + kGrow;
  static constexpr size_t bytes_fwd() { return sizeof(float) * (kWarps * kPerWarpFwd); }
  static constexpr size_t bytes_bwd() { return sizeof(float) * (kWarps * kPerWarpBwd); }
};

// Block of D contiguous-per-component values of the C channels of this lane, between global
// memory and lane-private staging.  ir_mul: component t of the lane's channels sits at
// base + t*extent + ch;  mul_ir: the lane's C*D values are contiguous at base + ch*D.
template <int D, int C, bool MUL_IR>
__device__ __forceinline__ void stage_block(Vec<C>* dst, const float* base, int extent, int ch, int lane) {
#pragma unroll
  for (int t = 0; t < D; ++t) {
    const float* src = MUL_IR ? base + (int64_t)ch * D + C * t : base + (int64_t)t * extent + ch;
    cp_async<4 * C>(dst + t * 32 + lane, src);
  }
}
template <int D, int C, bool MUL_IR>
__device__ __forceinline__ void stage_block_hint(Vec<C>* dst, const float* base, int extent, int ch, int lane, unsigned long long pol) {
#pragma unroll
  for (int t = 0; t < D; ++t) {
    const float* src = MUL_IR ? base + (int64_t)ch * D + C * t : base + (int64_t)t * extent + ch;
    cp_async_hint<4 * C>(dst + t * 32 + lane, src, pol);
  }
}

template <int D, int C, bool MUL_IR, int ROWS>
__device__ __forceinline__ void unstage_block(const Vec<C>* src, int lane, float (&X)[ROWS][C]) {
  float f[D * C];
#pragma unroll
  for (int t = 0; t < D; ++t) {
    float a[C];
    to_array(src[t * 32 + lane], a);
#pragma unroll
    for (int c = 0; c < C; ++c) f[C * t + c] = a[c];
  }
#pragma unroll
  for (int i = 0; i < D; ++i)
#pragma unroll
    for (int c = 0; c < C; ++c) X[i][c] = MUL_IR ? f[c * D + i] : f[C * i + c];
}

// registers -> global, same two layouts; RED: vector reduction, else streaming store
template <int D, int C, bool MUL_IR, bool RED, int ROWS>
__device__ __forceinline__ void emit_block(float* base, int extent, int ch, const float (&V)[ROWS][C], int row0, unsigned long long pol = 0) {
  if (MUL_IR) {
    float f[D * C];
#pragma unroll
    for (int i = 0; i < D; ++i)
#pragma unroll
      for (int c = 0; c < C; ++c) f[c * D + i] = V[row0 + i][c];
#pragma unroll
    for (int t = 0; t < D; ++t) {
      float v[C];
#pragma unroll
      for (int c = 0; c < C; ++c) v[c] = f[C * t + c];
      if (RED) red_add_hint(base + (int64_t)ch * D + C * t, v, pol); else st_stream(base + (int64_t)ch * D + C * t, v);
    }
  } else {
#pragma unroll
    for (int i = 0; i < D; ++i) {
      if (RED) red_add_hint(base + (int64_t)i * extent + ch, V[row0 + i], pol); else st_stream(base + (int64_t)i * extent + ch, V[row0 + i]);
    }
  }
}

// The channel-independent matrices M of one edge: M[q] = sum_t c[t] * x2[j[t]] for every table
// entry q of the group - one per non-zero (i,k) pair in the backward kernels (N = NPAIR), one per
// distinct value among them in the forward kernels (N = NVAL: many pairs carry the same combination
// of x2 up to sign, and every entry costs a broadcast read per warp and edge).  Lane L owns the
// entries L, L+32, ...; an entry has at most two terms (true for every coupling with l <= 3), whose
// coefficients and x2 positions the lane keeps in registers for the whole kernel, so the per-edge
// work is a handful of shared-memory reads and FMAs without any loop or branch.
template <int N>
struct MTerms {
  static constexpr int R = (N + 31) / 32;
  static constexpr int NPAD = (N + 3) / 4 * 4;
  float c[R][2];
  unsigned j[R];  // two 16-bit x2 positions per pair

  __device__ __forceinline__ void load(const CwParams& p, int lane) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int q = lane + 32 * r;
      c[r][0] = c[r][1] = 0.f;
      j[r] = 0;
      if (q < N) {
        const int t0 = __ldg(p.tab_start + q), t1 = __ldg(p.tab_start + q + 1);
        if (t1 > t0) { c[r][0] = __ldg(p.tab_c + t0); j[r] = (unsigned)__ldg(p.tab_j + t0); }
        if (t1 > t0 + 1) { c[r][1] = __ldg(p.tab_c + t0 + 1); j[r] |= (unsigned)__ldg(p.tab_j + t0 + 1) << 16; }
      }
    }
  }
  __device__ __forceinline__ void compute(float* M, const float* x2row, int lane) const {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float m = fmaf(c[r][1], x2row[j[r] >> 16], c[r][0] * x2row[j[r] & 0xffffu]);
      if (N % 32 == 0 || r + 1 < R || lane + 32 * r < NPAD) M[lane + 32 * r] = m;
    }
  }
};

// asynchronous loads of everything edge `pos` needs into the stage at `st`; returns the edge id
// The edge id (through the optional permutation) and the sender of the edge at position `pos`: two dependent
// index loads.  The kernels request them one edge earlier than they issue that edge's copies, so that their
// latency is hidden behind the arithmetic of an edge instead of being waited for in front of the copies.
struct EdgeIds { int eid, snd; };
__device__ __forceinline__ EdgeIds load_ids(const CwParams& p, int pos) {
  EdgeIds e;
  e.eid = p.order ? __ldg(p.order + pos) : pos;
  e.snd = p.senders ? __ldg(p.senders + e.eid) : e.eid;
  return e;
}

template <class G, int C, bool X1_MUL_IR>
__device__ __forceinline__ void issue_edge_ids(const CwParams& p, float* st, const EdgeIds ids, int ch, int lane, bool active,
                                               unsigned long long pol_stream, unsigned long long pol_keep) {
  float* x2s = st;
  Vec<C>* stage = reinterpret_cast<Vec<C>*>(x2s + Smem<G, C>::kX2);
  if (lane < (G::NX2 + 3) / 4) cp_async_hint<16>(x2s + 4 * lane, p.x2 + (int64_t)ids.eid * p.x2_stride + 4 * lane, pol_stream);
  if (active) {
    stage_block_hint<G::D1, C, X1_MUL_IR>(stage, p.x1 + (int64_t)ids.snd * p.x1_stride + p.x1_off, p.extent, ch, lane, pol_keep);
    const float* wrow = p.w + (int64_t)ids.eid * p.w_stride + ch;
    Vec<C>* wst = stage + G::D1 * 32;
#pragma unroll
    for (int q = 0; q < G::NPATH; ++q) cp_async_hint<4 * C>(wst + q * 32 + lane, wrow + p.w_off[q], pol_stream);
  }
  cp_async_commit();
}

template <class G, int C, int P>
struct FwdPaths {
  __device__ __forceinline__ static void run(const float (&X)[G::D1][C], const Vec<C>* wst, int lane, const float* M,
                                             float (&acc)[G::SUMD3][C]) {
    float W[C];
    to_array(wst[P * 32 + lane], W);
    G::template fwd_path<P, C>(X, W, M, acc);
    if constexpr (P + 1 < G::NPATH) FwdPaths<G, C, P + 1>::run(X, wst, lane, M, acc);
  }
};

template <class G, int C, int P, bool OUT_MUL_IR>
struct StoreOut {
  __device__ __forceinline__ static void run(float* orow, const CwParams& p, int ch, const float (&acc)[G::SUMD3][C]) {
    emit_block<G::d3(P), C, OUT_MUL_IR, false>(orow + p.out_off[P], p.extent, ch, acc, G::out_offset(P));
    if constexpr (P + 1 < G::NPATH) StoreOut<G, C, P + 1, OUT_MUL_IR>::run(orow, p, ch, acc);
  }
};

template <class G, int C, bool MUL_IR>
__global__ void __launch_bounds__(kWarps * 32, CW_MINBLOCKS) cw_fwd_kernel(const __grid_constant__ CwParams p) {
  extern __shared__ __align__(16) float smem[];
  using S = Smem<G, C>;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* mine = smem + warp * S::kPerWarpFwd;
  const int ch = blockIdx.y * (32 * C) + C * lane;   // first channel of this lane
  const bool active = ch < p.extent;
  MTerms<G::NVAL> mt;
  mt.load(p, lane);
  const unsigned long long pol_stream = policy_evict_first(), pol_keep = policy_evict_last();

  const int total_warps = gridDim.x * kWarps;
  for (int n = blockIdx.x * kWarps + warp; n < p.num_receivers; n += total_warps) {
    const int beg = __ldg(p.rowptr + n), end = __ldg(p.rowptr + n + 1);
    float acc[G::SUMD3][C];
#pragma unroll
    for (int a = 0; a < G::SUMD3; ++a)
#pragma unroll
      for (int c = 0; c < C; ++c) acc[a][c] = 0.f;
    float* Msm = mine;
    float* stages = mine + S::kM;
    EdgeIds ahead = {0, 0};                                        // ids of the edge whose copies are issued next
    if (beg < end) issue_edge_ids<G, C, MUL_IR>(p, stages, load_ids(p, beg), ch, lane, active, pol_stream, pol_keep);
    if (beg + 1 < end) ahead = load_ids(p, beg + 1);
    for (int pos = beg; pos < end; ++pos) {
      float* st = stages + ((pos - beg) & 1) * S::kPerStage;
      if (pos + 1 < end) {
        issue_edge_ids<G, C, MUL_IR>(p, stages + ((pos + 1 - beg) & 1) * S::kPerStage, ahead, ch, lane, active, pol_stream, pol_keep);
        if (pos + 2 < end) ahead = load_ids(p, pos + 2);           // used in the next trip
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncwarp();
      mt.compute(Msm, st, lane);
      __syncwarp();
      if (active) {
        const Vec<C>* stage = reinterpret_cast<const Vec<C>*>(st + S::kX2);
        float X[G::D1][C];
        unstage_block<G::D1, C, MUL_IR>(stage, lane, X);
        FwdPaths<G, C, 0>::run(X, stage + G::D1 * 32, lane, Msm, acc);
      }
      __syncwarp();
    }
    if (active) StoreOut<G, C, 0, MUL_IR>::run(p.out + (int64_t)n * p.out_stride, p, ch, acc);
  }
}

// ---- forward, staging by bulk copies ----------------------------------------------------------
//
// Same arithmetic as cw_fwd_kernel; the rows of the next edge are fetched by the copy engine
// (cp.async.bulk, one instruction per contiguous piece, issued by one lane) and their arrival
// is signalled on an mbarrier, instead of one cp.async per lane and piece.  The staged data
// keep their global layout: for mul_ir the whole [channel][component] block of the gathered
// row is one contiguous copy.
template <class G, int C>
struct SmemBulk {
  static constexpr int NCH = 32 * C;                                        // channels per warp
  static constexpr int kBar = 4;                                            // two 64-bit barriers
  static constexpr int kM = G::NPAIR_PAD;
  static constexpr int kX2 = 16;
  static constexpr int kPerStage = kX2 + (G::D1 + G::NPATH) * NCH;
  static constexpr int kPerWarp = kBar + kM + 2 * kPerStage;
  static constexpr size_t bytes() { return sizeof(float) * (kWarps * kPerWarp); }
};

template <class G, int C, bool MUL_IR>
__device__ __forceinline__ void bulk_issue_edge(const CwParams& p, float* st, unsigned long long* bar, int pos, int c0, int nch) {
  using S = SmemBulk<G, C>;
  const int eid = p.order ? __ldg(p.order + pos) : pos;
  const int snd = p.senders ? __ldg(p.senders + eid) : eid;
  constexpr unsigned x2_bytes = ((G::NX2 + 3) / 4) * 16;
  const unsigned row_bytes = (unsigned)nch * 4u;
  fence_proxy_async();
  mbar_expect_tx(bar, x2_bytes + row_bytes * (G::D1 + G::NPATH));
  bulk_g2s(st, p.x2 + (int64_t)eid * p.x2_stride, x2_bytes, bar);
  float* xs = st + S::kX2;
  const float* xrow = p.x1 + (int64_t)snd * p.x1_stride + p.x1_off;
  if (MUL_IR) {
    bulk_g2s(xs, xrow + (int64_t)c0 * G::D1, row_bytes * G::D1, bar);
  } else {
#pragma unroll
    for (int i = 0; i < G::D1; ++i) bulk_g2s(xs + i * S::NCH, xrow + (int64_t)i * p.extent + c0, row_bytes, bar);
  }
  float* ws = xs + G::D1 * S::NCH;
  const float* wrow = p.w + (int64_t)eid * p.w_stride + c0;
#pragma unroll
  for (int q = 0; q < G::NPATH; ++q) bulk_g2s(ws + q * S::NCH, wrow + p.w_off[q], row_bytes, bar);
}

template <class G, int C, int P>
struct FwdPathsBulk {
  __device__ __forceinline__ static void run(const float (&X)[G::D1][C], const float* ws, int lane, const float* M,
                                             float (&acc)[G::SUMD3][C]) {
    float W[C];
    to_array(*reinterpret_cast<const Vec<C>*>(ws + P * (32 * C) + C * lane), W);
    G::template fwd_path<P, C>(X, W, M, acc);
    if constexpr (P + 1 < G::NPATH) FwdPathsBulk<G, C, P + 1>::run(X, ws, lane, M, acc);
  }
};

template <class G, int C, bool MUL_IR>
__global__ void __launch_bounds__(kWarps * 32, C == 2 ? CW_MINBLOCKS : 2) cw_fwd_bulk_kernel(const __grid_constant__ CwParams p) {
  extern __shared__ __align__(16) float smem[];
  using S = SmemBulk<G, C>;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* mine = smem + warp * S::kPerWarp;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(mine);
  float* Msm = mine + S::kBar;
  float* stages = Msm + S::kM;
  const int c0 = blockIdx.y * S::NCH;
  const int ch = c0 + C * lane;
  const bool active = ch < p.extent;
  const int nch = min(S::NCH, p.extent - c0);
  MTerms<G::NVAL> mt;
  mt.load(p, lane);
  if (lane == 0) {
    mbar_init(bars + 0, 1);
    mbar_init(bars + 1, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  unsigned it = 0;  // edges consumed by this warp so far: stage = it & 1, parity = (it >> 1) & 1

  const int total_warps = gridDim.x * kWarps;
  for (int n = blockIdx.x * kWarps + warp; n < p.num_receivers; n += total_warps) {
    const int beg = __ldg(p.rowptr + n), end = __ldg(p.rowptr + n + 1);
    float acc[G::SUMD3][C];
#pragma unroll
    for (int a = 0; a < G::SUMD3; ++a)
#pragma unroll
      for (int c = 0; c < C; ++c) acc[a][c] = 0.f;
    if (beg < end && lane == 0) bulk_issue_edge<G, C, MUL_IR>(p, stages + (it & 1) * S::kPerStage, bars + (it & 1), beg, c0, nch);
    for (int pos = beg; pos < end; ++pos, ++it) {
      const unsigned s = it & 1;
      float* st = stages + s * S::kPerStage;
      if (pos + 1 < end && lane == 0)
        bulk_issue_edge<G, C, MUL_IR>(p, stages + (s ^ 1) * S::kPerStage, bars + (s ^ 1), pos + 1, c0, nch);
      mbar_wait(bars + s, (it >> 1) & 1, p.status);
      mt.compute(Msm, st, lane);
      __syncwarp();
      if (active) {
        const float* xs = st + S::kX2;
        float X[G::D1][C];
        if (MUL_IR) {
          float f[G::D1 * C];
          const Vec<C>* src = reinterpret_cast<const Vec<C>*>(xs + (int64_t)C * lane * G::D1);
#pragma unroll
          for (int t = 0; t < G::D1; ++t) {
            float a[C];
            to_array(src[t], a);
#pragma unroll
            for (int c = 0; c < C; ++c) f[C * t + c] = a[c];
          }
#pragma unroll
          for (int i = 0; i < G::D1; ++i)
#pragma unroll
            for (int c = 0; c < C; ++c) X[i][c] = f[c * G::D1 + i];
        } else {
#pragma unroll
          for (int i = 0; i < G::D1; ++i) to_array(*reinterpret_cast<const Vec<C>*>(xs + i * S::NCH + C * lane), X[i]);
        }
        FwdPathsBulk<G, C, 0>::run(X, xs + G::D1 * S::NCH, lane, Msm, acc);
      }
      __syncwarp();
    }
    if (active) StoreOut<G, C, 0, MUL_IR>::run(p.out + (int64_t)n * p.out_stride, p, ch, acc);
  }
}

// ---- backward ---------------------------------------------------------------------------------
template <class G, int C, int P, bool MUL_IR, bool NEED_R = true>
struct BwdPaths {
  __device__ __forceinline__ static void run(const float (&X)[G::D1][C], const Vec<C>* wst, const Vec<C>* grow, int lane,
                                             const float* M, const CwCoef& coef, const CwParams& p, float* gwrow,
                                             float (&gX)[G::D1][C], float (&r)[16]) {
    float W[C];
    to_array(wst[P * 32 + lane], W);
    float Gk[G::MAXD3][C];
    unstage_block<G::d3(P), C, MUL_IR>(grow + G::out_offset(P) * 32, lane, Gk);
    float gw[C];
    G::template bwd_path<P, C, NEED_R>(X, W, M, Gk, coef, gX, gw, r);
    if (p.need_gw) st_stream(gwrow + p.w_off[P], gw);
    if constexpr (P + 1 < G::NPATH) BwdPaths<G, C, P + 1, MUL_IR, NEED_R>::run(X, wst, grow, lane, M, coef, p, gwrow, gX, r);
  }
};

// cotangent row of a receiver -> lane-private staging; block P holds d3(P) vectors per lane
template <class G, int C, int P, bool MUL_IR>
struct StageG {
  __device__ __forceinline__ static void run(Vec<C>* dst, const float* grow, const CwParams& p, int ch, int lane) {
    stage_block<G::d3(P), C, MUL_IR>(dst + G::out_offset(P) * 32, grow + p.out_off[P], p.extent, ch, lane);
    if constexpr (P + 1 < G::NPATH) StageG<G, C, P + 1, MUL_IR>::run(dst, grow, p, ch, lane);
  }
};

// Sum of 16 per-lane values over the warp: on return lane L holds the total of r[L >> 1].
// Each step exchanges half of the remaining values with the partner lane, so the whole
// reduction costs about one shuffle per value instead of five.
__device__ __forceinline__ float reduce16(float (&r)[16], int lane) {
#pragma unroll
  for (int half = 8, bit = 16; half >= 1; half >>= 1, bit >>= 1) {
    const bool up = lane & bit;
#pragma unroll
    for (int t = 0; t < half; ++t) {
      const float send = up ? r[t] : r[t + half];
      const float keep = up ? r[t + half] : r[t];
      r[t] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
    }
  }
  return r[0] + __shfl_xor_sync(0xffffffffu, r[0], 1);
}

template <class G, int C, bool MUL_IR>
__global__ void __launch_bounds__(kWarps * 32, CW_MINBLOCKS) cw_bwd_kernel(const __grid_constant__ CwParams p, const __grid_constant__ CwCoef coef) {
  extern __shared__ __align__(16) float smem[];
  using S = Smem<G, C>;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* mine = smem + warp * S::kPerWarpBwd;
  Vec<C>* grow = reinterpret_cast<Vec<C>*>(mine + S::kPerWarpFwd);
  const int ch = blockIdx.y * (32 * C) + C * lane;
  const bool active = ch < p.extent;
  MTerms<G::NPAIR> mt;
  mt.load(p, lane);
  const unsigned long long pol_stream = policy_evict_first(), pol_keep = policy_evict_last();

  const int total_warps = gridDim.x * kWarps;
  for (int n = blockIdx.x * kWarps + warp; n < p.num_receivers; n += total_warps) {
    const int beg = __ldg(p.rowptr + n), end = __ldg(p.rowptr + n + 1);
    if (beg >= end) continue;
    const int nrow = p.recv_mod ? n % p.recv_mod : n;
    if (active) StageG<G, C, 0, MUL_IR>::run(grow, p.gout + (int64_t)nrow * p.out_stride, p, ch, lane);
    cp_async_commit();
    float* Msm = mine;
    float* stages = mine + S::kM;
    EdgeIds cur = {0, 0}, next = load_ids(p, beg), ahead = {0, 0};
    issue_edge_ids<G, C, MUL_IR>(p, stages, next, ch, lane, active, pol_stream, pol_keep);
    if (beg + 1 < end) ahead = load_ids(p, beg + 1);
    for (int pos = beg; pos < end; ++pos) {
      float* st = stages + ((pos - beg) & 1) * S::kPerStage;
      cur = next;
      if (pos + 1 < end) {
        next = ahead;
        issue_edge_ids<G, C, MUL_IR>(p, stages + ((pos + 1 - beg) & 1) * S::kPerStage, next, ch, lane, active, pol_stream, pol_keep);
        if (pos + 2 < end) ahead = load_ids(p, pos + 2);           // used in the next trip
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      const int eid = cur.eid;
      __syncwarp();
      mt.compute(Msm, st, lane);
      __syncwarp();
      float r[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) r[j] = 0.f;
      if (active) {
        const Vec<C>* stage = reinterpret_cast<const Vec<C>*>(st + S::kX2);
        float X[G::D1][C], gX[G::D1][C];
        unstage_block<G::D1, C, MUL_IR>(stage, lane, X);
#pragma unroll
        for (int i = 0; i < G::D1; ++i)
#pragma unroll
          for (int c = 0; c < C; ++c) gX[i][c] = 0.f;
        BwdPaths<G, C, 0, MUL_IR>::run(X, stage + G::D1 * 32, grow, lane, Msm, coef, p, p.gw + (int64_t)eid * p.w_stride + ch, gX, r);
        if (p.need_gx1) {
          emit_block<G::D1, C, MUL_IR, true>(p.gx1 + (int64_t)cur.snd * p.x1_stride + p.x1_off, p.extent, ch, gX, 0, pol_keep);
        }
      }
      if (p.need_gx2) {
        const float tot = reduce16(r, lane);
        if (!(lane & 1) && (lane >> 1) < G::NX2) atomicAdd(p.gx2 + (int64_t)eid * p.x2_stride + (lane >> 1), tot);
      }
      __syncwarp();
    }
  }
}

// ---- backward, one thread block per receiver ---------------------------------------------------
//
// Same arithmetic as cw_bwd_kernel with a different division of the work: the warps of a block
// share one receiver (its cotangent row is staged once per block instead of once per warp, which
// is what makes room in shared memory for four channels per thread at full occupancy) and deal
// the receiver's edges among themselves.  Nothing has to be combined afterwards, because every
// result of the backward pass belongs to an edge (weight gradient, x2 gradient) or is reduced in
// global memory anyway (x1 gradient).  A thread that owns four channels reads each broadcast
// entry of the per-edge matrices, issues each copy and computes each address once for four
// channels instead of two.
template <class G, int C, int P, bool MUL_IR>
struct StageGSplit {
  // the rows of the cotangent blocks are dealt round-robin to the warps of the block
  __device__ __forceinline__ static void run(Vec<C>* dst, const float* grow, const CwParams& p, int ch, int lane, int warp) {
    constexpr int D = G::d3(P);
    const float* base = grow + p.out_off[P];
#pragma unroll
    for (int t = 0; t < D; ++t) {
      if ((G::out_offset(P) + t) % kWarps == warp) {
        const float* src = MUL_IR ? base + (int64_t)ch * D + C * t : base + (int64_t)t * p.extent + ch;
        cp_async<4 * C>(dst + (G::out_offset(P) + t) * 32 + lane, src);
      }
    }
    if constexpr (P + 1 < G::NPATH) StageGSplit<G, C, P + 1, MUL_IR>::run(dst, grow, p, ch, lane, warp);
  }
};

template <class G, bool MUL_IR, bool BULK_RED, bool NEED_GX2>
__global__ void __launch_bounds__(kWarps * 32, 3) cw_bwd_block_kernel(const __grid_constant__ CwParams p, const __grid_constant__ CwCoef coef) {
  constexpr int C = 4;
  // BULK_RED (mul_ir rows only): the x1 gradient of an edge - the 32 lanes' C*D1 values are one contiguous run of
  // the sender's row - leaves as ONE bulk reduction per warp and edge instead of D1 vector reductions per lane.
  // Its shared-memory source is the slot the edge's x1 block was staged in (free once X is in registers); the
  // slot is refilled two trips later, after the issuing lane has waited for the reduction to have read it.
  constexpr bool kBulk = BULK_RED && MUL_IR;
  extern __shared__ __align__(16) float smem[];
  using S = Smem<G, C>;
  constexpr int kStage = S::kPerStage;
  constexpr int kPerWarp = S::kM + 2 * kStage;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  Vec<C>* grow = reinterpret_cast<Vec<C>*>(smem);                 // shared by the block
  float* mine = smem + S::kGrow + warp * kPerWarp;                // per warp: M, two edge stages
  float* Msm = mine;
  float* stages = mine + S::kM;
  const int ch = blockIdx.y * (32 * C) + C * lane;
  const bool active = ch < p.extent;
  MTerms<G::NPAIR> mt;
  mt.load(p, lane);
  const unsigned long long pol_stream = policy_evict_first(), pol_keep = policy_evict_last();

  for (int n = blockIdx.x; n < p.num_receivers; n += gridDim.x) {
    const int beg = __ldg(p.rowptr + n), end = __ldg(p.rowptr + n + 1);
    if (beg >= end) continue;                                      // same decision in every thread of the block
    const int nrow = p.recv_mod ? n % p.recv_mod : n;
    if (kBulk) {                                                   // the last reduction of the previous receiver has left its slot
      if (lane == 0) bulk_wait_read();
      __syncwarp();
    }
    __syncthreads();                                               // everybody is done with the previous cotangent row
    if (active) StageGSplit<G, C, 0, MUL_IR>::run(grow, p.gout + (int64_t)nrow * p.out_stride, p, ch, lane, warp);
    cp_async_commit();
    int pos = beg + warp;
    EdgeIds cur = {0, 0}, next = {0, 0}, ahead = {0, 0};
    if (pos < end) {
      next = load_ids(p, pos);
      issue_edge_ids<G, C, MUL_IR>(p, stages, next, ch, lane, active, pol_stream, pol_keep);
    } else {
      cp_async_commit();
    }
    if (pos + kWarps < end) ahead = load_ids(p, pos + kWarps);
    cp_async_wait<1>();                                            // this thread's share of the cotangent row has landed
    __syncthreads();                                               // ... and everybody else's
    for (int it = 0; pos < end; pos += kWarps, ++it) {
      float* st = stages + (it & 1) * kStage;
      cur = next;
      if (!kBulk) {
        if (pos + kWarps < end) {
          next = ahead;
          issue_edge_ids<G, C, MUL_IR>(p, stages + ((it + 1) & 1) * kStage, next, ch, lane, active, pol_stream, pol_keep);
          if (pos + 2 * kWarps < end) ahead = load_ids(p, pos + 2 * kWarps);   // used in the next trip
          cp_async_wait<1>();
        } else {
          cp_async_wait<0>();
        }
      } else {
        cp_async_wait<0>();                                          // the copies of this edge are the only ones in flight
      }
      const int eid = cur.eid;
      __syncwarp();
      mt.compute(Msm, st, lane);
      __syncwarp();
      if (kBulk) {
        // the other slot is the source of the previous edge's reduction: refill it only after that has been read
        // (the matrices above were computed in the meantime)
        if (lane == 0) bulk_wait_read();
        __syncwarp();
        if (pos + kWarps < end) {
          next = ahead;
          issue_edge_ids<G, C, MUL_IR>(p, stages + ((it + 1) & 1) * kStage, next, ch, lane, active, pol_stream, pol_keep);
          if (pos + 2 * kWarps < end) ahead = load_ids(p, pos + 2 * kWarps);
        }
      }
      float r[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) r[j] = 0.f;
      if (active) {
        const Vec<C>* stage = reinterpret_cast<const Vec<C>*>(st + S::kX2);
        float X[G::D1][C], gX[G::D1][C];
        unstage_block<G::D1, C, MUL_IR>(stage, lane, X);
#pragma unroll
        for (int i = 0; i < G::D1; ++i)
#pragma unroll
          for (int c = 0; c < C; ++c) gX[i][c] = 0.f;
        BwdPaths<G, C, 0, MUL_IR, NEED_GX2>::run(X, stage + G::D1 * 32, grow, lane, Msm, coef, p, p.gw + (int64_t)eid * p.w_stride + ch, gX, r);
        if (p.need_gx1 && !kBulk) {
          emit_block<G::D1, C, MUL_IR, true>(p.gx1 + (int64_t)cur.snd * p.x1_stride + p.x1_off, p.extent, ch, gX, 0, pol_keep);
        }
        if (p.need_gx1 && kBulk) {
          // the lane's C*D1 values in the order of the global row (channel-major), lane after lane
          float f[G::D1 * C];
#pragma unroll
          for (int i = 0; i < G::D1; ++i)
#pragma unroll
            for (int c = 0; c < C; ++c) f[c * G::D1 + i] = gX[i][c];
          __syncwarp();                                              // every lane has taken its X out of the slot
          float4* slot = reinterpret_cast<float4*>(st + S::kX2);
#pragma unroll
          for (int t = 0; t < G::D1; ++t) slot[lane * G::D1 + t] = make_float4(f[4 * t], f[4 * t + 1], f[4 * t + 2], f[4 * t + 3]);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0)
            bulk_reduce_add(p.gx1 + (int64_t)cur.snd * p.x1_stride + p.x1_off + (int64_t)(blockIdx.y * 32 * C) * G::D1, slot,
                            (unsigned)(G::D1 * 32 * C * sizeof(float)), pol_keep);
        }
      }
      if (NEED_GX2) {
        const float tot = reduce16(r, lane);
        // a reduction without return value: the warp does not wait for it (a load-add-store would stall on the load)
        if (!(lane & 1) && (lane >> 1) < G::NX2) atomicAdd(p.gx2 + (int64_t)eid * p.x2_stride + (lane >> 1), tot);
      }
      __syncwarp();
    }
  }
  if (kBulk && lane == 0) bulk_wait_all();                           // shared memory stays allocated until the last reduction is done
}

// ---- registry -----------------------------------------------------------------------------------
struct GroupEntry {
  const char* signature;
  int d1, npath, npair, nterm, sumd3, nx2, nval, nterm_fwd;
  int (*fwd)(const CwParams&, int, int, cudaStream_t);
  int (*bwd)(const CwParams&, const CwCoef&, int, int, cudaStream_t);
  int (*fwd_bulk)(const CwParams&, int, int, cudaStream_t);
  int (*bwd_block)(const CwParams&, const CwCoef&, int, int, cudaStream_t);
};

int grid_x(int num_receivers) {
  const int want = (num_receivers + kWarps - 1) / kWarps;
  const int cap = 148 * 32;
  return want < 1 ? 1 : (want < cap ? want : cap);
}

template <class G, int C, bool A>
int launch_fwd_t(const CwParams& p, cudaStream_t st) {
  const size_t smem = Smem<G, C>::bytes_fwd();
  static cueq::PerDeviceFlag configured;
  if (!configured.get()) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(cw_fwd_kernel<G, C, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set();
  }
  dim3 grid(grid_x(p.num_receivers), (p.extent + 32 * C - 1) / (32 * C));
  cw_fwd_kernel<G, C, A><<<grid, kWarps * 32, smem, st>>>(p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

template <class G, int C, bool A>
int launch_fwd_bulk_t(const CwParams& p, cudaStream_t st) {
  const size_t smem = SmemBulk<G, C>::bytes();
  static cueq::PerDeviceFlag configured;
  if (!configured.get()) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(cw_fwd_bulk_kernel<G, C, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set();
  }
  dim3 grid(grid_x(p.num_receivers), (p.extent + 32 * C - 1) / (32 * C));
  cw_fwd_bulk_kernel<G, C, A><<<grid, kWarps * 32, smem, st>>>(p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

template <class G>
int launch_fwd(const CwParams& p, int mul_ir, int cpl, cudaStream_t st) {
  if (cpl == 2) return mul_ir ? launch_fwd_t<G, 2, true>(p, st) : launch_fwd_t<G, 2, false>(p, st);
  return mul_ir ? launch_fwd_t<G, 4, true>(p, st) : launch_fwd_t<G, 4, false>(p, st);
}

template <class G>
int launch_fwd_bulk(const CwParams& p, int mul_ir, int cpl, cudaStream_t st) {
  if (cpl == 2) return mul_ir ? launch_fwd_bulk_t<G, 2, true>(p, st) : launch_fwd_bulk_t<G, 2, false>(p, st);
  return mul_ir ? launch_fwd_bulk_t<G, 4, true>(p, st) : launch_fwd_bulk_t<G, 4, false>(p, st);
}

template <class G, int C, bool A>
int launch_bwd_t(const CwParams& p, const CwCoef& coef, cudaStream_t st) {
  const size_t smem = Smem<G, C>::bytes_bwd();
  static cueq::PerDeviceFlag configured;
  if (!configured.get()) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(cw_bwd_kernel<G, C, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set();
  }
  dim3 grid(grid_x(p.num_receivers), (p.extent + 32 * C - 1) / (32 * C));
  cw_bwd_kernel<G, C, A><<<grid, kWarps * 32, smem, st>>>(p, coef);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

template <class G>
int launch_bwd(const CwParams& p, const CwCoef& coef, int mul_ir, int cpl, cudaStream_t st) {
  if (cpl == 2) return mul_ir ? launch_bwd_t<G, 2, true>(p, coef, st) : launch_bwd_t<G, 2, false>(p, coef, st);
  return mul_ir ? launch_bwd_t<G, 4, true>(p, coef, st) : launch_bwd_t<G, 4, false>(p, coef, st);
}

template <class G, bool A, bool BULK, bool GX2>
int launch_bwd_block_t(const CwParams& p, const CwCoef& coef, cudaStream_t st) {
  using S = Smem<G, 4>;
  const size_t smem = sizeof(float) * (S::kGrow + kWarps * S::kPerWarpFwd);
  static cueq::PerDeviceFlag configured;
  if (!configured.get()) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(cw_bwd_block_kernel<G, A, BULK, GX2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set();
  }
  // blocks walk the receivers with a grid stride; many short-lived blocks (a few receivers each) let the hardware
  // balance the uneven edge counts better than eight waves of long ones (l = 3 launch 3.48 -> 3.40 ms)
  const int cap = 148 * 96;
  dim3 grid(p.num_receivers < cap ? p.num_receivers : cap, (p.extent + 127) / 128);
  cw_bwd_block_kernel<G, A, BULK, GX2><<<grid, kWarps * 32, smem, st>>>(p, coef);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

// bulk: the x1 gradient leaves as one bulk reduction per warp and edge; needs mul_ir rows whose blocks start on
// 16-byte boundaries (checked here: a misaligned bulk operation is an illegal instruction, not an error code)
template <class G>
int launch_bwd_block(const CwParams& p, const CwCoef& coef, int mul_ir, int bulk, cudaStream_t st) {
  const bool aligned = (reinterpret_cast<uintptr_t>(p.gx1) % 16 == 0) && (p.x1_stride % 4 == 0) && (p.x1_off % 4 == 0) && (p.extent % 128 == 0);
  // the x2-gradient partials are a third of the arithmetic: a launch that does not need them runs without
  if (bulk && mul_ir && p.need_gx1 && aligned)
    return p.need_gx2 ? launch_bwd_block_t<G, true, true, true>(p, coef, st) : launch_bwd_block_t<G, true, true, false>(p, coef, st);
  if (mul_ir) return p.need_gx2 ? launch_bwd_block_t<G, true, false, true>(p, coef, st) : launch_bwd_block_t<G, true, false, false>(p, coef, st);
  return p.need_gx2 ? launch_bwd_block_t<G, false, false, true>(p, coef, st) : launch_bwd_block_t<G, false, false, false>(p, coef, st);
}

#define CW_ENTRY(G) {G::signature(), G::D1, G::NPATH, G::NPAIR, G::NTERM, G::SUMD3, G::NX2, G::NVAL, G::NTERM_FWD, &launch_fwd<G>, &launch_bwd<G>, &launch_fwd_bulk<G>, &launch_bwd_block<G>},
const GroupEntry kGroups[] = {CW_FOR_EACH_GROUP(CW_ENTRY)};
constexpr int kNumGroups = sizeof(kGroups) / sizeof(kGroups[0]);

int pick_cpl(const cueq_cw_args* a) {
  if (a->channels_per_lane == 2 || a->channels_per_lane == 4) return a->channels_per_lane;
  return a->extent >= 64 ? 2 : 4;
}

int fill_params(const cueq_cw_args* a, const GroupEntry& g, CwParams& p, int expected_terms) {
  if (!a) return cueq::fail("channelwise: null arguments");
  if (a->extent < 4 || a->extent % 4) return cueq::fail("channelwise: extent %d must be a positive multiple of 4", a->extent);
  if (a->x1_mul_ir != a->out_mul_ir) return cueq::fail("channelwise: x1 and out must use the same layout");
  if (a->staging != 0 && a->staging != 1) return cueq::fail("channelwise: staging must be 0 (cp.async) or 1 (bulk copy)");
  if (a->channels_per_lane != 0 && a->channels_per_lane != 2 && a->channels_per_lane != 4)
    return cueq::fail("channelwise: channels_per_lane must be 0 (auto), 2 or 4");
  if (a->num_paths != g.npath) return cueq::fail("channelwise: group has %d paths, got %d", g.npath, a->num_paths);
  if (a->num_terms != expected_terms) return cueq::fail("channelwise: this call's table has %d terms, got %d", expected_terms, a->num_terms);
  if (!a->rowptr || !a->tab_start || !a->tab_j || !a->tab_c) return cueq::fail("channelwise: null table or rowptr");
  if (a->num_receivers < 0) return cueq::fail("channelwise: negative receiver count");
  std::memset(&p, 0, sizeof(p));
  p.w = (const float*)a->w; p.x1 = (const float*)a->x1; p.x2 = (const float*)a->x2; p.out = (float*)a->out;
  p.gout = (const float*)a->gout; p.gw = (float*)a->gw; p.gx1 = (float*)a->gx1; p.gx2 = (float*)a->gx2;
  p.senders = a->senders; p.order = a->order; p.rowptr = a->rowptr;
  p.tab_start = a->tab_start; p.tab_j = a->tab_j; p.tab_c = a->tab_c;
  p.w_stride = a->w_stride; p.x1_stride = a->x1_stride; p.x2_stride = a->x2_stride; p.out_stride = a->out_stride;
  p.num_receivers = (int)a->num_receivers; p.extent = a->extent; p.x1_off = a->x1_offset;
  for (int q = 0; q < g.npath; ++q) {
    p.w_off[q] = a->w_offset[q];
    p.out_off[q] = a->out_offset[q];
    if ((p.w_off[q] | p.out_off[q]) & 3) return cueq::fail("channelwise: segment offsets must be multiples of 4 elements");
  }
  if (p.x1_off & 3) return cueq::fail("channelwise: x1 offset must be a multiple of 4 elements");
  if ((p.w_stride | p.x1_stride | p.out_stride) & 3) return cueq::fail("channelwise: row strides must be multiples of 4 elements");
  const uintptr_t ptrs = (uintptr_t)a->w | (uintptr_t)a->x1 | (uintptr_t)a->x2 | (uintptr_t)a->out | (uintptr_t)a->gout | (uintptr_t)a->gw | (uintptr_t)a->gx1;
  if (a->x2_stride & 3) return cueq::fail("channelwise: x2 row stride must be a multiple of 4 elements");
  if (ptrs & 15) return cueq::fail("channelwise: tensors must be 16-byte aligned");
  p.need_gw = a->gw != nullptr; p.need_gx1 = a->gx1 != nullptr; p.need_gx2 = a->gx2 != nullptr;
  return 0;
}

}  // namespace

extern "C" int cueq_b200_cw_num_groups(void) { return kNumGroups; }

extern "C" const char* cueq_b200_cw_group_signature(int g) { return (g >= 0 && g < kNumGroups) ? kGroups[g].signature : nullptr; }

extern "C" int cueq_b200_cw_group_info(int g, int32_t* d1, int32_t* npath, int32_t* npair, int32_t* nterm) {
  if (g < 0 || g >= kNumGroups) return cueq::fail("channelwise: group %d out of range", g);
  if (d1) *d1 = kGroups[g].d1;
  if (npath) *npath = kGroups[g].npath;
  if (npair) *npair = kGroups[g].npair;
  if (nterm) *nterm = kGroups[g].nterm;
  return 0;
}

extern "C" int cueq_b200_cw_forward(int g, const cueq_cw_args* a, void* stream) {
  if (g < 0 || g >= kNumGroups) return cueq::fail("channelwise: group %d out of range", g);
  CwParams p;
  if (int rc = fill_params(a, kGroups[g], p, kGroups[g].nterm_fwd)) return rc;
  if (!p.w || !p.x1 || !p.x2 || !p.out) return cueq::fail("channelwise forward: null tensor");
  if (p.num_receivers == 0) return 0;
  p.status = reinterpret_cast<int*>(a->status);
  if (a->variant < 0 || a->variant > 2) return cueq::fail("channelwise: variant must be 0 (automatic), 1 or 2");
  if (a->staging == 1) return kGroups[g].fwd_bulk(p, a->x1_mul_ir, pick_cpl(a), reinterpret_cast<cudaStream_t>(stream));
  return kGroups[g].fwd(p, a->x1_mul_ir, pick_cpl(a), reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int cueq_b200_cw_backward(int g, const cueq_cw_args* a, void* stream) {
  if (g < 0 || g >= kNumGroups) return cueq::fail("channelwise: group %d out of range", g);
  CwParams p;
  if (int rc = fill_params(a, kGroups[g], p, kGroups[g].nterm)) return rc;
  if (!p.w || !p.x1 || !p.x2 || !p.gout) return cueq::fail("channelwise backward: null tensor");
  if (!a->bwd_coef) return cueq::fail("channelwise backward: null coefficient table");
  if (kGroups[g].nterm > kMaxTerms) return cueq::fail("channelwise backward: too many terms");
  if (p.num_receivers == 0) return 0;
  p.recv_mod = a->recv_mod;
  CwCoef coef;
  std::memset(&coef, 0, sizeof(coef));
  for (int t = 0; t < kGroups[g].nterm; ++t) coef.c[t] = a->bwd_coef[t];
  if (a->variant < 0 || a->variant > 3) return cueq::fail("channelwise backward: variant must be 0 (automatic), 1, 2 or 3");
  // one thread block per receiver needs the four-channel layout (extent a multiple of 4 is given);
  // it is the default from 128 channels on, where a warp's 128 channels are all in use
  const bool block_per_receiver = a->variant >= 2 || (a->variant == 0 && a->channels_per_lane != 2 && a->extent % 128 == 0);
  if (a->variant == 3 && a->extent % 128) return cueq::fail("channelwise backward: variant 3 needs a multiple of 128 channels");
  // bulk reductions pay from three components per channel on (one 1.5 KB operation instead of three vector
  // reductions per lane); for the scalar block (512 bytes per edge) the vector reductions are faster
  const bool bulk = a->variant == 3 || (a->variant == 0 && kGroups[g].d1 >= 3);
  if (block_per_receiver)
    return kGroups[g].bwd_block(p, coef, a->x1_mul_ir, bulk, reinterpret_cast<cudaStream_t>(stream));
  return kGroups[g].bwd(p, coef, a->x1_mul_ir, pick_cpl(a), reinterpret_cast<cudaStream_t>(stream));
}

// ---- forward without caller-provided scratch ----------------------------------------------------
//
// cueq_b200_cw_forward needs two pieces of device memory besides its inputs and outputs: the
// CSR row pointers over receivers and the term tables.  Some hosts of this library cannot
// provide them: code that runs where device allocation is forbidden or owned by someone else
// (an inference-engine plugin whose enqueue call gets only its input and output bindings, a
// callback running inside a memory pool it must not grow, a real-time loop that may not call
// the allocator).  For those there is one entry point whose scratch lives in a fixed array
// inside the library image.  The array exists once per GPU that loads the library, for the
// life of the process, and every call reuses it.
namespace {

constexpr int kNoAllocMaxReceivers = 262144;   // row pointers: (N + 1) * 4 bytes = 1 MiB
constexpr int kNoAllocMaxPairs = 256;
constexpr int kNoAllocMaxTerms = 256;
constexpr size_t kScratchRowptr = 0;
constexpr size_t kScratchTabStart = ((size_t)(kNoAllocMaxReceivers + 1) * 4 + 255) & ~size_t(255);
constexpr size_t kScratchTabJ = kScratchTabStart + ((kNoAllocMaxPairs + 1) * 4 + 255) / 256 * 256;
constexpr size_t kScratchTabC = kScratchTabJ + (kNoAllocMaxTerms * 4 + 255) / 256 * 256;
constexpr size_t kScratchBytes = kScratchTabC + (kNoAllocMaxTerms * 4 + 255) / 256 * 256;

// Host code may only use this name with cudaGetSymbolAddress: as a plain expression it is the
// host-side shadow of the symbol, not a device address.
static __device__ __align__(256) unsigned char g_cw_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

struct NoAllocTables {
  int start[kNoAllocMaxPairs + 1];
  int j[kNoAllocMaxTerms];
  float c[kNoAllocMaxTerms];
};

// rowptr[r] = first position whose receiver is >= r (receivers sorted ascending); also copies
// the term tables from the kernel parameters into the scratch array
__global__ void cw_noalloc_prepare(const int* __restrict__ receivers, int num_edges, int num_receivers, int* __restrict__ rowptr,
                                   const __grid_constant__ NoAllocTables t, int npair, int nterm, int* tab_start, int* tab_j,
                                   float* tab_c) {
  const int gid = blockIdx.x * blockDim.x + threadIdx.x;
  for (int r = gid; r <= num_receivers; r += gridDim.x * blockDim.x) {
    int lo = 0, hi = num_edges;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(receivers + mid) < r) lo = mid + 1; else hi = mid;
    }
    rowptr[r] = lo;
  }
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i <= npair; i += blockDim.x) tab_start[i] = t.start[i];
    for (int i = threadIdx.x; i < nterm; i += blockDim.x) { tab_j[i] = t.j[i]; tab_c[i] = t.c[i]; }
  }
}

}  // namespace

extern "C" int cueq_b200_cw_forward_noalloc(int g, const cueq_cw_noalloc_args* a, void* stream) {
  if (g < 0 || g >= kNumGroups) return cueq::fail("channelwise (no-alloc): group %d out of range", g);
  if (!a) return cueq::fail("channelwise (no-alloc): null arguments");
  const GroupEntry& ge = kGroups[g];
  if (a->num_receivers > kNoAllocMaxReceivers)
    return cueq::fail("channelwise (no-alloc): %lld receivers exceed the built-in scratch (max %d); use cueq_b200_cw_forward",
                      (long long)a->num_receivers, kNoAllocMaxReceivers);
  if (ge.nval > kNoAllocMaxPairs || ge.nterm_fwd > kNoAllocMaxTerms)
    return cueq::fail("channelwise (no-alloc): group tables exceed the built-in scratch");
  if (a->num_edges < 0 || a->num_edges > 2147483647LL) return cueq::fail("channelwise (no-alloc): invalid edge count");
  if (!a->receivers && a->num_edges > 0) return cueq::fail("channelwise (no-alloc): null receivers");
  if (!a->tab_start_host || !a->tab_j_host || !a->tab_c_host) return cueq::fail("channelwise (no-alloc): null host table");

  int dev = 0;
  CUEQ_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return cueq::fail("channelwise (no-alloc): device ordinal %d not supported", dev);
  if (!g_scratch_ptr[dev]) {  // set-up, once per device, with that device current
    void* ptr = nullptr;
    CUEQ_CUDA_OK(cudaGetSymbolAddress(&ptr, g_cw_scratch));
    g_scratch_ptr[dev] = ptr;
  }
  unsigned char* scratch = static_cast<unsigned char*>(g_scratch_ptr[dev]);
  int* rowptr = reinterpret_cast<int*>(scratch + kScratchRowptr);
  int* tab_start = reinterpret_cast<int*>(scratch + kScratchTabStart);
  int* tab_j = reinterpret_cast<int*>(scratch + kScratchTabJ);
  float* tab_c = reinterpret_cast<float*>(scratch + kScratchTabC);

  cueq_cw_args full;
  std::memset(&full, 0, sizeof(full));
  full.w = a->w; full.x1 = a->x1; full.x2 = a->x2; full.out = a->out;
  full.senders = a->senders; full.order = nullptr; full.rowptr = rowptr;
  full.tab_start = tab_start; full.tab_j = tab_j; full.tab_c = tab_c;
  full.w_stride = a->w_stride; full.x1_stride = a->x1_stride; full.x2_stride = a->x2_stride; full.out_stride = a->out_stride;
  full.num_receivers = a->num_receivers; full.extent = a->extent; full.x1_offset = a->x1_offset;
  full.num_paths = a->num_paths; full.num_terms = a->num_terms;
  for (int q = 0; q < 8; ++q) { full.w_offset[q] = a->w_offset[q]; full.out_offset[q] = a->out_offset[q]; }
  full.x1_mul_ir = a->mul_ir; full.out_mul_ir = a->mul_ir; full.channels_per_lane = 0;
  CwParams p;
  if (int rc = fill_params(&full, ge, p, ge.nterm_fwd)) return rc;
  if (!p.w || !p.x1 || !p.x2 || !p.out) return cueq::fail("channelwise (no-alloc): null tensor");
  if (p.num_receivers == 0) return 0;

  NoAllocTables t;
  std::memset(&t, 0, sizeof(t));
  for (int i = 0; i <= ge.nval; ++i) t.start[i] = a->tab_start_host[i];
  for (int i = 0; i < ge.nterm_fwd; ++i) { t.j[i] = a->tab_j_host[i]; t.c[i] = a->tab_c_host[i]; }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int blocks = (int)((a->num_receivers + 1 + 255) / 256);
  cw_noalloc_prepare<<<blocks < 1 ? 1 : blocks, 256, 0, st>>>(a->receivers, (int)a->num_edges, (int)a->num_receivers, rowptr, t, ge.nval,
                                                              ge.nterm_fwd, tab_start, tab_j, tab_c);
  CUEQ_CUDA_OK(cudaGetLastError());
  return ge.fwd(p, a->mul_ir, pick_cpl(&full), st);
}

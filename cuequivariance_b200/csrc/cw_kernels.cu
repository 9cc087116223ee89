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
//   * one warp owns one receiver at a time; a lane owns four consecutive channels (one
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
#include <cstring>

#include "common.cuh"
#include "generated/cw_groups.cuh"

namespace {

constexpr int kMaxPaths = 8;
constexpr int kMaxTerms = 160;
constexpr int kWarps = 4;  // warps per CTA

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
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void red_add_v4(float* addr, const float (&v)[4]) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3])
               : "memory");
}
__device__ __forceinline__ void st_stream_v4(float* addr, const float (&v)[4]) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3])
               : "memory");
}

// shared memory carve-up, in floats
template <class G>
struct Smem {
  static constexpr int kTabInts = (G::NPAIR + 1) + G::NTERM;               // tab_start + tab_j
  static constexpr int kTab = ((kTabInts + G::NTERM + 3) / 4) * 4;          // + tab_c
  static constexpr int kM = G::NPAIR_PAD;                                   // per stage
  static constexpr int kStage = (G::D1 + G::NPATH) * 32 * 4;                // per stage: x1 block + weights
  static constexpr int kPerWarpFwd = 2 * kM + 2 * kStage;
  static constexpr int kGrow = G::SUMD3 * 32 * 4;                           // cotangent row of the receiver
  static constexpr int kPerWarpBwd = kPerWarpFwd + kGrow;
  static constexpr size_t bytes_fwd() { return sizeof(float) * (kTab + kWarps * kPerWarpFwd); }
  static constexpr size_t bytes_bwd() { return sizeof(float) * (kTab + kWarps * kPerWarpBwd); }
};

// x1 block of one edge -> lane-private staging (D1 float4 per lane)
template <class G, bool MUL_IR>
__device__ __forceinline__ void stage_x1(float4* dst, const float* row, int extent, int c0, int lane) {
#pragma unroll
  for (int t = 0; t < G::D1; ++t) {
    const float* src = MUL_IR ? row + (int64_t)(c0 + 4 * lane) * G::D1 + 4 * t : row + (int64_t)t * extent + c0 + 4 * lane;
    cp_async16(dst + t * 32 + lane, src);
  }
}

// staging -> X[i][c]
template <class G, bool MUL_IR>
__device__ __forceinline__ void unstage_x1(const float4* src, int lane, float (&X)[G::D1][4]) {
  float f[G::D1 * 4];
#pragma unroll
  for (int t = 0; t < G::D1; ++t) {
    const float4 v = src[t * 32 + lane];
    f[4 * t + 0] = v.x; f[4 * t + 1] = v.y; f[4 * t + 2] = v.z; f[4 * t + 3] = v.w;
  }
#pragma unroll
  for (int i = 0; i < G::D1; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) X[i][c] = MUL_IR ? f[c * G::D1 + i] : f[4 * i + c];
}

// M[q] = sum_t c[t] * x2[j[t]] for every pair q of the group, spread over the lanes
template <class G>
__device__ __forceinline__ void compute_m(float* M, const int* tab_start, const int* tab_j, const float* tab_c,
                                          const float* __restrict__ x2row, int lane) {
  for (int q = lane; q < G::NPAIR; q += 32) {
    const int t0 = tab_start[q], t1 = tab_start[q + 1];
    float m = 0.f;
    for (int t = t0; t < t1; ++t) m = fmaf(tab_c[t], __ldg(x2row + tab_j[t]), m);
    M[q] = m;
  }
}

template <class G>
__device__ __forceinline__ void load_tables(float* smem, const CwParams& p, int*& tab_start, int*& tab_j, float*& tab_c) {
  tab_start = reinterpret_cast<int*>(smem);
  tab_j = tab_start + (G::NPAIR + 1);
  tab_c = smem + Smem<G>::kTabInts;
  for (int i = threadIdx.x; i < G::NPAIR + 1; i += blockDim.x) tab_start[i] = p.tab_start[i];
  for (int i = threadIdx.x; i < G::NTERM; i += blockDim.x) {
    tab_j[i] = p.tab_j[i];
    tab_c[i] = p.tab_c[i];
  }
  __syncthreads();
}

template <class G, int P, bool X1_MUL_IR>
struct FwdPaths {
  __device__ __forceinline__ static void run(const float (&X)[G::D1][4], const float4* wst, int lane, const float* M,
                                             float (&acc)[G::SUMD3][4]) {
    const float4 v = wst[P * 32 + lane];
    const float W[4] = {v.x, v.y, v.z, v.w};
    G::template fwd_path<P>(X, W, M, acc);
    if constexpr (P + 1 < G::NPATH) FwdPaths<G, P + 1, X1_MUL_IR>::run(X, wst, lane, M, acc);
  }
};

template <class G, int P, bool OUT_MUL_IR>
struct StoreOut {
  __device__ __forceinline__ static void run(float* orow, const CwParams& p, int c0, int lane, const float (&acc)[G::SUMD3][4]) {
    constexpr int D3 = G::d3(P);
    constexpr int O = G::out_offset(P);
    float* base = orow + p.out_off[P];
    if (OUT_MUL_IR) {
      float f[D3 * 4];
#pragma unroll
      for (int k = 0; k < D3; ++k)
#pragma unroll
        for (int c = 0; c < 4; ++c) f[c * D3 + k] = acc[O + k][c];
#pragma unroll
      for (int t = 0; t < D3; ++t) {
        const float v[4] = {f[4 * t], f[4 * t + 1], f[4 * t + 2], f[4 * t + 3]};
        st_stream_v4(base + (int64_t)(c0 + 4 * lane) * D3 + 4 * t, v);
      }
    } else {
#pragma unroll
      for (int k = 0; k < D3; ++k) st_stream_v4(base + (int64_t)k * p.extent + c0 + 4 * lane, acc[O + k]);
    }
    if constexpr (P + 1 < G::NPATH) StoreOut<G, P + 1, OUT_MUL_IR>::run(orow, p, c0, lane, acc);
  }
};

template <class G, bool X1_MUL_IR, bool OUT_MUL_IR>
__global__ void __launch_bounds__(kWarps * 32) cw_fwd_kernel(const __grid_constant__ CwParams p) {
  extern __shared__ __align__(16) float smem[];
  int *tab_start, *tab_j;
  float* tab_c;
  load_tables<G>(smem, p, tab_start, tab_j, tab_c);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* mine = smem + Smem<G>::kTab + warp * Smem<G>::kPerWarpFwd;
  float* Msm[2] = {mine, mine + Smem<G>::kM};
  float4* stage[2] = {reinterpret_cast<float4*>(mine + 2 * Smem<G>::kM),
                      reinterpret_cast<float4*>(mine + 2 * Smem<G>::kM + Smem<G>::kStage)};
  const int c0 = blockIdx.y * 128;
  const bool active = c0 + 4 * lane < p.extent;

  auto issue = [&](int pos, int s) {
    const int eid = p.order ? __ldg(p.order + pos) : pos;
    if (active) {
      const int snd = p.senders ? __ldg(p.senders + eid) : eid;
      stage_x1<G, X1_MUL_IR>(stage[s], p.x1 + (int64_t)snd * p.x1_stride + p.x1_off, p.extent, c0, lane);
      const float* wrow = p.w + (int64_t)eid * p.w_stride + c0 + 4 * lane;
      float4* wst = stage[s] + G::D1 * 32;
#pragma unroll
      for (int q = 0; q < G::NPATH; ++q) cp_async16(wst + q * 32 + lane, wrow + p.w_off[q]);
    }
    cp_async_commit();
    return eid;
  };

  const int total_warps = gridDim.x * kWarps;
  for (int n = blockIdx.x * kWarps + warp; n < p.num_receivers; n += total_warps) {
    const int beg = __ldg(p.rowptr + n), end = __ldg(p.rowptr + n + 1);
    float acc[G::SUMD3][4];
#pragma unroll
    for (int a = 0; a < G::SUMD3; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.f;
    int eid = 0, eid_next = 0;
    if (beg < end) eid_next = issue(beg, 0);
    for (int pos = beg; pos < end; ++pos) {
      const int s = (pos - beg) & 1;
      eid = eid_next;
      if (pos + 1 < end) eid_next = issue(pos + 1, s ^ 1);
      compute_m<G>(Msm[s], tab_start, tab_j, tab_c, p.x2 + (int64_t)eid * p.x2_stride, lane);
      if (pos + 1 < end) cp_async_wait<1>(); else cp_async_wait<0>();
      __syncwarp();
      if (active) {
        float X[G::D1][4];
        unstage_x1<G, X1_MUL_IR>(stage[s], lane, X);
        FwdPaths<G, 0, X1_MUL_IR>::run(X, stage[s] + G::D1 * 32, lane, Msm[s], acc);
      }
      __syncwarp();
    }
    if (active) StoreOut<G, 0, OUT_MUL_IR>::run(p.out + (int64_t)n * p.out_stride, p, c0, lane, acc);
  }
}

// ---- backward ---------------------------------------------------------------------------------
template <class G, int P, bool X1_MUL_IR, bool OUT_MUL_IR>
struct BwdPaths {
  __device__ __forceinline__ static void run(const float (&X)[G::D1][4], const float4* wst, const float4* grow, int lane,
                                             const float* M, const CwCoef& coef, const CwParams& p, int64_t eid, int c0,
                                             float (&gX)[G::D1][4], float (&r)[G::NX2]) {
    constexpr int D3 = G::d3(P);
    constexpr int O = G::out_offset(P);
    const float4 v = wst[P * 32 + lane];
    const float W[4] = {v.x, v.y, v.z, v.w};
    float Gk[G::MAXD3][4];
    {
      float f[D3 * 4];
#pragma unroll
      for (int t = 0; t < D3; ++t) {
        const float4 g = grow[(O + t) * 32 + lane];
        f[4 * t + 0] = g.x; f[4 * t + 1] = g.y; f[4 * t + 2] = g.z; f[4 * t + 3] = g.w;
      }
#pragma unroll
      for (int k = 0; k < D3; ++k)
#pragma unroll
        for (int c = 0; c < 4; ++c) Gk[k][c] = OUT_MUL_IR ? f[c * D3 + k] : f[4 * k + c];
    }
    float gw[4];
    G::template bwd_path<P>(X, W, M, Gk, coef, gX, gw, r);
    if (p.need_gw) st_stream_v4(p.gw + eid * p.w_stride + p.w_off[P] + c0 + 4 * lane, gw);
    if constexpr (P + 1 < G::NPATH)
      BwdPaths<G, P + 1, X1_MUL_IR, OUT_MUL_IR>::run(X, wst, grow, lane, M, coef, p, eid, c0, gX, r);
  }
};

// cotangent row of a receiver -> lane-private staging; block P holds d3(P) float4 per lane
template <class G, int P, bool OUT_MUL_IR>
struct StageG {
  __device__ __forceinline__ static void run(float4* dst, const float* grow, const CwParams& p, int c0, int lane) {
    constexpr int D3 = G::d3(P);
    constexpr int O = G::out_offset(P);
    const float* base = grow + p.out_off[P];
#pragma unroll
    for (int t = 0; t < D3; ++t) {
      const float* src = OUT_MUL_IR ? base + (int64_t)(c0 + 4 * lane) * D3 + 4 * t : base + (int64_t)t * p.extent + c0 + 4 * lane;
      cp_async16(dst + (O + t) * 32 + lane, src);
    }
    if constexpr (P + 1 < G::NPATH) StageG<G, P + 1, OUT_MUL_IR>::run(dst, grow, p, c0, lane);
  }
};

template <class G, bool X1_MUL_IR, bool OUT_MUL_IR>
__global__ void __launch_bounds__(kWarps * 32) cw_bwd_kernel(const __grid_constant__ CwParams p, const __grid_constant__ CwCoef coef) {
  extern __shared__ __align__(16) float smem[];
  int *tab_start, *tab_j;
  float* tab_c;
  load_tables<G>(smem, p, tab_start, tab_j, tab_c);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* mine = smem + Smem<G>::kTab + warp * Smem<G>::kPerWarpBwd;
  float* Msm[2] = {mine, mine + Smem<G>::kM};
  float4* stage[2] = {reinterpret_cast<float4*>(mine + 2 * Smem<G>::kM),
                      reinterpret_cast<float4*>(mine + 2 * Smem<G>::kM + Smem<G>::kStage)};
  float4* grow = reinterpret_cast<float4*>(mine + Smem<G>::kPerWarpFwd);
  const int c0 = blockIdx.y * 128;
  const bool active = c0 + 4 * lane < p.extent;

  auto issue = [&](int pos, int s) {
    const int eid = p.order ? __ldg(p.order + pos) : pos;
    if (active) {
      const int snd = p.senders ? __ldg(p.senders + eid) : eid;
      stage_x1<G, X1_MUL_IR>(stage[s], p.x1 + (int64_t)snd * p.x1_stride + p.x1_off, p.extent, c0, lane);
      const float* wrow = p.w + (int64_t)eid * p.w_stride + c0 + 4 * lane;
      float4* wst = stage[s] + G::D1 * 32;
#pragma unroll
      for (int q = 0; q < G::NPATH; ++q) cp_async16(wst + q * 32 + lane, wrow + p.w_off[q]);
    }
    cp_async_commit();
    return eid;
  };

  const int total_warps = gridDim.x * kWarps;
  for (int n = blockIdx.x * kWarps + warp; n < p.num_receivers; n += total_warps) {
    const int beg = __ldg(p.rowptr + n), end = __ldg(p.rowptr + n + 1);
    if (beg >= end) continue;
    if (active) StageG<G, 0, OUT_MUL_IR>::run(grow, p.gout + (int64_t)n * p.out_stride, p, c0, lane);
    cp_async_commit();
    int eid = 0, eid_next = issue(beg, 0);
    for (int pos = beg; pos < end; ++pos) {
      const int s = (pos - beg) & 1;
      eid = eid_next;
      if (pos + 1 < end) eid_next = issue(pos + 1, s ^ 1);
      compute_m<G>(Msm[s], tab_start, tab_j, tab_c, p.x2 + (int64_t)eid * p.x2_stride, lane);
      if (pos + 1 < end) cp_async_wait<1>(); else cp_async_wait<0>();
      __syncwarp();
      float r[G::NX2];
#pragma unroll
      for (int j = 0; j < G::NX2; ++j) r[j] = 0.f;
      if (active) {
        float X[G::D1][4], gX[G::D1][4];
        unstage_x1<G, X1_MUL_IR>(stage[s], lane, X);
#pragma unroll
        for (int i = 0; i < G::D1; ++i) gX[i][0] = gX[i][1] = gX[i][2] = gX[i][3] = 0.f;
        BwdPaths<G, 0, X1_MUL_IR, OUT_MUL_IR>::run(X, stage[s] + G::D1 * 32, grow, lane, Msm[s], coef, p, (int64_t)eid, c0, gX, r);
        if (p.need_gx1) {
          const int snd = p.senders ? __ldg(p.senders + eid) : eid;
          float* grow1 = p.gx1 + (int64_t)snd * p.x1_stride + p.x1_off;
          if (X1_MUL_IR) {
            float f[G::D1 * 4];
#pragma unroll
            for (int i = 0; i < G::D1; ++i)
#pragma unroll
              for (int c = 0; c < 4; ++c) f[c * G::D1 + i] = gX[i][c];
#pragma unroll
            for (int t = 0; t < G::D1; ++t) {
              const float v[4] = {f[4 * t], f[4 * t + 1], f[4 * t + 2], f[4 * t + 3]};
              red_add_v4(grow1 + (int64_t)(c0 + 4 * lane) * G::D1 + 4 * t, v);
            }
          } else {
#pragma unroll
            for (int i = 0; i < G::D1; ++i) red_add_v4(grow1 + (int64_t)i * p.extent + c0 + 4 * lane, gX[i]);
          }
        }
      }
      if (p.need_gx2) {
#pragma unroll
        for (int j = 0; j < G::NX2; ++j) r[j] = cueq::warp_sum(r[j]);
        float mine_r = 0.f;
#pragma unroll
        for (int j = 0; j < G::NX2; ++j)
          if (lane == j) mine_r = r[j];
        if (lane < G::NX2) atomicAdd(p.gx2 + (int64_t)eid * p.x2_stride + lane, mine_r);
      }
      __syncwarp();
    }
  }
}

// ---- registry -----------------------------------------------------------------------------------
struct GroupEntry {
  const char* signature;
  int d1, npath, npair, nterm, sumd3, nx2;
  int (*fwd)(const CwParams&, int, int, cudaStream_t);
  int (*bwd)(const CwParams&, const CwCoef&, int, int, cudaStream_t);
};

int grid_x(int num_receivers) {
  const int want = (num_receivers + kWarps - 1) / kWarps;
  const int cap = 148 * 16;
  return want < 1 ? 1 : (want < cap ? want : cap);
}

template <class G, bool A, bool B>
int launch_fwd_t(const CwParams& p, cudaStream_t st) {
  const size_t smem = Smem<G>::bytes_fwd();
  static bool configured = false;
  if (!configured) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(cw_fwd_kernel<G, A, B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid(grid_x(p.num_receivers), (p.extent + 127) / 128);
  cw_fwd_kernel<G, A, B><<<grid, kWarps * 32, smem, st>>>(p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

template <class G>
int launch_fwd(const CwParams& p, int x1_mul_ir, int out_mul_ir, cudaStream_t st) {
  if (x1_mul_ir) return out_mul_ir ? launch_fwd_t<G, true, true>(p, st) : launch_fwd_t<G, true, false>(p, st);
  return out_mul_ir ? launch_fwd_t<G, false, true>(p, st) : launch_fwd_t<G, false, false>(p, st);
}

template <class G, bool A, bool B>
int launch_bwd_t(const CwParams& p, const CwCoef& coef, cudaStream_t st) {
  const size_t smem = Smem<G>::bytes_bwd();
  static bool configured = false;
  if (!configured) {
    CUEQ_CUDA_OK(cudaFuncSetAttribute(cw_bwd_kernel<G, A, B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid(grid_x(p.num_receivers), (p.extent + 127) / 128);
  cw_bwd_kernel<G, A, B><<<grid, kWarps * 32, smem, st>>>(p, coef);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

template <class G>
int launch_bwd(const CwParams& p, const CwCoef& coef, int x1_mul_ir, int out_mul_ir, cudaStream_t st) {
  if (x1_mul_ir) return out_mul_ir ? launch_bwd_t<G, true, true>(p, coef, st) : launch_bwd_t<G, true, false>(p, coef, st);
  return out_mul_ir ? launch_bwd_t<G, false, true>(p, coef, st) : launch_bwd_t<G, false, false>(p, coef, st);
}

#define CW_ENTRY(G) {G::signature(), G::D1, G::NPATH, G::NPAIR, G::NTERM, G::SUMD3, G::NX2, &launch_fwd<G>, &launch_bwd<G>},
const GroupEntry kGroups[] = {CW_FOR_EACH_GROUP(CW_ENTRY)};
constexpr int kNumGroups = sizeof(kGroups) / sizeof(kGroups[0]);

int fill_params(const cueq_cw_args* a, const GroupEntry& g, CwParams& p) {
  if (!a) return cueq::fail("channelwise: null arguments");
  if (a->extent < 4 || a->extent % 4) return cueq::fail("channelwise: extent %d must be a positive multiple of 4", a->extent);
  if (a->num_paths != g.npath) return cueq::fail("channelwise: group has %d paths, got %d", g.npath, a->num_paths);
  if (a->num_terms != g.nterm) return cueq::fail("channelwise: group has %d terms, got %d", g.nterm, a->num_terms);
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
  const uintptr_t ptrs = (uintptr_t)a->w | (uintptr_t)a->x1 | (uintptr_t)a->out | (uintptr_t)a->gout | (uintptr_t)a->gw | (uintptr_t)a->gx1;
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
  if (int rc = fill_params(a, kGroups[g], p)) return rc;
  if (!p.w || !p.x1 || !p.x2 || !p.out) return cueq::fail("channelwise forward: null tensor");
  if (p.num_receivers == 0) return 0;
  return kGroups[g].fwd(p, a->x1_mul_ir, a->out_mul_ir, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int cueq_b200_cw_backward(int g, const cueq_cw_args* a, void* stream) {
  if (g < 0 || g >= kNumGroups) return cueq::fail("channelwise: group %d out of range", g);
  CwParams p;
  if (int rc = fill_params(a, kGroups[g], p)) return rc;
  if (!p.w || !p.x1 || !p.x2 || !p.gout) return cueq::fail("channelwise backward: null tensor");
  if (!a->bwd_coef) return cueq::fail("channelwise backward: null coefficient table");
  if (kGroups[g].nterm > kMaxTerms) return cueq::fail("channelwise backward: too many terms");
  if (p.num_receivers == 0) return 0;
  CwCoef coef;
  std::memset(&coef, 0, sizeof(coef));
  for (int t = 0; t < kGroups[g].nterm; ++t) coef.c[t] = a->bwd_coef[t];
  return kGroups[g].bwd(p, coef, a->x1_mul_ir, a->out_mul_ir, reinterpret_cast<cudaStream_t>(stream));
}

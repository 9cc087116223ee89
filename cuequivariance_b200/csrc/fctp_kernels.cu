// Fully connected ("uvw") tensor product: the CUDA-core kernels around the tensor-core GEMM.
//
// For one path (l1, l2, l3) of ``uvw,iu,jv,kw+ijk`` (descriptor:
// cuequivariance/group_theory/descriptors/irreps_tp.py:22-91) with coupling tensor C[i,j,k]:
//   build   : Z[(z,k), (u,v)] = sum_ij C[i,j,k] x1[z,i,u] x2[z,j,v]         (GEMM operand: bf16 for the
//             bf16 GEMM, float32 for the float32-accurate three-pass TF32 GEMM; rows may be column
//             blocks of a wider matrix, so that the paths feeding one output irrep share one GEMM)
//   GEMMs   : out[(z,k), w] += Z W;   gW = Z^T gout;   gZ = gout W^T          (gemm_tc.cu)
//   consume : gx1[z,i,u] += sum_jkv C[i,j,k] gZ[(z,k),(u,v)] x2[z,j,v]
//             gx2[z,j,v] += sum_iku C[i,j,k] gZ[(z,k),(u,v)] x1[z,i,u]
// Both kernels first contract the coupling tensor with one operand per sample
// (T[k,i,v] = sum_j C x2[j,v], S[k,j,u] = sum_i C x1[i,u]; a few hundred values kept in shared
// memory), so the per-element work on the big (u,v) axis is d1 (or d1+d2) multiply-adds instead
// of the number of non-zero couplings.  One CTA per sample; lanes run along v, so every access
// to Z / gZ is a contiguous 128-byte row segment.
#include <cuda_bf16.h>

#include <cstdint>
#include <cstring>

#include "common.cuh"

namespace {

constexpr int kMaxD = 7;            // irrep dimension up to l = 3
constexpr int kThreadsF = 256;
constexpr int kThreadsFast = 64;    // compile-time kernels: small blocks, more of them per SM (the phases of a sample - load,
                                    // per-sample tables, main loop, write-back - are serial inside a block and overlap across blocks)

struct FctpParams {
  const void* x1;
  const void* x2;
  void* z;            // build: bf16 output; consume: gZ input
  float* gx1;
  float* gx2;
  int64_t ld1, ld2;   // row pitches of x1 / x2 (and gx1 / gx2) in elements
  int64_t batch;
  int off1, off2;     // element offsets of the path's segments inside a row
  int d1, d2, d3, U, V;
  int z_is_bf16;      // element type of Z / gZ
  int64_t ldz;        // row pitch of Z / gZ in elements (>= U*V)
  float cg[kMaxD * kMaxD * kMaxD];  // C[i][j][k], row-major, already scaled by the path normalisation
};

template <typename T> __device__ __forceinline__ float ldf(const T* p, int64_t i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return __ldg(p + i); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

// shared: xs1[d1*U], xs2[d2*V], T[d3*d1*V], S[d3*d2*U]
template <typename TX>
__device__ __forceinline__ void load_sample(const FctpParams& p, int64_t z, float* xs1, float* xs2) {
  const TX* r1 = reinterpret_cast<const TX*>(p.x1) + z * p.ld1 + p.off1;
  const TX* r2 = reinterpret_cast<const TX*>(p.x2) + z * p.ld2 + p.off2;
  for (int t = threadIdx.x; t < p.d1 * p.U; t += blockDim.x) xs1[t] = ldf<TX>(r1, t);
  for (int t = threadIdx.x; t < p.d2 * p.V; t += blockDim.x) xs2[t] = ldf<TX>(r2, t);
}

__device__ __forceinline__ void contract_T(const FctpParams& p, const float* xs2, float* T) {
  // T[(k*d1 + i)*V + v] = sum_j C[i,j,k] x2[j,v]
  for (int t = threadIdx.x; t < p.d3 * p.d1 * p.V; t += blockDim.x) {
    const int v = t % p.V, ki = t / p.V, i = ki % p.d1, k = ki / p.d1;
    float acc = 0.f;
    for (int j = 0; j < p.d2; ++j) acc = fmaf(p.cg[(i * p.d2 + j) * p.d3 + k], xs2[j * p.V + v], acc);
    T[t] = acc;
  }
}

__device__ __forceinline__ void contract_S(const FctpParams& p, const float* xs1, float* S) {
  // S[(k*d2 + j)*U + u] = sum_i C[i,j,k] x1[i,u]
  for (int t = threadIdx.x; t < p.d3 * p.d2 * p.U; t += blockDim.x) {
    const int u = t % p.U, kj = t / p.U, j = kj % p.d2, k = kj / p.d2;
    float acc = 0.f;
    for (int i = 0; i < p.d1; ++i) acc = fmaf(p.cg[(i * p.d2 + j) * p.d3 + k], xs1[i * p.U + u], acc);
    S[t] = acc;
  }
}

__device__ __forceinline__ void store_pair(__nv_bfloat16* dst, float a0, float a1) {
  *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a0, a1);
}
__device__ __forceinline__ void store_pair(float* dst, float a0, float a1) { *reinterpret_cast<float2*>(dst) = make_float2(a0, a1); }

template <typename TX, typename TZ>
__global__ void __launch_bounds__(kThreadsF) fctp_build_z_kernel(const __grid_constant__ FctpParams p) {
  extern __shared__ __align__(16) float sm[];
  float* xs1 = sm;
  float* xs2 = xs1 + ((p.d1 * p.U + 1) & ~1);   // T below is read in pairs: keep it on an 8-byte boundary (V is even)
  float* T = xs2 + p.d2 * p.V;
  TZ* Z = reinterpret_cast<TZ*>(p.z);
  for (int64_t z = blockIdx.x; z < p.batch; z += gridDim.x) {
    __syncthreads();
    load_sample<TX>(p, z, xs1, xs2);
    __syncthreads();
    contract_T(p, xs2, T);
    __syncthreads();
    // a thread owns one pair of v (its T values stay in registers) and strides over u; the
    // threads of a warp share u, so x1 is read as a broadcast and Z rows are written contiguously
    const int vpairs = p.V / 2;
    const int ugroups = blockDim.x / vpairs;
    const int vp = threadIdx.x % vpairs, ug = threadIdx.x / vpairs;
    if (ug < ugroups) {
      for (int k = 0; k < p.d3; ++k) {
        float2 tt[kMaxD];
#pragma unroll
        for (int i = 0; i < kMaxD; ++i)
          tt[i] = i < p.d1 ? *reinterpret_cast<const float2*>(T + (k * p.d1 + i) * p.V + 2 * vp) : make_float2(0.f, 0.f);
        TZ* zrow = Z + (z * p.d3 + k) * p.ldz + 2 * vp;
        for (int u = ug; u < p.U; u += ugroups) {
          float a0 = 0.f, a1 = 0.f;
#pragma unroll
          for (int i = 0; i < kMaxD; ++i) {
            if (i < p.d1) {
              const float xi = xs1[i * p.U + u];
              a0 = fmaf(tt[i].x, xi, a0);
              a1 = fmaf(tt[i].y, xi, a1);
            }
          }
          store_pair(zrow + u * p.V, a0, a1);
        }
      }
    }
  }
}

template <typename TX, typename TZ>
__global__ void __launch_bounds__(kThreadsF) fctp_consume_gz_kernel(const __grid_constant__ FctpParams p) {
  extern __shared__ float sm[];
  float* xs1 = sm;
  float* xs2 = xs1 + p.d1 * p.U;
  float* T = xs2 + p.d2 * p.V;
  float* S = T + p.d3 * p.d1 * p.V;
  float* g2 = S + p.d3 * p.d2 * p.U;   // [d2*V] block-level accumulator of gx2
  float* g1 = g2 + p.d2 * p.V;         // [d1*U] block-level accumulator of gx1
  const TZ* GZ = reinterpret_cast<const TZ*>(p.z);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  // a thread owns one v for the whole sample and walks a share of the u range: its x2-gradient partials stay
  // in registers over u (no shared atomics in the inner loop), the x1-gradient partials of a row u are summed
  // over v with warp shuffles
  const int vwarps = (p.V + 31) / 32;                          // warps that together cover the v axis
  const int ugroups = nwarps / vwarps > 0 ? nwarps / vwarps : 1;
  const int v = (warp % vwarps) * 32 + lane;
  const int ug = warp / vwarps;
  const bool v_ok = v < p.V && ug < ugroups;
  for (int64_t z = blockIdx.x; z < p.batch; z += gridDim.x) {
    __syncthreads();
    load_sample<TX>(p, z, xs1, xs2);
    for (int t = threadIdx.x; t < p.d2 * p.V; t += blockDim.x) g2[t] = 0.f;
    for (int t = threadIdx.x; t < p.d1 * p.U; t += blockDim.x) g1[t] = 0.f;
    __syncthreads();
    contract_T(p, xs2, T);
    contract_S(p, xs1, S);
    __syncthreads();
    float a2[kMaxD];
#pragma unroll
    for (int j = 0; j < kMaxD; ++j) a2[j] = 0.f;
    if (ug < ugroups) {
      for (int u = ug; u < p.U; u += ugroups) {
        float a1[kMaxD];
#pragma unroll
        for (int i = 0; i < kMaxD; ++i) a1[i] = 0.f;
        if (v_ok) {
          for (int k = 0; k < p.d3; ++k) {
            const float g = ldf<TZ>(GZ, (z * p.d3 + k) * p.ldz + u * p.V + v);
#pragma unroll
            for (int i = 0; i < kMaxD; ++i)
              if (i < p.d1) a1[i] = fmaf(g, T[(k * p.d1 + i) * p.V + v], a1[i]);
#pragma unroll
            for (int j = 0; j < kMaxD; ++j)
              if (j < p.d2) a2[j] = fmaf(g, S[(k * p.d2 + j) * p.U + u], a2[j]);
          }
        }
#pragma unroll
        for (int i = 0; i < kMaxD; ++i) {
          if (i < p.d1) {
            const float tot = cueq::warp_sum(a1[i]);
            if (lane == 0) {
              if (vwarps == 1) g1[i * p.U + u] = tot; else atomicAdd(g1 + i * p.U + u, tot);
            }
          }
        }
      }
      if (v_ok) {
#pragma unroll
        for (int j = 0; j < kMaxD; ++j)
          if (j < p.d2) atomicAdd(g2 + j * p.V + v, a2[j]);
      }
    }
    __syncthreads();
    if (p.gx1)
      for (int t = threadIdx.x; t < p.d1 * p.U; t += blockDim.x) p.gx1[z * p.ld1 + p.off1 + t] += g1[t];
    if (p.gx2)
      for (int t = threadIdx.x; t < p.d2 * p.V; t += blockDim.x) p.gx2[z * p.ld2 + p.off2 + t] += g2[t];
  }
}

// ---- float32 operands, irrep dimensions known at compile time -------------------------------------
//
// The two kernels above keep every loop bound in a register: their inner loops carry predicated-off
// multiply-adds for the unused part of the 7-wide unrolling, load one 4-byte element of Z / gZ per
// thread at a time and spend as many instructions on index arithmetic as on the contraction.  For
// the float32 route (x and Z both float32, V a power of two) the kernels below are instantiated per
// (d1, d2, d3): a thread owns 4 x 4 tiles of (u, v) (16-byte accesses to Z / gZ, 128-bit reads of the
// per-sample tables for 16 multiply-adds each), groups of V/4 threads share a u tile, and the sums
// over v are taken by shuffles inside such a group.
__host__ __device__ constexpr int pad4(int n) { return (n + 3) & ~3; }

template <int D1, int D2, int D3>
struct FastSmem {
  // float offsets inside dynamic shared memory; every block starts on a 16-byte boundary
  __host__ __device__ static int xs1(int, int) { return 0; }
  __host__ __device__ static int xs2(int U, int) { return pad4(D1 * U); }
  __host__ __device__ static int cg(int U, int V) { return xs2(U, V) + pad4(D2 * V); }
  __host__ __device__ static int T(int U, int V) { return cg(U, V) + pad4(D1 * D2 * D3); }
  __host__ __device__ static int S(int U, int V) { return T(U, V) + D3 * D1 * V; }          // V % 4 == 0
  __host__ __device__ static int g2(int U, int V) { return S(U, V) + pad4(D3 * D2 * U); }
  __host__ __device__ static int g1(int U, int V) { return g2(U, V) + D2 * V; }
  __host__ __device__ static int build_floats(int U, int V) { return S(U, V); }
  __host__ __device__ static int consume_floats(int U, int V) { return g1(U, V) + pad4(D1 * U); }
};

template <int D1, int D2, int D3>
__device__ __forceinline__ void fast_prologue(const FctpParams& p, int64_t z, float* sm, int vshift, bool with_S) {
  using L = FastSmem<D1, D2, D3>;
  float* xs1 = sm + L::xs1(p.U, p.V);
  float* xs2 = sm + L::xs2(p.U, p.V);
  const float* cg = sm + L::cg(p.U, p.V);
  load_sample<float>(p, z, xs1, xs2);
  __syncthreads();
  float* T = sm + L::T(p.U, p.V);
  for (int t = threadIdx.x; t < D3 * D1 * p.V; t += blockDim.x) {
    const int v = t & (p.V - 1), ki = t >> vshift, i = ki % D1, k = ki / D1;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < D2; ++j) acc = fmaf(cg[(i * D2 + j) * D3 + k], xs2[j * p.V + v], acc);
    T[t] = acc;
  }
  if (with_S) {
    float* S = sm + L::S(p.U, p.V);
    for (int t = threadIdx.x; t < D3 * D2 * p.U; t += blockDim.x) {
      const int u = t % p.U, kj = t / p.U, j = kj % D2, k = kj / D2;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < D1; ++i) acc = fmaf(cg[(i * D2 + j) * D3 + k], xs1[i * p.U + u], acc);
      S[t] = acc;
    }
  }
}

template <int D1, int D2, int D3>
__global__ void __launch_bounds__(kThreadsFast) fctp_build_z_f32_kernel(const __grid_constant__ FctpParams p) {
  using L = FastSmem<D1, D2, D3>;
  extern __shared__ __align__(16) float sm[];
  // a thread owns a 4 x 4 tile of (u, v): per k it reads d1 128-bit rows of T (its four v, kept over all its u
  // tiles) and per tile d1 128-bit pieces of x1 (its four u) for 16 d1 multiply-adds and four 16-byte stores
  const int vshift = __ffs(p.V) - 1, gshift = vshift - 2;     // V = 1 << vshift; a u tile is shared by V/4 threads
  const int vq = threadIdx.x & ((1 << gshift) - 1), ug = threadIdx.x >> gshift, ugroups = kThreadsFast >> gshift;
  const int utiles = p.U >> 2;
  for (int t = threadIdx.x; t < D1 * D2 * D3; t += blockDim.x) sm[L::cg(p.U, p.V) + t] = p.cg[t];
  const float* xs1 = sm + L::xs1(p.U, p.V);
  const float* T = sm + L::T(p.U, p.V);
  float* Z = reinterpret_cast<float*>(p.z);
  for (int64_t z = blockIdx.x; z < p.batch; z += gridDim.x) {
    __syncthreads();
    fast_prologue<D1, D2, D3>(p, z, sm, vshift, false);
    __syncthreads();
#pragma unroll 1
    for (int k = 0; k < D3; ++k) {
      float4 tt[D1];
#pragma unroll
      for (int i = 0; i < D1; ++i) tt[i] = *reinterpret_cast<const float4*>(T + (k * D1 + i) * p.V + 4 * vq);
      float* zrow = Z + (z * D3 + k) * p.ldz + 4 * vq;
      for (int uq = ug; uq < utiles; uq += ugroups) {
        float4 a[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) a[r] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < D1; ++i) {
          const float4 x4 = *reinterpret_cast<const float4*>(xs1 + i * p.U + 4 * uq);
          const float xr[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            a[r].x = fmaf(tt[i].x, xr[r], a[r].x); a[r].y = fmaf(tt[i].y, xr[r], a[r].y);
            a[r].z = fmaf(tt[i].z, xr[r], a[r].z); a[r].w = fmaf(tt[i].w, xr[r], a[r].w);
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) *reinterpret_cast<float4*>(zrow + (int64_t)(4 * uq + r) * p.V) = a[r];
      }
    }
  }
}

template <int D1, int D2, int D3>
__global__ void __launch_bounds__(kThreadsFast, 8) fctp_consume_gz_f32_kernel(const __grid_constant__ FctpParams p) {
  using L = FastSmem<D1, D2, D3>;
  extern __shared__ __align__(16) float sm[];
  // the same 4 x 4 tiles: per k four 16-byte loads of gZ, d1 128-bit rows of T and d2 128-bit pieces of S feed
  // 16 (d1 + d2) multiply-adds; the x1-gradient partials are summed over v by shuffles in a group of V/4 threads
  const int vshift = __ffs(p.V) - 1, gshift = vshift - 2;
  const int gsize = 1 << gshift;
  const int vq = threadIdx.x & (gsize - 1), ug = threadIdx.x >> gshift, ugroups = kThreadsFast >> gshift;
  const int utiles = p.U >> 2;
  for (int t = threadIdx.x; t < D1 * D2 * D3; t += blockDim.x) sm[L::cg(p.U, p.V) + t] = p.cg[t];
  const float* T = sm + L::T(p.U, p.V);
  const float* S = sm + L::S(p.U, p.V);
  float* g2 = sm + L::g2(p.U, p.V);
  float* g1 = sm + L::g1(p.U, p.V);
  const float* GZ = reinterpret_cast<const float*>(p.z);
  for (int64_t z = blockIdx.x; z < p.batch; z += gridDim.x) {
    __syncthreads();
    for (int t = threadIdx.x; t < D2 * p.V; t += blockDim.x) g2[t] = 0.f;
    fast_prologue<D1, D2, D3>(p, z, sm, vshift, true);
    __syncthreads();
    float a2[D2][4];
#pragma unroll
    for (int j = 0; j < D2; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) a2[j][c] = 0.f;
    // every thread makes the same number of trips, so the shuffles below always see the full warp
    for (int q0 = 0; q0 < utiles; q0 += ugroups) {
      const int uq = q0 + ug;
      const bool ok = uq < utiles;
      const int us = ok ? 4 * uq : 0;
      float a1[D1][4];
#pragma unroll
      for (int i = 0; i < D1; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r) a1[i][r] = 0.f;
#pragma unroll
      for (int k = 0; k < D3; ++k) {
        float4 g[4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
          g[r] = ok ? __ldcs(reinterpret_cast<const float4*>(GZ + (z * D3 + k) * p.ldz + (int64_t)(us + r) * p.V + 4 * vq))
                    : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < D1; ++i) {
          const float4 t4 = *reinterpret_cast<const float4*>(T + (k * D1 + i) * p.V + 4 * vq);
#pragma unroll
          for (int r = 0; r < 4; ++r)
            a1[i][r] = fmaf(g[r].x, t4.x, fmaf(g[r].y, t4.y, fmaf(g[r].z, t4.z, fmaf(g[r].w, t4.w, a1[i][r]))));
        }
#pragma unroll
        for (int j = 0; j < D2; ++j) {
          const float4 s4 = *reinterpret_cast<const float4*>(S + (k * D2 + j) * p.U + us);
          const float sr[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            a2[j][0] = fmaf(g[r].x, sr[r], a2[j][0]); a2[j][1] = fmaf(g[r].y, sr[r], a2[j][1]);
            a2[j][2] = fmaf(g[r].z, sr[r], a2[j][2]); a2[j][3] = fmaf(g[r].w, sr[r], a2[j][3]);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < D1; ++i) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float tot = a1[i][r];
          for (int o = gsize >> 1; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
          a1[i][r] = tot;
        }
        if (ok && vq == 0) *reinterpret_cast<float4*>(g1 + i * p.U + us) = make_float4(a1[i][0], a1[i][1], a1[i][2], a1[i][3]);   // one group per u tile
      }
    }
#pragma unroll
    for (int j = 0; j < D2; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) atomicAdd(g2 + j * p.V + 4 * vq + c, a2[j][c]);
    __syncthreads();
    if (p.gx1)
      for (int t = threadIdx.x; t < D1 * p.U; t += blockDim.x) p.gx1[z * p.ld1 + p.off1 + t] += g1[t];
    if (p.gx2)
      for (int t = threadIdx.x; t < D2 * p.V; t += blockDim.x) p.gx2[z * p.ld2 + p.off2 + t] += g2[t];
  }
}

using FastKernel = void (*)(const FctpParams);

template <int D1, int D2, int D3>
void fast_pick(FastKernel& build, FastKernel& consume, int U, int V, size_t& smem_build, size_t& smem_consume) {
  build = fctp_build_z_f32_kernel<D1, D2, D3>;
  consume = fctp_consume_gz_f32_kernel<D1, D2, D3>;
  smem_build = sizeof(float) * FastSmem<D1, D2, D3>::build_floats(U, V);
  smem_consume = sizeof(float) * FastSmem<D1, D2, D3>::consume_floats(U, V);
}

template <int D1, int D2>
bool fast_pick3(int d3, FastKernel& b, FastKernel& c, int U, int V, size_t& sb, size_t& sc) {
  switch (d3) {
    case 1: fast_pick<D1, D2, 1>(b, c, U, V, sb, sc); return true;
    case 3: fast_pick<D1, D2, 3>(b, c, U, V, sb, sc); return true;
    case 5: fast_pick<D1, D2, 5>(b, c, U, V, sb, sc); return true;
    case 7: fast_pick<D1, D2, 7>(b, c, U, V, sb, sc); return true;
  }
  return false;
}

template <int D1>
bool fast_pick2(int d2, int d3, FastKernel& b, FastKernel& c, int U, int V, size_t& sb, size_t& sc) {
  switch (d2) {
    case 1: return fast_pick3<D1, 1>(d3, b, c, U, V, sb, sc);
    case 3: return fast_pick3<D1, 3>(d3, b, c, U, V, sb, sc);
    case 5: return fast_pick3<D1, 5>(d3, b, c, U, V, sb, sc);
    case 7: return fast_pick3<D1, 7>(d3, b, c, U, V, sb, sc);
  }
  return false;
}

// The compile-time kernels apply to float32 x and Z, odd irrep dimensions up to 7, U a multiple of 4, V a power
// of two in 16..128 and 16-byte aligned rows of Z; everything else takes the generic kernels.
bool fast_lookup(const cueq_fctp_args* a, const FctpParams& p, FastKernel& b, FastKernel& c, size_t& sb, size_t& sc) {
  if (a->x_dtype != CUEQ_F32 || a->z_dtype != CUEQ_F32) return false;
  if (p.V < 16 || p.V > 128 || (p.V & (p.V - 1)) || (p.U & 3)) return false;
  if ((p.ldz & 3) || (reinterpret_cast<uintptr_t>(p.z) & 15)) return false;
  switch (p.d1) {
    case 1: return fast_pick2<1>(p.d2, p.d3, b, c, p.U, p.V, sb, sc);
    case 3: return fast_pick2<3>(p.d2, p.d3, b, c, p.U, p.V, sb, sc);
    case 5: return fast_pick2<5>(p.d2, p.d3, b, c, p.U, p.V, sb, sc);
    case 7: return fast_pick2<7>(p.d2, p.d3, b, c, p.U, p.V, sb, sc);
  }
  return false;
}

int launch_fast(FastKernel k, size_t smem, const FctpParams& p, cudaStream_t st) {
  if (smem > 48 * 1024) CUEQ_CUDA_OK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  k<<<(unsigned)(p.batch < 148 * 64 ? p.batch : 148 * 64), kThreadsFast, smem, st>>>(p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

int fill(const cueq_fctp_args* a, FctpParams& p) {
  if (!a) return cueq::fail("fctp: null arguments");
  if (a->d1 < 1 || a->d1 > kMaxD || a->d2 < 1 || a->d2 > kMaxD || a->d3 < 1 || a->d3 > kMaxD)
    return cueq::fail("fctp: irrep dimensions must be in 1..%d", kMaxD);
  if (a->U < 1 || a->V < 2 || (a->V & 1)) return cueq::fail("fctp: V must be even and U positive");
  if (!a->x1 || !a->x2 || !a->z || !a->cg) return cueq::fail("fctp: null tensor");
  if (a->batch < 0) return cueq::fail("fctp: negative batch");
  std::memset(&p, 0, sizeof(p));
  p.x1 = a->x1; p.x2 = a->x2; p.z = a->z; p.gx1 = (float*)a->gx1; p.gx2 = (float*)a->gx2;
  p.ld1 = a->ld1; p.ld2 = a->ld2; p.batch = a->batch; p.off1 = a->off1; p.off2 = a->off2;
  p.d1 = a->d1; p.d2 = a->d2; p.d3 = a->d3; p.U = a->U; p.V = a->V; p.z_is_bf16 = a->z_dtype == CUEQ_BF16;
  p.ldz = a->ldz > 0 ? a->ldz : (int64_t)a->U * a->V;
  if (p.ldz < (int64_t)a->U * a->V || (p.ldz & 1)) return cueq::fail("fctp: the row pitch of Z must be even and at least U*V");
  for (int t = 0; t < a->d1 * a->d2 * a->d3; ++t) p.cg[t] = a->cg[t];
  return 0;
}

unsigned grid_for(int64_t batch) { return (unsigned)(batch < 148 * 16 ? (batch < 1 ? 1 : batch) : 148 * 16); }

}  // namespace

extern "C" int cueq_b200_fctp_build_z(const cueq_fctp_args* a, void* stream) {
  FctpParams p;
  if (int rc = fill(a, p)) return rc;
  if (p.batch == 0) return 0;
  if (a->x_dtype != CUEQ_F32 && a->x_dtype != CUEQ_BF16) return cueq::fail("fctp: x must be float32 or bfloat16");
  const size_t smem = sizeof(float) * (((p.d1 * p.U + 1) & ~1) + p.d2 * p.V + p.d3 * p.d1 * p.V);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  {
    FastKernel fb, fc;
    size_t sb, sc;
    if (fast_lookup(a, p, fb, fc, sb, sc)) return launch_fast(fb, sb, p, st);
  }
  if (a->z_dtype != CUEQ_F32 && a->z_dtype != CUEQ_BF16) return cueq::fail("fctp: Z must be float32 or bfloat16");
  const bool xb = a->x_dtype == CUEQ_BF16, zb = a->z_dtype == CUEQ_BF16;
  if (!xb && !zb) fctp_build_z_kernel<float, float><<<grid_for(p.batch), kThreadsF, smem, st>>>(p);
  else if (!xb && zb) fctp_build_z_kernel<float, __nv_bfloat16><<<grid_for(p.batch), kThreadsF, smem, st>>>(p);
  else if (xb && !zb) fctp_build_z_kernel<__nv_bfloat16, float><<<grid_for(p.batch), kThreadsF, smem, st>>>(p);
  else fctp_build_z_kernel<__nv_bfloat16, __nv_bfloat16><<<grid_for(p.batch), kThreadsF, smem, st>>>(p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int cueq_b200_fctp_consume_gz(const cueq_fctp_args* a, void* stream) {
  FctpParams p;
  if (int rc = fill(a, p)) return rc;
  if (p.batch == 0) return 0;
  if (a->x_dtype != CUEQ_F32 && a->x_dtype != CUEQ_BF16) return cueq::fail("fctp: x must be float32 or bfloat16");
  if (a->z_dtype != CUEQ_F32 && a->z_dtype != CUEQ_BF16) return cueq::fail("fctp: gZ must be float32 or bfloat16");
  const size_t smem = sizeof(float) * (p.d1 * p.U + p.d2 * p.V + p.d3 * p.d1 * p.V + p.d3 * p.d2 * p.U + p.d2 * p.V + p.d1 * p.U);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  {
    FastKernel fb, fc;
    size_t sb, sc;
    if (fast_lookup(a, p, fb, fc, sb, sc)) return launch_fast(fc, sc, p, st);
  }
  const unsigned grid = grid_for(p.batch);
  const bool xb = a->x_dtype == CUEQ_BF16, zb = a->z_dtype == CUEQ_BF16;
  if (!xb && !zb) fctp_consume_gz_kernel<float, float><<<grid, kThreadsF, smem, st>>>(p);
  else if (!xb && zb) fctp_consume_gz_kernel<float, __nv_bfloat16><<<grid, kThreadsF, smem, st>>>(p);
  else if (xb && !zb) fctp_consume_gz_kernel<__nv_bfloat16, float><<<grid, kThreadsF, smem, st>>>(p);
  else fctp_consume_gz_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreadsF, smem, st>>>(p);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

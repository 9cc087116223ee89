// Spherical harmonics of edge vectors, fused: normalisation and all requested degrees in one pass over the
// vectors, forward and backward to the vectors.
//
// The reference module (cuequivariance_torch/operations/spherical_harmonics.py:76-93) normalises the
// vectors with a torch op and then evaluates the polynomial of
// cue.descriptors.spherical_harmonics (spherical_harmonics_.py:23-52) through the segmented-polynomial
// executor: the [E, 3] vectors, the normalised copy and the [E, sum(2l+1)] result each make their own
// trip through memory, and so do the cotangents on the way back.  Here one thread owns one vector: it
// reads 3 numbers and writes sum(2l+1) (forward), or reads 3 + sum(2l+1) and writes 3 (backward:
// g_vec = P (J^T g) / |v| with P = 1 - n n^T the projector that differentiating the normalisation gives).
// Memory-bound by construction: 12 + 4 sum(2l+1) bytes per edge each way in float32.
#include "common.cuh"
#include "generated/sh_poly.cuh"

namespace {

template <typename T>
__device__ __forceinline__ void eval_all(T x, T y, T z, unsigned mask, T* __restrict__ out) {
  int o = 0;
  if (mask & 1u) { sh_eval_l0(x, y, z, out + o); o += 1; }
  if (mask & 2u) { sh_eval_l1(x, y, z, out + o); o += 3; }
  if (mask & 4u) { sh_eval_l2(x, y, z, out + o); o += 5; }
  if (mask & 8u) { sh_eval_l3(x, y, z, out + o); o += 7; }
  if (mask & 16u) { sh_eval_l4(x, y, z, out + o); o += 9; }
}

template <typename T>
__device__ __forceinline__ void vjp_all(T x, T y, T z, unsigned mask, const T* __restrict__ g, T& gx, T& gy, T& gz) {
  int o = 0;
  if (mask & 1u) { sh_vjp_l0(x, y, z, g + o, gx, gy, gz); o += 1; }
  if (mask & 2u) { sh_vjp_l1(x, y, z, g + o, gx, gy, gz); o += 3; }
  if (mask & 4u) { sh_vjp_l2(x, y, z, g + o, gx, gy, gz); o += 5; }
  if (mask & 8u) { sh_vjp_l3(x, y, z, g + o, gx, gy, gz); o += 7; }
  if (mask & 16u) { sh_vjp_l4(x, y, z, g + o, gx, gy, gz); o += 9; }
}

constexpr int kMaxOut = 25;   // 1 + 3 + 5 + 7 + 9

template <typename T>
__device__ __forceinline__ T inv_norm(T x, T y, T z) {
  // torch.nn.functional.normalize: v / max(|v|, 1e-12)
  const T n = sqrt(x * x + y * y + z * z);
  return T(1) / (n > T(1e-12) ? n : T(1e-12));
}

template <typename T>
__global__ void __launch_bounds__(256) sh_forward_kernel(const T* __restrict__ vec, T* __restrict__ out, int64_t rows, int64_t ld_vec,
                                                         int64_t ld_out, unsigned mask, int width, int normalize) {
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x) {
    T x = vec[r * ld_vec], y = vec[r * ld_vec + 1], z = vec[r * ld_vec + 2];
    if (normalize) {
      const T s = inv_norm(x, y, z);
      x *= s; y *= s; z *= s;
    }
    T y_all[kMaxOut];
    eval_all(x, y, z, mask, y_all);
    T* dst = out + r * ld_out;
#pragma unroll
    for (int k = 0; k < kMaxOut; ++k)
      if (k < width) dst[k] = y_all[k];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) sh_backward_kernel(const T* __restrict__ vec, const T* __restrict__ gout, T* __restrict__ gvec,
                                                          int64_t rows, int64_t ld_vec, int64_t ld_g, int64_t ld_gvec, unsigned mask,
                                                          int width, int normalize) {
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x) {
    T x = vec[r * ld_vec], y = vec[r * ld_vec + 1], z = vec[r * ld_vec + 2];
    T s = T(1);
    if (normalize) {
      s = inv_norm(x, y, z);
      x *= s; y *= s; z *= s;
    }
    T g[kMaxOut];
    const T* src = gout + r * ld_g;
#pragma unroll
    for (int k = 0; k < kMaxOut; ++k) g[k] = k < width ? src[k] : T(0);
    T gx = T(0), gy = T(0), gz = T(0);
    vjp_all(x, y, z, mask, g, gx, gy, gz);
    if (normalize) {   // d(v/|v|) = (1 - n n^T) dv / |v|
      const T dot = gx * x + gy * y + gz * z;
      gx = (gx - dot * x) * s; gy = (gy - dot * y) * s; gz = (gz - dot * z) * s;
    }
    T* dst = gvec + r * ld_gvec;
    dst[0] = gx; dst[1] = gy; dst[2] = gz;
  }
}

int width_of(unsigned mask) {
  int w = 0;
  for (int l = 0; l <= kShLmax; ++l)
    if (mask >> l & 1u) w += 2 * l + 1;
  return w;
}

int check(const cueq_sh_args* a) {
  if (!a) return cueq::fail("spherical harmonics: null arguments");
  if (a->rows < 0) return cueq::fail("spherical harmonics: negative row count");
  if (a->ls_mask == 0 || (a->ls_mask >> (kShLmax + 1))) return cueq::fail("spherical harmonics: degrees must be within 0..%d", kShLmax);
  if (a->dtype != CUEQ_F32 && a->dtype != CUEQ_F64) return cueq::fail("spherical harmonics: float32 or float64 only");
  if (!a->vec || !a->y) return cueq::fail("spherical harmonics: null tensor");
  return 0;
}

unsigned grid_for(int64_t rows) {
  const int64_t want = (rows + 255) / 256;
  return (unsigned)(want < 1 ? 1 : (want < 148 * 16 ? want : 148 * 16));
}

}  // namespace

extern "C" int cueq_b200_sh_width(uint32_t ls_mask) { return width_of(ls_mask); }

extern "C" int cueq_b200_sh_forward(const cueq_sh_args* a, void* stream) {
  if (int rc = check(a)) return rc;
  if (a->rows == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int w = width_of(a->ls_mask);
  if (a->dtype == CUEQ_F32)
    sh_forward_kernel<float><<<grid_for(a->rows), 256, 0, st>>>((const float*)a->vec, (float*)a->y, a->rows, a->ld_vec, a->ld_y, a->ls_mask, w, a->normalize);
  else
    sh_forward_kernel<double><<<grid_for(a->rows), 256, 0, st>>>((const double*)a->vec, (double*)a->y, a->rows, a->ld_vec, a->ld_y, a->ls_mask, w, a->normalize);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int cueq_b200_sh_backward(const cueq_sh_args* a, void* stream) {
  if (int rc = check(a)) return rc;
  if (!a->gvec) return cueq::fail("spherical harmonics backward: null gradient tensor");
  if (a->rows == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int w = width_of(a->ls_mask);
  if (a->dtype == CUEQ_F32)
    sh_backward_kernel<float><<<grid_for(a->rows), 256, 0, st>>>((const float*)a->vec, (const float*)a->y, (float*)a->gvec, a->rows, a->ld_vec, a->ld_y,
                                                                   a->ld_gvec, a->ls_mask, w, a->normalize);
  else
    sh_backward_kernel<double><<<grid_for(a->rows), 256, 0, st>>>((const double*)a->vec, (const double*)a->y, (double*)a->gvec, a->rows, a->ld_vec,
                                                                    a->ld_y, a->ld_gvec, a->ls_mask, w, a->normalize);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

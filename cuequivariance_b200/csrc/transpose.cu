// Per-row, per-block transposition between the mul_ir and ir_mul layouts.
//
// Takes the place of the reference's closed `segmented_transpose`
// (cuequivariance_torch/primitives/transpose.py:155-183): block b of every row is a [u, v]
// tile at `offset` and is written back as [v, u].  One CTA per row; the row is staged in
// shared memory so that both the global read and the global write are contiguous.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256) segmented_transpose_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                  int64_t rows, int dim,
                                                                  const int4* __restrict__ info, int num_blocks) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tile = reinterpret_cast<T*>(smem_raw);
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * dim;
    T* yr = y + r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) tile[i] = xr[i];
    __syncthreads();
    for (int b = 0; b < num_blocks; ++b) {
      const int4 d = __ldg(info + b);
      const int off = d.x, u = d.y, v = d.z;
      for (int e = threadIdx.x; e < u * v; e += blockDim.x) {
        const int j = e / u, i = e - j * u;  // destination [j, i] of a [v, u] tile
        yr[off + e] = tile[off + i * v + j];
      }
    }
    __syncthreads();
  }
}

template <typename T>
int launch(const void* x, void* y, int64_t rows, int64_t dim, const int32_t* info, int nb, cudaStream_t st) {
  const size_t smem = (size_t)dim * sizeof(T);
  if (smem > 200 * 1024) return cueq::fail("segmented_transpose: row of %lld elements does not fit shared memory", (long long)dim);
  if (smem > 48 * 1024) CUEQ_CUDA_OK(cudaFuncSetAttribute(segmented_transpose_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const unsigned grid = (unsigned)std::min<int64_t>(rows, 148 * 8);
  segmented_transpose_kernel<T><<<grid, 256, smem, st>>>(reinterpret_cast<const T*>(x), reinterpret_cast<T*>(y), rows, (int)dim,
                                                        reinterpret_cast<const int4*>(info), nb);
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace

extern "C" int cueq_b200_segmented_transpose(const void* x, void* y, int64_t rows, int64_t dim,
                                             const int32_t* info_dev, int32_t num_blocks, int32_t dtype,
                                             void* stream) {
  if (rows == 0 || dim == 0) return 0;
  if (!x || !y || !info_dev) return cueq::fail("segmented_transpose: null argument");
  if (x == y) return cueq::fail("segmented_transpose: x and y must not alias");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case CUEQ_F32: return launch<float>(x, y, rows, dim, info_dev, num_blocks, st);
    case CUEQ_F64: return launch<double>(x, y, rows, dim, info_dev, num_blocks, st);
    case CUEQ_BF16:
    case CUEQ_F16: return launch<uint16_t>(x, y, rows, dim, info_dev, num_blocks, st);
    default: return cueq::fail("segmented_transpose: invalid dtype %d", dtype);
  }
}

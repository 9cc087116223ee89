// Straight-line ("static") kernels for polynomials known at build time.
//
// Same contract as the generic uniform-1d executor (u1d_generic.cu; reference call site
// cuequivariance_torch/primitives/segmented_polynomial_uniform_1d.py:294-316), float32 only:
// one thread evaluates one (row, channel) pair, but instead of walking a path table it runs
// the code generated for that polynomial (generated/u1d_static.cuh): every operand segment is
// loaded once into a register, every path is a few multiplies.  Used for the symmetric
// contraction, whose ~2,000 paths make the table-driven kernel instruction- and L1-bound.
#include <cstring>

#include "common.cuh"
#include "generated/u1d_static.cuh"

namespace {

constexpr int kMaxBuf = 8;

struct StaticBuf {
  void* ptr;
  const void* index;
  int32_t mode;
  int32_t index_is_64;
  int32_t row_size;  // elements per row
  int32_t vec;       // 1: segments have a channel axis, 0: scalar segments
};

struct StaticParams {
  StaticBuf buf[kMaxBuf];
  int64_t batch;
  int32_t extent;
};

template <class K>
__global__ void __launch_bounds__(128) u1d_static_kernel(const __grid_constant__ StaticParams P) {
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= P.batch * P.extent) return;
  const int64_t z = gid / P.extent;
  const int u = (int)(gid - z * P.extent);
  const int X = P.extent;
  const float* in_base[K::NUM_INPUTS];
  int in_stride[K::NUM_INPUTS];
#pragma unroll
  for (int b = 0; b < K::NUM_INPUTS; ++b) {
    const StaticBuf& s = P.buf[b];
    const int64_t row = s.mode == CUEQ_SHARED ? 0 : s.mode == CUEQ_BATCHED ? z : cueq::load_index(s.index, s.index_is_64, z);
    in_base[b] = reinterpret_cast<const float*>(s.ptr) + row * s.row_size + (s.vec ? u : 0);
    in_stride[b] = s.vec ? X : 1;
  }
  float* out_base[K::NUM_OUTPUTS];
  int out_stride[K::NUM_OUTPUTS];
  bool out_atomic[K::NUM_OUTPUTS];
#pragma unroll
  for (int j = 0; j < K::NUM_OUTPUTS; ++j) {
    const StaticBuf& s = P.buf[K::NUM_INPUTS + j];
    const int64_t row = s.mode == CUEQ_SHARED ? 0 : s.mode == CUEQ_BATCHED ? z : cueq::load_index(s.index, s.index_is_64, z);
    out_base[j] = reinterpret_cast<float*>(s.ptr) + row * s.row_size + (s.vec ? u : 0);
    out_stride[j] = s.vec ? X : 1;
    out_atomic[j] = s.mode != CUEQ_BATCHED || (!s.vec && X > 1);
  }
  auto in = [&](int b, int s) -> float { return __ldg(in_base[b] + s * in_stride[b]); };
  auto out = [&](int j, int s, float v) {
    float* p = out_base[j] + s * out_stride[j];
    if (out_atomic[j]) atomicAdd(p, v); else *p = v;
  };
  K::run(in, out);
}

struct StaticEntry {
  const char* digest;
  const char* name;
  int num_inputs, num_outputs;
  void (*launch)(const StaticParams&, unsigned, cudaStream_t);
};

template <class K>
void launch_t(const StaticParams& P, unsigned grid, cudaStream_t st) { u1d_static_kernel<K><<<grid, 128, 0, st>>>(P); }

#define U1D_ENTRY(K) {K::digest(), K::name(), K::NUM_INPUTS, K::NUM_OUTPUTS, &launch_t<K>},
const StaticEntry kStatic[] = {U1D_STATIC_FOR_EACH(U1D_ENTRY)};
constexpr int kNumStatic = sizeof(kStatic) / sizeof(kStatic[0]);

}  // namespace

extern "C" int cueq_b200_u1d_static_find(const char* digest) {
  if (!digest) return -1;
  for (int i = 0; i < kNumStatic; ++i)
    if (std::strcmp(kStatic[i].digest, digest) == 0) return i;
  return -1;
}

extern "C" const char* cueq_b200_u1d_static_name(int id) { return (id >= 0 && id < kNumStatic) ? kStatic[id].name : nullptr; }

extern "C" int cueq_b200_u1d_static_launch(int id, int64_t batch, int32_t extent, const cueq_buffer* buffers,
                                           const int32_t* buffer_dim, const int32_t* buffer_num_segments, int32_t num_buffers,
                                           void* stream) {
  if (id < 0 || id >= kNumStatic) return cueq::fail("u1d_static: kernel id %d out of range", id);
  const StaticEntry& e = kStatic[id];
  if (num_buffers != e.num_inputs + e.num_outputs) return cueq::fail("u1d_static: %s takes %d buffers, got %d", e.name, e.num_inputs + e.num_outputs, num_buffers);
  if (num_buffers > kMaxBuf) return cueq::fail("u1d_static: too many buffers");
  if (!buffers || !buffer_dim || !buffer_num_segments) return cueq::fail("u1d_static: null argument");
  if (batch < 0 || extent < 1) return cueq::fail("u1d_static: invalid batch or extent");
  StaticParams P;
  std::memset(&P, 0, sizeof(P));
  for (int b = 0; b < num_buffers; ++b) {
    const cueq_buffer& s = buffers[b];
    if (s.dtype != CUEQ_F32) return cueq::fail("u1d_static: buffer %d is not float32", b);
    if (s.mode != CUEQ_SHARED && s.mode != CUEQ_BATCHED && s.mode != CUEQ_INDEXED) return cueq::fail("u1d_static: buffer %d has invalid mode", b);
    if (s.mode == CUEQ_BATCHED && s.rows != batch) return cueq::fail("u1d_static: batched buffer %d has %lld rows, batch is %lld", b, (long long)s.rows, (long long)batch);
    if (s.mode == CUEQ_SHARED && s.rows != 1) return cueq::fail("u1d_static: shared buffer %d must have one row", b);
    if (s.mode == CUEQ_INDEXED && !s.index && batch > 0) return cueq::fail("u1d_static: indexed buffer %d has no index", b);
    P.buf[b].ptr = s.ptr; P.buf[b].index = s.index; P.buf[b].mode = s.mode; P.buf[b].index_is_64 = s.index_is_64;
    P.buf[b].vec = buffer_dim[b];
    P.buf[b].row_size = buffer_num_segments[b] * (buffer_dim[b] ? extent : 1);
  }
  if (batch == 0) return 0;
  P.batch = batch;
  P.extent = extent;
  const int64_t grid = (batch * extent + 127) / 128;
  if (grid > 2147483647LL) return cueq::fail("u1d_static: batch too large for one launch");
  e.launch(P, (unsigned)grid, reinterpret_cast<cudaStream_t>(stream));
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

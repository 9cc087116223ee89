// Generic executor for polynomials with scalar coefficients and one uniform mode `u`.
//
// Takes the place of the reference's closed `uniform_1d` op (call site:
// cuequivariance_torch/primitives/segmented_polynomial_uniform_1d.py:294-316): for every batch
// row z, operation and path
//     out[row_out(z)][seg_out, u] += c * prod_k in_k[row_k(z)][seg_k, u]
// where each buffer is shared (one row), batched (row z) or indexed (row index[z]) and a
// buffer with scalar segments has no `u` axis (a scalar output of vector inputs is summed
// over u).
//
// This kernel is the table-driven path: any polynomial, any number of operands, modest
// speed.  One thread owns one (row z, channel u) pair and walks the path table, which is
// sorted by output segment so that the running sum of a segment stays in a register and is
// written once.  The table is read through the read-only path (every lane reads the same
// entry, so it is a broadcast served by L1).  Polynomials on the throughput-critical path have
// specialised kernels (cw_*.cu) and only fall back to this one for shapes those do not cover.
#include <algorithm>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"

namespace {

constexpr int kMaxOperands = CUEQ_MAX_OPERANDS;
constexpr int kMaxBuffers = CUEQ_MAX_BUFFERS;

// ---- device tables (one blob, 16-byte aligned pieces) ---------------------------------------
struct TableHeader {
  int32_t num_ops;
  int32_t extent;
  int32_t num_buffers;
  int32_t total_paths;
  int64_t ops_offset;     // OpEntry[num_ops]
  int64_t indices_offset; // uint16 [total_paths][8]
  int64_t coeff_offset;   // double [total_paths]
  int64_t pad;
};

struct OpEntry {
  int32_t num_operands;
  int32_t out_operand;
  int32_t num_paths;
  int32_t path_start;
  int32_t buffers[kMaxOperands];
};

struct BufferDev {
  void* ptr;
  const void* index;
  int64_t rows;
  int32_t mode;
  int32_t dtype;
  int32_t index_is_64;
  int32_t ndim;      // 0: scalar segments, 1: (u,) segments
  int32_t row_size;  // elements per row
  int32_t pad;
};

struct LaunchParams {
  BufferDev buf[kMaxBuffers];
  const char* tables;
  int64_t batch;
  int32_t extent;
  int32_t warp_uniform_rows;  // extent % 32 == 0: all lanes of a warp work on one row
};

template <typename M>
__device__ __forceinline__ void accumulate_out(const BufferDev& b, int64_t row, int seg, int u,
                                               int extent, M acc, bool reduce_u, bool warp_rows) {
  M* out = reinterpret_cast<M*>(b.ptr) + row * (int64_t)b.row_size;
  if (b.ndim == 1) {
    M* p = out + (int64_t)seg * extent + u;
    if (b.mode == CUEQ_BATCHED) *p += acc;  // this thread is the only writer of (row, seg, u)
    else atomicAdd(p, acc);
  } else {
    M* p = out + seg;
    if (reduce_u) {
      if (warp_rows) {
        acc = cueq::warp_sum(acc);
        if ((threadIdx.x & 31) == 0) atomicAdd(p, acc);
      } else {
        atomicAdd(p, acc);
      }
    } else {
      if (b.mode == CUEQ_BATCHED) *p += acc;
      else atomicAdd(p, acc);
    }
  }
}

template <typename M, bool UNIFORM_IO>
__global__ void __launch_bounds__(256) u1d_generic_kernel(const LaunchParams P) {
  const int extent = P.extent;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= P.batch * extent) return;
  const int64_t z = gid / extent;
  const int u = (int)(gid - z * extent);

  const TableHeader* H = reinterpret_cast<const TableHeader*>(P.tables);
  const OpEntry* ops = reinterpret_cast<const OpEntry*>(P.tables + H->ops_offset);
  const uint4* pidx = reinterpret_cast<const uint4*>(P.tables + H->indices_offset);
  const double* pcoef = reinterpret_cast<const double*>(P.tables + H->coeff_offset);
  const bool reduce_u = extent > 1;

  for (int o = 0; o < H->num_ops; ++o) {
    const OpEntry op = ops[o];
    const void* base[kMaxOperands];
    int dtype[kMaxOperands];
    int stride[kMaxOperands];  // element stride between segments
    int off[kMaxOperands];     // channel offset inside a segment
    bool has_vec_input = false;
#pragma unroll
    for (int k = 0; k < kMaxOperands; ++k) {
      base[k] = nullptr; dtype[k] = 0; stride[k] = 0; off[k] = 0;
      if (k < op.num_operands && k != op.out_operand) {
        const BufferDev& b = P.buf[op.buffers[k]];
        int64_t row = b.mode == CUEQ_SHARED ? 0
                    : b.mode == CUEQ_BATCHED ? z
                                             : cueq::load_index(b.index, b.index_is_64, z);
        const int esz = b.dtype == CUEQ_F64 ? 8 : b.dtype == CUEQ_F32 ? 4 : 2;
        base[k] = reinterpret_cast<const char*>(b.ptr) + row * (int64_t)b.row_size * esz;
        dtype[k] = b.dtype;
        stride[k] = b.ndim ? extent : 1;
        off[k] = b.ndim ? u : 0;
        has_vec_input |= (b.ndim != 0);
      }
    }
    const BufferDev& ob = P.buf[op.buffers[op.out_operand]];
    const int64_t orow = ob.mode == CUEQ_SHARED ? 0
                       : ob.mode == CUEQ_BATCHED ? z
                                                 : cueq::load_index(ob.index, ob.index_is_64, z);
    // an operation whose operands are all scalars is evaluated once per row (by the u == 0
    // thread) even when other operations of the polynomial spread over u
    const M lane_weight = (ob.ndim == 0 && !has_vec_input && u != 0) ? (M)0 : (M)1;
    int cur = -1;
    M acc = 0;
    for (int p = 0; p < op.num_paths; ++p) {
      const uint4 raw = __ldg(pidx + op.path_start + p);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      M prod = lane_weight * (M)__ldg(pcoef + op.path_start + p);
      int seg_out = 0;
#pragma unroll
      for (int k = 0; k < kMaxOperands; ++k) {
        if (k < op.num_operands) {
          const int s = (w[k >> 1] >> ((k & 1) * 16)) & 0xffff;
          if (k == op.out_operand) {
            seg_out = s;
          } else {
            const int64_t e = (int64_t)s * stride[k] + off[k];
            if (UNIFORM_IO) prod *= __ldg(reinterpret_cast<const M*>(base[k]) + e);
            else prod *= cueq::load_as<M>(base[k], dtype[k], e);
          }
        }
      }
      if (seg_out != cur) {
        if (cur >= 0) accumulate_out<M>(ob, orow, cur, u, extent, acc, reduce_u, P.warp_uniform_rows);
        cur = seg_out;
        acc = 0;
      }
      acc += prod;
    }
    if (cur >= 0) accumulate_out<M>(ob, orow, cur, u, extent, acc, reduce_u, P.warp_uniform_rows);
  }
}

}  // namespace

// ---- plan (host) ------------------------------------------------------------------------------
struct cueq_plan {
  int32_t extent = 1;
  int32_t num_inputs = 0, num_outputs = 0;
  int32_t math_dtype = CUEQ_F32;
  std::vector<int32_t> buffer_dim, buffer_nseg;
  std::vector<char> blob;
};

extern "C" int cueq_b200_u1d_plan_create(const cueq_u1d_desc* d, cueq_plan** out) {
  if (!d || !out) return cueq::fail("u1d_plan_create: null argument");
  const int nb = d->num_inputs + d->num_outputs;
  if (nb <= 0 || nb > kMaxBuffers) return cueq::fail("u1d_plan_create: %d buffers (max %d)", nb, kMaxBuffers);
  if (d->operand_extent < 1) return cueq::fail("u1d_plan_create: operand_extent must be >= 1");
  if (d->math_dtype != CUEQ_F32 && d->math_dtype != CUEQ_F64)
    return cueq::fail("u1d_plan_create: math_dtype must be float32 or float64");
  for (int b = 0; b < nb; ++b) {
    if (d->buffer_dim[b] != 0 && d->buffer_dim[b] != 1)
      return cueq::fail("u1d_plan_create: buffer %d has %d modes (0 or 1 supported)", b, d->buffer_dim[b]);
    if (d->buffer_num_segments[b] < 0 || d->buffer_num_segments[b] > 65535)
      return cueq::fail("u1d_plan_create: buffer %d has %d segments (max 65535)", b, d->buffer_num_segments[b]);
  }
  cueq_plan* plan = new (std::nothrow) cueq_plan();
  if (!plan) return cueq::fail("u1d_plan_create: out of host memory");
  plan->extent = d->operand_extent;
  plan->num_inputs = d->num_inputs;
  plan->num_outputs = d->num_outputs;
  plan->math_dtype = d->math_dtype;
  plan->buffer_dim.assign(d->buffer_dim, d->buffer_dim + nb);
  plan->buffer_nseg.assign(d->buffer_num_segments, d->buffer_num_segments + nb);

  int64_t total_paths = 0;
  for (int o = 0; o < d->num_operations; ++o) total_paths += d->num_paths[o];
  std::vector<OpEntry> ops(d->num_operations);
  std::vector<uint16_t> idx((size_t)total_paths * kMaxOperands, 0);
  std::vector<double> coef((size_t)total_paths, 0.0);

  int64_t op_cursor = 0, idx_cursor = 0, path_cursor = 0;
  for (int o = 0; o < d->num_operations; ++o) {
    const int n = d->num_operands[o];
    if (n < 1 || n > kMaxOperands) {
      delete plan;
      return cueq::fail("u1d_plan_create: operation %d has %d operands (max %d)", o, n, kMaxOperands);
    }
    OpEntry& e = ops[o];
    std::memset(&e, 0, sizeof(e));
    e.num_operands = n;
    e.out_operand = -1;
    for (int k = 0; k < n; ++k) {
      const int b = d->operations[op_cursor + k];
      if (b < 0 || b >= nb) { delete plan; return cueq::fail("u1d_plan_create: buffer id %d out of range", b); }
      e.buffers[k] = b;
      if (b >= d->num_inputs) {
        if (e.out_operand >= 0) { delete plan; return cueq::fail("u1d_plan_create: operation %d has two outputs", o); }
        e.out_operand = k;
      }
    }
    if (e.out_operand < 0) { delete plan; return cueq::fail("u1d_plan_create: operation %d has no output", o); }
    const int np = d->num_paths[o];
    e.num_paths = np;
    e.path_start = (int32_t)path_cursor;
    // stable sort of the paths by output segment
    std::vector<int> order(np);
    for (int p = 0; p < np; ++p) order[p] = p;
    const int32_t* pi = d->path_indices + idx_cursor;
    const int ko = e.out_operand;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return pi[a * n + ko] < pi[b * n + ko]; });
    for (int q = 0; q < np; ++q) {
      const int p = order[q];
      for (int k = 0; k < n; ++k) {
        const int s = pi[p * n + k];
        if (s < 0 || s >= d->buffer_num_segments[e.buffers[k]]) {
          delete plan;
          return cueq::fail("u1d_plan_create: operation %d path %d operand %d: segment %d out of range", o, p, k, s);
        }
        idx[(size_t)(path_cursor + q) * kMaxOperands + k] = (uint16_t)s;
      }
      coef[path_cursor + q] = d->path_coefficients[path_cursor + p];
    }
    op_cursor += n;
    idx_cursor += (int64_t)np * n;
    path_cursor += np;
  }

  auto align16 = [](int64_t x) { return (x + 15) & ~int64_t(15); };
  TableHeader h;
  std::memset(&h, 0, sizeof(h));
  h.num_ops = d->num_operations;
  h.extent = d->operand_extent;
  h.num_buffers = nb;
  h.total_paths = (int32_t)total_paths;
  h.ops_offset = align16(sizeof(TableHeader));
  h.indices_offset = align16(h.ops_offset + (int64_t)ops.size() * sizeof(OpEntry));
  h.coeff_offset = align16(h.indices_offset + (int64_t)idx.size() * sizeof(uint16_t));
  const int64_t total = align16(h.coeff_offset + (int64_t)coef.size() * sizeof(double)) + 16;
  plan->blob.assign((size_t)total, 0);
  std::memcpy(plan->blob.data(), &h, sizeof(h));
  if (!ops.empty()) std::memcpy(plan->blob.data() + h.ops_offset, ops.data(), ops.size() * sizeof(OpEntry));
  if (!idx.empty()) std::memcpy(plan->blob.data() + h.indices_offset, idx.data(), idx.size() * sizeof(uint16_t));
  if (!coef.empty()) std::memcpy(plan->blob.data() + h.coeff_offset, coef.data(), coef.size() * sizeof(double));
  *out = plan;
  return 0;
}

extern "C" void cueq_b200_plan_destroy(cueq_plan* plan) { delete plan; }

extern "C" size_t cueq_b200_plan_table_bytes(const cueq_plan* plan) { return plan ? plan->blob.size() : 0; }

extern "C" const void* cueq_b200_plan_table_data(const cueq_plan* plan) { return plan ? plan->blob.data() : nullptr; }

extern "C" int cueq_b200_u1d_launch(const cueq_plan* plan, const void* tables_dev, int64_t batch,
                                    const cueq_buffer* buffers, int32_t num_buffers, void* stream) {
  if (!plan || !tables_dev || !buffers) return cueq::fail("u1d_launch: null argument");
  const int nb = plan->num_inputs + plan->num_outputs;
  if (num_buffers != nb) return cueq::fail("u1d_launch: got %d buffers, the plan has %d", num_buffers, nb);
  if (batch < 0) return cueq::fail("u1d_launch: negative batch");
  if ((reinterpret_cast<uintptr_t>(tables_dev) & 15) != 0) return cueq::fail("u1d_launch: tables_dev must be 16-byte aligned");
  LaunchParams P;
  std::memset(&P, 0, sizeof(P));
  bool uniform_io = true;
  for (int b = 0; b < nb; ++b) {
    const cueq_buffer& s = buffers[b];
    BufferDev& t = P.buf[b];
    if (s.mode != CUEQ_SHARED && s.mode != CUEQ_BATCHED && s.mode != CUEQ_INDEXED)
      return cueq::fail("u1d_launch: buffer %d has invalid mode %d", b, s.mode);
    if (s.mode == CUEQ_SHARED && s.rows != 1) return cueq::fail("u1d_launch: shared buffer %d must have one row, has %lld", b, (long long)s.rows);
    if (s.mode == CUEQ_BATCHED && s.rows != batch)
      return cueq::fail("u1d_launch: batched buffer %d has %lld rows, batch is %lld", b, (long long)s.rows, (long long)batch);
    if (s.mode == CUEQ_INDEXED && !s.index && batch > 0) return cueq::fail("u1d_launch: indexed buffer %d has no index", b);
    if (s.dtype < CUEQ_F32 || s.dtype > CUEQ_F16) return cueq::fail("u1d_launch: buffer %d has invalid dtype %d", b, s.dtype);
    if (b >= plan->num_inputs && s.dtype != plan->math_dtype)
      return cueq::fail("u1d_launch: output buffer %d must have the math dtype", b);
    if (!s.ptr && s.rows > 0) return cueq::fail("u1d_launch: buffer %d is null", b);
    t.ptr = s.ptr;
    t.index = s.index;
    t.rows = s.rows;
    t.mode = s.mode;
    t.dtype = s.dtype;
    t.index_is_64 = s.index_is_64;
    t.ndim = plan->buffer_dim[b];
    t.row_size = plan->buffer_nseg[b] * (t.ndim ? plan->extent : 1);
    if (s.dtype != plan->math_dtype) uniform_io = false;
  }
  if (batch == 0) return 0;
  P.tables = reinterpret_cast<const char*>(tables_dev);
  P.batch = batch;
  P.extent = plan->extent;
  P.warp_uniform_rows = (plan->extent % 32 == 0) ? 1 : 0;
  const int64_t threads = batch * (int64_t)plan->extent;
  const int block = 256;
  const int64_t grid = (threads + block - 1) / block;
  if (grid > 2147483647LL) return cueq::fail("u1d_launch: batch too large for one launch");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (plan->math_dtype == CUEQ_F32) {
    if (uniform_io) u1d_generic_kernel<float, true><<<(unsigned)grid, block, 0, st>>>(P);
    else u1d_generic_kernel<float, false><<<(unsigned)grid, block, 0, st>>>(P);
  } else {
    if (uniform_io) u1d_generic_kernel<double, true><<<(unsigned)grid, block, 0, st>>>(P);
    else u1d_generic_kernel<double, false><<<(unsigned)grid, block, 0, st>>>(P);
  }
  CUEQ_CUDA_OK(cudaGetLastError());
  return 0;
}

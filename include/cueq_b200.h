/*
 * cueq_b200 - C ABI of the B200 (sm_100a) executor for segmented polynomials.
 *
 * This is the boundary a host binding (ctypes, cffi, pybind, ...) talks to.  It takes the
 * place of the closed native package the reference front-end calls into:
 *   torch.ops.cuequivariance.uniform_1d        (cuequivariance_torch/primitives/segmented_polynomial_uniform_1d.py:32-77, call at :294-316)
 *   cuequivariance_ops_torch.segmented_transpose (cuequivariance_torch/primitives/transpose.py:171-183)
 *   cuequivariance_ops_torch.FusedTensorProductOp4 (cuequivariance_torch/primitives/segmented_polynomial_fused_tp.py:51-72)
 *
 * Conventions
 *   - every function returns 0 on success, non-zero on error; the message of the last error of
 *     the calling thread is available from cueq_b200_last_error();
 *   - the library never allocates or frees device memory, never synchronises and never changes
 *     the current device: the caller passes inputs, zero-initialised outputs, the device copy of
 *     the plan tables and a stream (a cudaStream_t passed as void*), and all device pointers
 *     belong to the device that is current at the call;
 *   - plans are immutable host objects, safe to share between threads and devices;
 *   - index tensors are not range-checked unless stated (same precondition as the reference,
 *     cuequivariance_torch/primitives/segmented_polynomial.py:278-279).
 */
#ifndef CUEQ_B200_H
#define CUEQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CUEQ_B200_ABI_VERSION 1
#define CUEQ_MAX_BUFFERS 16  /* inputs + outputs of one polynomial */
#define CUEQ_MAX_OPERANDS 8  /* operands of one tensor product     */

/* element types of buffers / math */
enum { CUEQ_F32 = 0, CUEQ_F64 = 1, CUEQ_BF16 = 2, CUEQ_F16 = 3 };

/* how the batch axis of a buffer is addressed: the BATCH_DIM_* constants of the reference
 * (segmented_polynomial_uniform_1d.py:25-30) */
enum { CUEQ_SHARED = 0, CUEQ_BATCHED = 1, CUEQ_INDEXED = 2 };

typedef struct cueq_plan cueq_plan;

/* A polynomial with scalar coefficients and one uniform mode: the lists that
 * SegmentedPolynomialFromUniform1dJit serialises (segmented_polynomial_uniform_1d.py:188-218).
 * Buffers are numbered inputs first, then outputs. */
typedef struct {
  int32_t operand_extent;             /* extent of the single mode u (1 if there is none)        */
  int32_t num_inputs;
  int32_t num_outputs;
  const int32_t* buffer_dim;          /* [num_inputs+num_outputs] 0: scalar segments, 1: (u,)    */
  const int32_t* buffer_num_segments; /* [num_inputs+num_outputs]                                */
  int32_t num_operations;
  const int32_t* num_operands;        /* [num_operations]                                        */
  const int32_t* operations;          /* concatenated buffer ids, one per operand                */
  const int32_t* num_paths;           /* [num_operations]                                        */
  const int32_t* path_indices;        /* concatenated [num_paths][num_operands] segment ids      */
  const double* path_coefficients;    /* concatenated [num_paths]                                */
  int32_t math_dtype;                 /* CUEQ_F32 or CUEQ_F64                                    */
} cueq_u1d_desc;

/* One buffer at launch time. */
typedef struct {
  void* ptr;          /* device pointer, row-major [rows, operand_size], contiguous               */
  int64_t rows;
  int32_t mode;       /* CUEQ_SHARED (rows == 1), CUEQ_BATCHED (rows == batch), CUEQ_INDEXED      */
  int32_t dtype;      /* CUEQ_F32 / F64 / BF16 / F16                                              */
  const void* index;  /* device pointer [batch] when mode == CUEQ_INDEXED, else NULL               */
  int32_t index_is_64; /* 1: int64 indices, 0: int32                                              */
  int32_t reserved;
} cueq_buffer;

int cueq_b200_abi_version(void);
/* Measurement aid, no reference counterpart: `blocks` x 256 threads each run 16 chains of `iters` dependent
 * float32 multiply-adds in registers (2 * blocks * 256 * 16 * iters flop).  Timed by the caller with CUDA
 * events, it gives the float32 FMA peak that the straight-line symmetric-contraction kernels are rated against. */
int cueq_b200_selftest_fma_peak(void* sink, int32_t blocks, int32_t iters, void* stream);
/* The same with the packed float32x2 multiply-add of sm_100 (two multiply-adds per thread and instruction). */
int cueq_b200_selftest_fma2_peak(void* sink, int32_t blocks, int32_t iters, void* stream);
/* Debug aid (the reference documents index range as an unchecked precondition,
 * cuequivariance_torch/primitives/segmented_polynomial.py:278-279): sets *status (device int32) to 3 if any of
 * the n gather / scatter indices lies outside [0, rows).  Nothing traps; the host reads the word. */
int cueq_b200_check_index_range(const void* index, int64_t n, int64_t rows, int32_t index_is_64, void* status,
                                void* stream);
/* One asynchronous device-to-device copy on `stream` (cudaMemcpyAsync); dst or src may be memory of
 * another GPU of the node mapped into this process.  Used for the exchange of node features between
 * the ranks of a receiver-sharded product, which then needs no SM.  The reference has no multi-GPU
 * code; there is no counterpart. */
int cueq_b200_copy_async(void* dst, const void* src, size_t bytes, void* stream);
/* Pushes up to eight pieces of local device memory into other buffers - typically memory of peer GPUs mapped
 * into this process - with one small kernel (16-byte stores over NVLink; `blocks_per_piece` thread blocks of
 * 256 threads per piece, 0 = 4).  Asynchronous on `stream`, never blocks the host.  Pieces must be 16-byte
 * aligned and a multiple of 16 bytes.  No counterpart in the reference (it has no multi-GPU code). */
typedef struct {
  void* dst[8];
  const void* src[8];
  int64_t bytes[8];
  int32_t num_pieces;
  int32_t blocks_per_piece;
} cueq_push_args;
int cueq_b200_push(const cueq_push_args* args, void* stream);
/* Sharing a device buffer with the other processes of the node (CUDA IPC).  export: writes the 64-byte handle of
 * the allocation containing `ptr` and the offset of `ptr` inside it.  open: maps that allocation for the CURRENT
 * device (peer access to the exporting GPU is enabled as needed) and returns its base; the pointer is then
 * base + offset.  close: unmaps.  No counterpart in the reference. */
int cueq_b200_ipc_export(const void* ptr, void* handle64, int64_t* offset);
int cueq_b200_ipc_open(const void* handle64, void** base);
int cueq_b200_ipc_close(void* base);
/* Enables direct access from the current device to `peer_device` (cudaDeviceEnablePeerAccess; already
 * enabled counts as success), so that the copies above travel over NVLink instead of through the host. */
int cueq_b200_enable_peer_access(int peer_device);
const char* cueq_b200_last_error(void);
/* sizeof() of an argument block as this library was compiled, so that a binding can check its own
   declaration before the first launch: 0 cueq_u1d_desc, 1 cueq_buffer, 2 cueq_cw_args,
   3 cueq_cw_noalloc_args, 4 cueq_gemm_args, 5 cueq_fctp_args, 6 cueq_fctp_fused_args,
   7 cueq_fctp_fused_task, 8 cueq_fctp_fused_gx_args, 9 cueq_fctp_fused_unit,
   10 cueq_fctp_fused_gw_args, 11 cueq_fctp_fused_wunit, 12 cueq_gemm_f32x3_args,
   13 cueq_gemm_f32x3_tn_args, 14 cueq_sh_args; -1 for any other number. */
int64_t cueq_b200_sizeof(int which);

/* ---- generic uniform-1d executor (replaces torch.ops.cuequivariance.uniform_1d) ----------- */

/* Compiles the description into a plan (host only, no CUDA call). */
int cueq_b200_u1d_plan_create(const cueq_u1d_desc* desc, cueq_plan** out);
void cueq_b200_plan_destroy(cueq_plan* plan);

/* The plan's device tables: the caller copies `cueq_b200_plan_table_bytes` bytes from
 * `cueq_b200_plan_table_data` to 16-byte aligned device memory once per device and passes
 * that pointer to every launch. */
size_t cueq_b200_plan_table_bytes(const cueq_plan* plan);
const void* cueq_b200_plan_table_data(const cueq_plan* plan);

/* out_j[row_j(z)] += sum_ops sum_paths c * prod_k in_k[row_k(z)]  for z in [0, batch).
 * Outputs must be zero-initialised by the caller (they are accumulated into).  Asynchronous on
 * `stream`. */
int cueq_b200_u1d_launch(const cueq_plan* plan, const void* tables_dev, int64_t batch,
                         const cueq_buffer* buffers, int32_t num_buffers, void* stream);

/* ---- layout transposition (replaces segmented_transpose) ---------------------------------- */

/* Per row, per block b: a [u_b, v_b] tile at `offset_b` becomes [v_b, u_b].  `info` is a
 * device int32 array [num_blocks][4] = (offset, u, v, unused), the reference's format
 * (transpose.py:155-168).  x and y are [rows, dim] contiguous and must not alias. */
int cueq_b200_segmented_transpose(const void* x, void* y, int64_t rows, int64_t dim,
                                  const int32_t* info_dev, int32_t num_blocks, int32_t dtype,
                                  void* stream);


/* ---- spherical harmonics of 3-vectors, normalisation fused -----------------------------------
 *
 * Replaces, for degrees 0..4, what SphericalHarmonics.forward does in two steps
 * (cuequivariance_torch/operations/spherical_harmonics.py:76-93: torch normalize, then the polynomial of
 * cue.descriptors.spherical_harmonics, cuequivariance/group_theory/descriptors/spherical_harmonics_.py:23-52)
 * and its first derivative.  `ls_mask` has bit l set for every requested degree; the output row holds the
 * blocks of the requested degrees in ascending order (cueq_b200_sh_width elements).  forward: y = Y(vec or
 * vec/|vec|); backward: `y` is the COTANGENT of the output and gvec[rows, 3] receives the gradient with
 * respect to vec.  Row pitches in elements; float32 or float64. */
typedef struct {
  const void* vec;      /* [rows, ld_vec], 3 used columns                                          */
  void* y;              /* forward: output [rows, ld_y]; backward: its cotangent (read only)       */
  void* gvec;           /* backward: [rows, ld_gvec], 3 columns written; forward: unused           */
  int64_t rows, ld_vec, ld_y, ld_gvec;
  uint32_t ls_mask;
  int32_t normalize;    /* 1: divide the vectors by max(|v|, 1e-12) first                          */
  int32_t dtype;        /* CUEQ_F32 or CUEQ_F64                                                    */
  int32_t reserved;
} cueq_sh_args;
int cueq_b200_sh_width(uint32_t ls_mask);
int cueq_b200_sh_forward(const cueq_sh_args* args, void* stream);
int cueq_b200_sh_backward(const cueq_sh_args* args, void* stream);

/* ---- channelwise ("uvu") tensor product, specialised kernels --------------------------------
 *
 * Replace the uniform_1d op for the polynomial uv,iu,jv,kuv+ijk of
 * cue.descriptors.channelwise_tensor_product (cuequivariance/group_theory/descriptors/irreps_tp.py:232-321)
 * as called by ChannelWiseTensorProduct.forward (cuequivariance_torch/operations/tp_channel_wise.py:186-258),
 * float32, with the gather of x1 by sender, the scatter-add to receivers and the mul_ir<->ir_mul
 * transpositions (tp_channel_wise.py:221-222,258) fused.  One call handles one *group*: the paths
 * that read the same irrep of x1.  Built-in groups are enumerated with cueq_b200_cw_num_groups /
 * cueq_b200_cw_group_signature ("l1:l2.l3,l2.l3,..." in descriptor path order).
 *
 * Edges are addressed through a CSR over receivers: rowptr[n]..rowptr[n+1] are the positions
 * of receiver n, order[pos] the edge id at a position (NULL: positions are edge ids, i.e. the
 * edge list is sorted by receiver), senders[edge] the x1 row (NULL: the edge id).
 * The tables describe M[i,k] = sum_j C[i,j,k] x2[j]: entry q owns terms tab_start[q]..tab_start[q+1],
 * each term a coefficient tab_c[t] and an x2 element tab_j[t].  Backward call: one entry per non-zero
 * (i,k) pair, path by path, i-major.  Forward call: one entry per DISTINCT value among a path's pairs
 * (pairs that carry the same combination of x2 up to sign share an entry; order of first appearance in
 * k-major order, first coefficient positive - cuequivariance_b200/channelwise.py:value_pattern).  bwd_coef (host memory,
 * num_terms floats) lists the coefficients in the backward term order. */
typedef struct {
  const void* w;        /* [E, w_stride]    per-edge weights                                  */
  const void* x1;       /* [N1, x1_stride]  node features                                     */
  const void* x2;       /* [E, x2_stride]   per-edge second operand (one scalar per component) */
  void* out;            /* forward: [num_receivers, out_stride], every row is overwritten       */
  const void* gout;     /* backward: cotangent of out                                           */
  void* gw;             /* backward: [E, w_stride], overwritten; NULL to skip                   */
  void* gx1;            /* backward: [N1, x1_stride], ACCUMULATED into (zero it first); NULL to skip */
  void* gx2;            /* backward: [E, x2_stride], ACCUMULATED into (zero it first); NULL to skip  */
  const int32_t* senders;
  const int32_t* order;
  const int32_t* rowptr;
  const int32_t* tab_start;
  const int32_t* tab_j;
  const float* tab_c;
  const float* bwd_coef;
  int64_t w_stride, x1_stride, x2_stride, out_stride; /* row strides in elements               */
  int64_t num_receivers;
  int32_t extent;       /* channels per segment (multiple of 4)                                 */
  int32_t x1_offset;    /* element offset of the group's irrep block in an x1 row               */
  int32_t num_paths, num_terms;
  int32_t w_offset[8];  /* element offset of each path's weight segment in a w row              */
  int32_t out_offset[8];/* element offset of each path's output block in an out row             */
  int32_t x1_mul_ir;    /* 1: x1/gx1 blocks are [channel][component], 0: [component][channel]   */
  int32_t out_mul_ir;   /* same for out/gout (must equal x1_mul_ir)                             */
  int32_t channels_per_lane; /* 0: automatic; 2 or 4: channels owned by one thread              */
  int32_t staging;      /* forward only: 0 = per-lane cp.async staging, 1 = bulk copies (TMA) + mbarrier */
  void* status;         /* nullable device int32: set to 1 if a bounded wait on a bulk copy ran out */
  int32_t recv_mod;     /* backward only: if > 0 the CSR has several rows per receiver (row r belongs to
                           receiver r % recv_mod), used to visit the edges in sender-range passes        */
  int32_t variant;      /* backward only: 0 = the library chooses (3 from 128 channels on for x1 degrees >= 1,
                           2 for the scalar block, 1 otherwise); 1 = one warp per receiver (2 or 4 channels
                           per thread); 2 = one thread block per receiver: its warps share the staged
                           cotangent row and split the receiver's edges, four channels per thread;
                           3 = as 2, with the x1 gradient of an edge leaving as one bulk reduction
                           (cp.reduce.async.bulk) per warp instead of vector reductions per lane (mul_ir
                           rows, 128 | extent; falls back to 2 where the rows are not 16-byte aligned)        */
} cueq_cw_args;

int cueq_b200_cw_num_groups(void);
const char* cueq_b200_cw_group_signature(int group);
int cueq_b200_cw_group_info(int group, int32_t* d1, int32_t* num_paths, int32_t* num_pairs, int32_t* num_terms);
int cueq_b200_cw_forward(int group, const cueq_cw_args* args, void* stream);
int cueq_b200_cw_backward(int group, const cueq_cw_args* args, void* stream);

/* ---- kernels written out at build time for known polynomials ---------------------------------
 *
 * Same contract as cueq_b200_u1d_launch (float32 only, outputs zero-initialised by the caller,
 * accumulated with atomics unless batched), for polynomials whose straight-line code was
 * generated when the library was built - the counterpart of the per-polynomial NVRTC kernels of
 * the reference's closed op (CHANGELOG.md:38,49).  `digest` identifies the polynomial
 * (cuequivariance_b200/static_poly.py); _find returns a kernel id or -1. */
int cueq_b200_u1d_static_find(const char* digest);
const char* cueq_b200_u1d_static_name(int id);
int cueq_b200_u1d_static_launch(int id, int64_t batch, int32_t extent, const cueq_buffer* buffers,
                                const int32_t* buffer_dim, const int32_t* buffer_num_segments,
                                int32_t num_buffers, void* stream);

/* ---- tensor-core GEMM for the dense (uvw) contractions --------------------------------------
 *
 * C[M,N] (+)= A[M,K] * B[N,K]^T, bf16 operands (both K-major, leading dimensions lda/ldb in
 * elements), float32 result, written with TMA + tcgen05.mma + TMEM.  Stands where the closed
 * FusedTensorProductOp4 kernel does its dense contraction
 * (cuequivariance_torch/primitives/segmented_polynomial_fused_tp.py:51-72).  N must be a
 * multiple of 64 and K of 64.  `status` (nullable device int32) is set to 2 if an internal
 * bounded wait ran out (the result is then invalid). */
/* General form.  An operand is K-major when stored [M or N][K] (K contiguous, the default) or
 * MN-major when stored [K][M or N]; ld* are the row pitches in elements.  Output row r is written at
 * C + (r / rows_per_group) * group_stride + (r % rows_per_group) * ldc (rows_per_group < 1 counts as
 * 1; group_stride 0 means rows_per_group * ldc, i.e. plain C + r * ldc), as float32 (optionally
 * accumulated into) or bf16. */
typedef struct {
  const void* A;
  const void* B;
  void* C;
  int64_t M, N, K;
  int64_t lda, ldb, ldc;
  int64_t group_stride;
  int32_t rows_per_group;
  int32_t accumulate;
  int32_t out_bf16;
  int32_t a_mn_major, b_mn_major;
  int32_t c_is_zero;    /* 1: C holds zeros, so the library may split K over several CTAs and add
                           their partial sums atomically (it also may when accumulate is set)    */
  void* status;
} cueq_gemm_args;
int cueq_b200_gemm_bf16(const cueq_gemm_args* args, void* stream);
int cueq_b200_gemm_bf16_tn(const void* A, const void* B, float* C, int64_t M, int64_t N, int64_t K,
                           int64_t lda, int64_t ldb, int64_t ldc, int32_t accumulate, void* status,
                           void* stream);

/* float32-accurate dense layer on the tensor cores: C[M,N] = A[M,K] * B[N,K]^T (+ bias[N]),
 * K a multiple of 32, every operand float32.  Three TF32 passes over operands split as x = hi + lo
 * (hi = x rounded to TF32, i.e. to 10 mantissa bits, lo = (x - hi) rounded likewise): the caller
 * passes B already split (B_hi, B_lo, same shape and pitch), A is split inside the kernel.
 * The layer that produces per-edge tensor-product weights from edge scalars in the reference's
 * convolution (cuequivariance_torch/layers/tp_conv_fully_connected.py:145-152,219-238) has this
 * shape.  C is written (not accumulated); rows of A, B, C and bias must be 16-byte aligned. */
typedef struct {
  const void* A;        /* device float32 [M, lda]                                                 */
  const void* B_hi;     /* device float32 [N, ldb]                                                 */
  const void* B_lo;     /* device float32 [N, ldb]                                                 */
  const void* bias;     /* nullable device float32 [N]                                             */
  void* C;              /* device float32 [M, ldc]                                                 */
  int64_t M, N, K, lda, ldb, ldc;
  void* status;         /* nullable device int32: 2 if a bounded wait ran out                      */
} cueq_gemm_f32x3_args;
int cueq_b200_gemm_f32x3(const cueq_gemm_f32x3_args* args, void* stream);

/* The same arithmetic for a reduction over rows: C[M,N] += sum_k A[k,M] * B[k,N], and optionally
 * colsum[M] += sum_k A[k,M] - the weight and bias gradients of the layer above (A = cotangent,
 * B = the layer's input).  C and colsum are float32 and are accumulated into with atomic adds (zero
 * them first; the K range is spread over many CTAs).  M and N multiples of 4, rows 16-byte aligned. */
typedef struct {
  const void* A;        /* device float32 [K, lda]                                                 */
  const void* B;        /* device float32 [K, ldb]                                                 */
  void* C;              /* device float32 [M, ldc], accumulated into                               */
  void* colsum;         /* nullable device float32 [M], accumulated into                           */
  int64_t M, N, K, lda, ldb, ldc;
  void* status;         /* nullable device int32: 2 if a bounded wait ran out                      */
} cueq_gemm_f32x3_tn_args;
int cueq_b200_gemm_f32x3_tn(const cueq_gemm_f32x3_tn_args* args, void* stream);

/* ---- fully connected ("uvw") tensor product: kernels around the tensor-core GEMM -----------------
 *
 * For one path of uvw,iu,jv,kw+ijk (cue.descriptors.fully_connected_tensor_product,
 * cuequivariance/group_theory/descriptors/irreps_tp.py:22-91; module forward at
 * cuequivariance_torch/operations/tp_fully_connected.py:166-207) with coupling tensor cg[i][j][k]
 * (host array, d1*d2*d3 floats, normalisation included):
 *   build_z   : Z[(z,k), (u,v)] = sum_ij cg[i,j,k] x1[z, off1 + i*U + u] x2[z, off2 + j*V + v]   ([batch*d3, U*V], bf16 or float32)
 *   consume_gz: gx1[z, off1 + i*U + u] += sum_jkv cg[i,j,k] gZ[(z,k),(u,v)] x2[...]
 *               gx2[z, off2 + j*V + v] += sum_iku cg[i,j,k] gZ[(z,k),(u,v)] x1[...]
 * x1/x2 are float32 or bf16 (x_dtype), component-major (ir_mul) rows of pitch ld1/ld2; gx1/gx2
 * are float32 with the same pitches (either may be NULL); z is the output of build_z or the gZ
 * input of consume_gz (float32 or bf16, z_dtype), rows `ldz` elements apart: a block of columns of a
 * wider matrix when the paths that feed one output irrep are contracted by a single GEMM. */
typedef struct {
  const void* x1;
  const void* x2;
  void* z;
  void* gx1;
  void* gx2;
  const float* cg;
  int64_t ld1, ld2, batch;
  int32_t off1, off2;
  int32_t d1, d2, d3, U, V;
  int32_t x_dtype, z_dtype;
  int32_t ldz;          /* row pitch of z in elements; 0 = U*V */
} cueq_fctp_args;
int cueq_b200_fctp_build_z(const cueq_fctp_args* args, void* stream);
int cueq_b200_fctp_consume_gz(const cueq_fctp_args* args, void* stream);

/* ---- fully connected product with the coupled operand built on chip ---------------------------
 *
 * Same operation as build_z + GEMM (+ consume_gz) above - the dense contraction behind
 * FusedTensorProductOp4 (cuequivariance_torch/primitives/segmented_polynomial_fused_tp.py:51-72)
 * for the descriptor uvw,iu,jv,kw+ijk (cuequivariance/group_theory/descriptors/irreps_tp.py:22-91) -
 * but Z = C . x1 . x2 is produced tile by tile in shared memory as the tensor-core operand and is
 * never written to device memory.  Restrictions: all three multiplicities are 64, irrep dimensions
 * 1, 3 or 5, x1 / x2 / W in bfloat16, rows in ir_mul layout (component-major blocks of 64).
 *
 * A task is one (output irrep, component k): `out_off` = offset of that component's 64 outputs in
 * an output row; its paths are all the paths that end in that irrep, each with the offsets of its
 * x1 / x2 segments, the first row of its [4096, 64] weight block inside W (W is one bf16 array
 * [w_rows, 64], row = (u * 64 + v) within a block) and c[i * 5 + j] = C[i, j, k] (normalisation
 * included).  Forward writes every task's [batch, 64] block once (no accumulation). */
#define CUEQ_FCTP_FUSED_MAX_TASKS 12
#define CUEQ_FCTP_FUSED_MAX_PATHS 4
typedef struct {
  int32_t off1, off2;   /* element offsets of the path's x1 / x2 segments inside a row            */
  int32_t d1, d2;       /* irrep dimensions of x1 / x2 for this path                               */
  int32_t w_row0;       /* first row of the path's weight block in W                               */
  int32_t reserved;
  float c[25];          /* C[i, j, k] for the task's k at c[i * 5 + j]                             */
  float reserved2;
} cueq_fctp_fused_path;
typedef struct {
  int32_t out_off;      /* element offset inside an output row                                     */
  int32_t num_paths;    /* 1 .. CUEQ_FCTP_FUSED_MAX_PATHS                                          */
  cueq_fctp_fused_path paths[CUEQ_FCTP_FUSED_MAX_PATHS];
} cueq_fctp_fused_task;
typedef struct {
  const void* x1;       /* device bf16 [batch, ld1]                                                */
  const void* x2;       /* device bf16 [batch, ld2]                                                */
  const void* w;        /* device bf16 [w_rows, 64]                                                */
  void* out;            /* device float32 or bf16 [batch, ldo]                                     */
  int64_t ld1, ld2, ldo, batch, w_rows;
  int32_t out_dtype;    /* CUEQ_F32 or CUEQ_BF16                                                   */
  int32_t num_tasks;    /* 1 .. CUEQ_FCTP_FUSED_MAX_TASKS                                          */
  const cueq_fctp_fused_task* tasks;  /* HOST array, copied into the launch parameters            */
  void* status;         /* nullable device int32: 2 if a bounded wait ran out                      */
} cueq_fctp_fused_args;
int cueq_b200_fctp_fused_forward(const cueq_fctp_fused_args* args, void* stream);

/* Gradient of the same product with respect to x1 or x2 ("a" = the operand being differentiated,
 * "b" = the other one):
 *   gxa[z, ia, a] += sum_k sum_jb C[ia, jb, k] sum_b (sum_w gout[z, k, w] W[(a, b), w]) xb[z, jb, b]
 * `w` rows are ordered (a, b): the forward array for x1; for x2 a copy with every [64 u][64 v]
 * block transposed to [v][u], and c[k][ia * 5 + jb] then holds C[jb_as_i, ia_as_j, k].
 * A unit is one path and up to two components k (goff[k] = offset of that component's 64 values
 * in a cotangent row).  gxa is float32 and is accumulated into (zero it first). */
#define CUEQ_FCTP_FUSED_MAX_UNITS 32
typedef struct {
  int32_t offa, offb;   /* element offsets of the path's segments in a gxa row / an xb row          */
  int32_t da, db;       /* irrep dimensions of the differentiated / the other operand              */
  int32_t w_row0;       /* first row of the path's weight block                                    */
  int32_t nk;           /* 1 or 2 components                                                       */
  int32_t goff[2];
  float c[2][25];
} cueq_fctp_fused_unit;
typedef struct {
  const void* xb;       /* device bf16 [batch, ldb]                                                */
  const void* gout;     /* device bf16 [batch, ldg]                                                */
  const void* w;        /* device bf16 [w_rows, 64]                                                */
  void* gxa;            /* device float32 [batch, lda], accumulated into                           */
  int64_t ldb, ldg, lda, batch, w_rows;
  int32_t num_units;    /* 1 .. CUEQ_FCTP_FUSED_MAX_UNITS                                          */
  int32_t reserved;
  const cueq_fctp_fused_unit* units;  /* HOST array                                                */
  void* status;         /* nullable device int32: 2 if a bounded wait ran out                      */
} cueq_fctp_fused_gx_args;
int cueq_b200_fctp_fused_gx(const cueq_fctp_fused_gx_args* args, void* stream);

/* Gradient of the same product with respect to the (shared) weights:
 *   gw[(u, v), w] += sum_z sum_k (sum_ij C[i, j, k] x1[z, i, u] x2[z, j, v]) gout[z, k, w]
 * One unit per (path, component k); gw is the float32 array [w_rows, 64] laid out like W and
 * is accumulated into (zero it first). */
#define CUEQ_FCTP_FUSED_MAX_WUNITS 48
typedef struct {
  int32_t off1, off2;   /* element offsets of the path's x1 / x2 segments                          */
  int32_t d1, d2;
  int32_t w_row0;       /* first row of the path's block in gw                                     */
  int32_t goff;         /* element offset of component k of the path's output irrep in a cotangent row */
  float c[25];          /* c[i * 5 + j] = C[i, j, k]                                               */
  float reserved;
} cueq_fctp_fused_wunit;
typedef struct {
  const void* x1;       /* device bf16 [batch, ld1]                                                */
  const void* x2;       /* device bf16 [batch, ld2]                                                */
  const void* gout;     /* device bf16 [batch, ldg]                                                */
  void* gw;             /* device float32 [w_rows, 64], accumulated into                           */
  int64_t ld1, ld2, ldg, batch, w_rows;
  int32_t num_units;    /* 1 .. CUEQ_FCTP_FUSED_MAX_WUNITS                                         */
  int32_t reserved;
  const cueq_fctp_fused_wunit* units;  /* HOST array                                               */
  void* status;         /* nullable device int32: 2 if a bounded wait ran out                      */
} cueq_fctp_fused_gw_args;
int cueq_b200_fctp_fused_gw(const cueq_fctp_fused_gw_args* args, void* stream);

/* Self-test (no counterpart in the reference): launches one thread that waits on a barrier nothing
 * arrives on.  After about half a second the wait gives up, `status` (device int32) becomes 2 and
 * `waited_cycles` (nullable device int64) receives the SM cycles spent; the context stays usable.
 * This is the time-out path of every bounded wait in the tensor-core kernels. */
int cueq_b200_selftest_bounded_wait(void* status, void* waited_cycles, void* stream);

/* ---- channelwise forward for callers that cannot allocate ----------------------------------
 *
 * No counterpart in the reference.  cueq_b200_cw_forward expects the caller to keep the CSR row
 * pointers and the term tables in device memory of its own.  A caller that is not allowed to
 * obtain device memory - a plugin whose host hands it nothing but input and output buffers, code
 * running under an allocator it must not touch, a latency-critical loop where cudaMalloc is
 * banned - can use this variant instead: it takes the receiver index itself (int32, sorted
 * ascending, one entry per edge) and the term tables as HOST arrays, and keeps the derived row
 * pointers and the device copy of the tables in a fixed array inside the library (about 1 MiB,
 * present on every GPU that loads the library until the process exits).
 *
 * Limits and rules
 *   - at most 262,144 receivers (more is rejected with an error; use cueq_b200_cw_forward);
 *   - edges must already be sorted by receiver (there is no `order` argument);
 *   - the call performs no cudaMalloc/cudaFree and calls no allocating routine; it enqueues two
 *     kernels on `stream` (row pointers + tables, then the product);
 *   - the first call on a device looks up the address of the built-in array (with that device
 *     current); make that first call outside any stream capture;
 *   - all calls on one GPU share the array, which keeps what the last call wrote; every call
 *     rewrites the parts it uses, nothing has to be cleared, but two calls that overlap on the
 *     GPU (different streams) race on it: serialise them. */
typedef struct {
  const void* w;
  const void* x1;
  const void* x2;
  void* out;
  const int32_t* senders;        /* device, [num_edges]; NULL: x1 row = edge id                     */
  const int32_t* receivers;      /* device, [num_edges], sorted ascending, values in [0, num_receivers) */
  const int32_t* tab_start_host; /* host, [entries + 1] (the forward table of cw_forward)             */
  const int32_t* tab_j_host;     /* host, [num_terms]                                                */
  const float* tab_c_host;       /* host, [num_terms]                                                */
  int64_t w_stride, x1_stride, x2_stride, out_stride;
  int64_t num_edges, num_receivers;
  int32_t extent, x1_offset, num_paths, num_terms;
  int32_t w_offset[8];
  int32_t out_offset[8];
  int32_t mul_ir;                /* layout of x1 and out, as in cueq_cw_args                         */
  int32_t reserved;
} cueq_cw_noalloc_args;

int cueq_b200_cw_forward_noalloc(int group, const cueq_cw_noalloc_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CUEQ_B200_H */

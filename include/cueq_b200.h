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
const char* cueq_b200_last_error(void);

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

#ifdef __cplusplus
}
#endif
#endif /* CUEQ_B200_H */

"""``torch.ops.cuequivariance.uniform_1d`` implemented on the cuequivariance_b200 executor.

Schema and argument meaning are those of the reference call site
(cuequivariance_torch/primitives/segmented_polynomial_uniform_1d.py:32-77,242-316):
``tensors`` = inputs followed by index tensors; ``batch_dim[b]`` says how buffer ``b`` is
addressed; ``index_buffer`` holds, for every buffer, the position of its index tensor (or -1)
followed by the row count of every indexed buffer; ``dtypes[b]`` names the input whose dtype
buffer ``b`` takes (-1: the math dtype); operations and paths are flattened lists.  The op is
registered as a composite, so autograd (to any order) comes from the executor's own
differentiable function.
"""
from __future__ import annotations

from typing import List

import numpy as np
import torch

from cuequivariance_b200 import _lib as _native
from cuequivariance_b200.executor import BufferSpec, CallConfig, PolynomialFunction, Uniform1dProgram
from cuequivariance_b200.channelwise import attach_specialisation
from cuequivariance_b200.polynomial import Operation, Polynomial
from cuequivariance_b200.stp import Operand, Path, SegmentedTensorProduct
from cuequivariance_b200.transpose import _launch as _transpose_launch

BATCH_DIM_AUTO = -1
BATCH_DIM_SHARED = 0
BATCH_DIM_BATCHED = 1
BATCH_DIM_INDEXED = 2

_SCHEMA = (
    "uniform_1d(str name, ScalarType math_dtype, int operand_extent, int num_inputs, int num_outputs, int num_index, "
    "int[] buffer_dim, int[] buffer_num_segments, int[] batch_dim, int[] index_buffer, int[] dtypes, int num_operations, "
    "int[] num_operands, int[] operations, int[] num_paths, int[] path_indices_start, int[] path_coefficients_start, "
    "int[] path_indices, float[] path_coefficients, int batch_size, Tensor[] tensors) -> Tensor[]"
)
_library = torch.library.Library("cuequivariance", "DEF")
_library.define(_SCHEMA)
_PROGRAMS: dict = {}


def _program(math_dtype, extent, num_inputs, num_outputs, buffer_dim, buffer_nseg, dtypes, num_operands, operations,
             num_paths, path_indices, path_coefficients, name) -> Uniform1dProgram:
    key = (math_dtype, extent, num_inputs, num_outputs, tuple(buffer_dim), tuple(buffer_nseg), tuple(dtypes),
           tuple(num_operands), tuple(operations), tuple(num_paths), tuple(path_indices), tuple(path_coefficients))
    prog = _PROGRAMS.get(key)
    if prog is None:
        operands = [Operand(d, (((extent,) if d else ()),) * n) for d, n in zip(buffer_dim, buffer_nseg)]
        ops, ob, pi, pc = [], 0, 0, 0
        for n_opnd, n_path in zip(num_operands, num_paths):
            buffers = tuple(operations[ob : ob + n_opnd])
            stp = SegmentedTensorProduct(tuple("u" if buffer_dim[b] else "" for b in buffers), "", [operands[b] for b in buffers], [])
            idx = np.array(path_indices[pi : pi + n_path * n_opnd], dtype=np.int64).reshape(n_path, n_opnd)
            stp.paths = [Path(tuple(int(i) for i in row), np.float64(c)) for row, c in zip(idx, path_coefficients[pc : pc + n_path])]
            ops.append((Operation(buffers), stp))
            ob, pi, pc = ob + n_opnd, pi + n_path * n_opnd, pc + n_path
        poly = Polynomial(operands[:num_inputs], operands[num_inputs:], ops)
        prog = Uniform1dProgram(poly, math_dtype, list(dtypes[num_inputs:]), name)
        attach_specialisation(prog)
        _PROGRAMS[key] = prog
    return prog


def _uniform_1d(name, math_dtype, operand_extent, num_inputs, num_outputs, num_index, buffer_dim, buffer_num_segments,
                batch_dim, index_buffer, dtypes, num_operations, num_operands, operations, num_paths, path_indices_start,
                path_coefficients_start, path_indices, path_coefficients, batch_size, tensors) -> List[torch.Tensor]:
    nb = num_inputs + num_outputs
    inputs, index_tensors = list(tensors[:num_inputs]), list(tensors[num_inputs:])
    index_rows = list(index_buffer[nb:])
    prog = _program(math_dtype, operand_extent, num_inputs, num_outputs, list(buffer_dim), list(buffer_num_segments),
                    list(dtypes), list(num_operands), list(operations), list(num_paths), list(path_indices),
                    list(path_coefficients), name)
    batch = None if batch_size == BATCH_DIM_AUTO else int(batch_size)

    def see(n):
        nonlocal batch
        if batch is None:
            batch = n
        elif batch != n:
            raise ValueError(f"inconsistent batch size: {n} vs {batch}")

    in_specs = []
    for b in range(num_inputs):
        x, mode = inputs[b], batch_dim[b]
        if mode == BATCH_DIM_INDEXED:
            idx = index_tensors[index_buffer[b]]
            see(idx.shape[0])
            in_specs.append(BufferSpec(_native.INDEXED, x.shape[0], idx))
        elif mode == BATCH_DIM_SHARED or (mode == BATCH_DIM_AUTO and x.shape[0] == 1):
            in_specs.append(BufferSpec(_native.SHARED, 1, None))
        else:
            see(x.shape[0])
            in_specs.append(BufferSpec(_native.BATCHED, x.shape[0], None))
    for b in range(num_inputs, nb):
        if batch_dim[b] == BATCH_DIM_INDEXED:
            see(index_tensors[index_buffer[b]].shape[0])
    if batch is None:
        batch = 1
    out_specs = []
    for b in range(num_inputs, nb):
        mode = batch_dim[b]
        if mode == BATCH_DIM_INDEXED:
            out_specs.append(BufferSpec(_native.INDEXED, index_rows[index_buffer[b]], index_tensors[index_buffer[b]]))
        elif mode == BATCH_DIM_SHARED or batch == 1:
            out_specs.append(BufferSpec(_native.SHARED, 1, None))
        else:
            out_specs.append(BufferSpec(_native.BATCHED, batch, None))
    cfg = CallConfig(batch, tuple(in_specs), tuple(out_specs))
    return list(PolynomialFunction.apply(prog, cfg, *inputs))


_library.impl("uniform_1d", _uniform_1d, "CompositeImplicitAutograd")


def segmented_transpose(x: torch.Tensor, info: torch.Tensor, contiguous: bool = True) -> torch.Tensor:
    """Per row, every ``[u, v]`` tile listed in ``info`` (rows ``offset, u, v, -1``) becomes
    ``[v, u]``; elements outside the listed tiles are copied unchanged."""
    dim = x.shape[-1]
    rows = sorted([int(v) for v in r[:3]] for r in info.cpu().tolist())
    full, off = [], 0
    for o, u, v in rows:
        if o > off:
            full.append([off, 1, o - off, -1])
        full.append([o, u, v, -1])
        off = o + u * v
    if off < dim:
        full.append([off, 1, dim - off, -1])
    return _transpose_launch(x, torch.tensor(full, dtype=torch.int32, device=x.device).reshape(-1, 4))

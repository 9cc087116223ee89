"""CPU oracle: evaluates a segmented polynomial the way the reference's naive method does.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Restates, in its own code, the
algorithm of ``SegmentedPolynomialNaive`` and ``_tensor_product_fx``
(cuequivariance_torch/primitives/segmented_polynomial_naive.py):

* gather: ``inputs[k] = inputs[k][index]`` for every indexed input (:376-377);
* per operation, per path: slice one segment per input operand, reshape it to
  ``(Z, *segment_shape)``, and contract ``einsum(coeff, seg_0, ..., seg_{n-2})`` with a
  leading batch letter on every operand (:87-132); the coefficient is the float64 table
  cast to the input dtype, or to ``math_dtype`` together with the segments when one is
  given (:107-127);
* paths that land in the same output segment are added in path order and the segments
  are concatenated (:137-160);
* scatter: ``zeros(rows, size).scatter_add_(0, index, out)`` for an indexed output
  (:409-418); an un-indexed output with one row is the sum over the batch, a one-row
  result is broadcast to the requested rows (:419-429);
* operations bound to the same output add up (:430-433).

The polynomial is duck-typed: anything with ``inputs``/``outputs`` (objects with
``segments`` and ``size``) and ``operations`` = pairs ``(operation.buffers, stp)`` where
``stp`` has ``operand_subscripts``, ``coefficient_subscripts``, ``operands`` and
``paths`` (``indices``, ``coefficients``).  Everything runs on the CPU with torch ops, is
differentiable by autograd (which is how gradient oracles are obtained), and uses as
many host threads as torch is configured with.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

_BATCH = "Z"


def _segment_views(x: torch.Tensor, operand) -> List[torch.Tensor]:
    views, off = [], 0
    for shape in operand.segments:
        n = math.prod(shape)
        views.append(x[:, off : off + n].reshape((x.shape[0],) + tuple(shape)))
        off += n
    return views


def tensor_product(stp, out_operand: int, inputs: Sequence[torch.Tensor], math_dtype=None, dtype=None) -> torch.Tensor:
    """One segmented tensor product; ``inputs`` are the non-output operands in operand
    order, each ``[Z or 1, operand_size]``.  Returns ``[Z, size of out operand]``.  A
    product without inputs is the constant given by its coefficients (one row, ``dtype``;
    reference :185-239, 406-408)."""
    n = len(stp.operands)
    if n == 1:
        out = torch.zeros(1, stp.operands[0].size, dtype=dtype)
        offs = stp.operands[0].offsets()
        for path in stp.paths:
            c = torch.tensor(path.coefficients, dtype=torch.float64).to(dtype).reshape(-1)
            o = offs[path.indices[0]]
            out[0, o : o + c.numel()] += c
        return out
    in_ops = [k for k in range(n) if k != out_operand]
    subs = list(stp.operand_subscripts)
    formula = (
        ",".join([stp.coefficient_subscripts] + [_BATCH + subs[k] for k in in_ops])
        + "->" + _BATCH + subs[out_operand]
    )
    io_dtype = inputs[0].dtype
    views = {k: _segment_views(x, stp.operands[k]) for k, x in zip(in_ops, inputs)}
    out_op = stp.operands[out_operand]
    per_segment: List[Optional[torch.Tensor]] = [None] * len(out_op.segments)
    for path in stp.paths:
        segs = [views[k][path.indices[k]] for k in in_ops]
        c = torch.tensor(path.coefficients, dtype=torch.float64)
        if math_dtype is not None:
            segs = [s.to(math_dtype) for s in segs]
            c = c.to(math_dtype)
        else:
            c = c.to(io_dtype)
        r = torch.einsum(formula, c, *segs)
        if math_dtype is not None:
            r = r.to(io_dtype)
        r = r.reshape(r.shape[0], -1)
        s = path.indices[out_operand]
        per_segment[s] = r if per_segment[s] is None else per_segment[s] + r
    rows = max([x.shape[0] for x in inputs] + [1])
    pieces = []
    for s, shape in enumerate(out_op.segments):
        if per_segment[s] is None:
            pieces.append(torch.zeros(rows, math.prod(shape), dtype=io_dtype))
        else:
            p = per_segment[s]
            pieces.append(p if p.shape[0] == rows else p.expand(rows, p.shape[1]))
    return torch.cat(pieces, dim=1)


def segmented_polynomial(
    poly,
    inputs: Sequence[torch.Tensor],
    input_indices: Optional[Dict[int, torch.Tensor]] = None,
    output_shapes: Optional[Dict[int, int]] = None,
    output_indices: Optional[Dict[int, torch.Tensor]] = None,
    math_dtype=None,
    output_dtype_map: Optional[Sequence[int]] = None,
) -> List[torch.Tensor]:
    """Evaluate ``poly``.  ``output_shapes[j]`` is the row count of output ``j`` (int)."""
    input_indices = dict(input_indices or {})
    output_indices = dict(output_indices or {})
    output_shapes = {k: (v if isinstance(v, int) else v.shape[0]) for k, v in (output_shapes or {}).items()}
    n_in = len(poly.inputs)
    xs = list(inputs)
    for i, (x, op) in enumerate(zip(xs, poly.inputs)):
        if x.ndim != 2 or x.shape[1] != op.size:
            raise ValueError(f"input {i} has shape {tuple(x.shape)}, expected (*, {op.size})")
    src = list(xs)
    for k, idx in input_indices.items():
        xs[k] = xs[k][idx.long()]
    batch = 1
    for x in xs:
        if x.shape[0] != 1:
            if batch not in (1, x.shape[0]):
                raise ValueError("inconsistent batch sizes")
            batch = x.shape[0]
    dmap = list(output_dtype_map) if output_dtype_map is not None else [0] * len(poly.outputs)
    results: List[Optional[torch.Tensor]] = [None] * len(poly.outputs)
    for operation, stp in poly.operations:
        buffers = tuple(getattr(operation, "buffers", operation))
        k_out = [k for k, b in enumerate(buffers) if b >= n_in][0]
        j = buffers[k_out] - n_in
        ins = [xs[b] for k, b in enumerate(buffers) if k != k_out]
        out = tensor_product(stp, k_out, ins, math_dtype, dtype=xs[0].dtype)
        rows = output_shapes.get(j, batch)
        if j in output_indices:
            idx = output_indices[j].long()
            if out.shape[0] == 1 and idx.shape[0] > 1:
                out = out.expand(idx.shape[0], out.shape[1])
            dt = src[dmap[j]].dtype if dmap[j] >= 0 else out.dtype
            val = torch.zeros(rows, out.shape[1], dtype=dt).scatter_add(
                0, idx[:, None].expand_as(out), out.to(dt)
            )
        elif rows == out.shape[0]:
            val = out
        elif rows == 1:
            val = out.sum(dim=0, keepdim=True)
        elif out.shape[0] == 1:
            val = out.expand(rows, out.shape[1]).clone()
        else:
            raise ValueError(f"batch mismatch: output rows {rows}, computed rows {out.shape[0]}")
        results[j] = val if results[j] is None else results[j] + val
    for j, r in enumerate(results):
        if r is None:
            rows = output_shapes.get(j, batch)
            results[j] = torch.zeros(rows, poly.outputs[j].size, dtype=xs[0].dtype)
    return results


def transpose_layout(x: torch.Tensor, blocks: Sequence[tuple], to_ir_mul: bool) -> torch.Tensor:
    """Per row, per ``(mul, dim)`` block: mul_ir ``(mul, dim)`` <-> ir_mul ``(dim, mul)``
    (reference: cuequivariance_torch/primitives/transpose.py:134-152)."""
    out, off = [], 0
    for mul, dim in blocks:
        n = mul * dim
        seg = x[:, off : off + n]
        if to_ir_mul:
            seg = seg.reshape(-1, mul, dim).transpose(1, 2)
        else:
            seg = seg.reshape(-1, dim, mul).transpose(1, 2)
        out.append(seg.reshape(x.shape[0], n))
        off += n
    return torch.cat(out, dim=1) if out else x

"""TEST INFRASTRUCTURE ONLY - a second, independent CPU evaluator in plain numpy.

Plays the role of the reference's numpy evaluator
(cuequivariance/segmented_polynomials/segmented_polynomial.py:383-410 and
evaluate.py:25-139: ``compute_last_operand`` contracts, per path, the coefficient tensor with
one segment of every input operand by ``numpy.einsum`` and adds the result into the output
segment).  It shares no code with ``oracle/naive.py`` (which restates the torch executor):
no torch, no autograd, float64 throughout, explicit loops over operations and paths, and
gather / scatter written with ``numpy.take`` and ``numpy.add.at``.  The CPU tests require the
two oracles to agree; a disagreement would point at the oracle rather than at the kernels.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import numpy as np


def _segments(x: np.ndarray, operand):
    out, off = [], 0
    for shape in operand.segments:
        n = math.prod(shape)
        out.append(x[:, off : off + n].reshape((x.shape[0],) + tuple(shape)))
        off += n
    return out


def evaluate(poly, inputs: Sequence[np.ndarray], input_indices: Optional[Dict[int, np.ndarray]] = None,
             output_rows: Optional[Dict[int, int]] = None, output_indices: Optional[Dict[int, np.ndarray]] = None):
    """Returns the list of outputs (float64).  Semantics of the index arguments as in the torch
    executor: an indexed input is gathered, an indexed output scatter-added, an un-indexed
    output with one requested row is the sum over the batch."""
    input_indices, output_rows, output_indices = dict(input_indices or {}), dict(output_rows or {}), dict(output_indices or {})
    xs = [np.asarray(x, dtype=np.float64) for x in inputs]
    for k, idx in input_indices.items():
        xs[k] = np.take(xs[k], np.asarray(idx, dtype=np.int64), axis=0)
    batch = max([x.shape[0] for x in xs] + [1])
    n_in = len(poly.inputs)
    results = [None] * len(poly.outputs)
    for operation, stp in poly.operations:
        buffers = tuple(getattr(operation, "buffers", operation))
        k_out = [k for k, b in enumerate(buffers) if b >= n_in][0]
        j = buffers[k_out] - n_in
        in_ops = [k for k in range(len(buffers)) if k != k_out]
        subs = list(stp.operand_subscripts)
        formula = ",".join([stp.coefficient_subscripts] + ["Z" + subs[k] for k in in_ops]) + "->Z" + subs[k_out]
        views = {k: _segments(xs[buffers[k]], stp.operands[k]) for k in in_ops}
        out_op = stp.operands[k_out]
        rows = max([xs[buffers[k]].shape[0] for k in in_ops] + [1])
        out = np.zeros((rows, out_op.size))
        offs = out_op.offsets()
        for path in stp.paths:
            segs = []
            for k in in_ops:
                s = views[k][path.indices[k]]
                segs.append(np.broadcast_to(s, (rows,) + s.shape[1:]))
            if segs:
                r = np.einsum(formula, np.asarray(path.coefficients, dtype=np.float64), *segs)
            else:  # a product without inputs is the constant given by its coefficients
                r = np.asarray(path.coefficients, dtype=np.float64).reshape(1, -1)
            o = offs[path.indices[k_out]]
            out[:, o : o + r[0].size] += r.reshape(rows, -1)
        want = output_rows.get(j, batch)
        if j in output_indices:
            idx = np.asarray(output_indices[j], dtype=np.int64)
            if out.shape[0] == 1 and idx.shape[0] > 1:
                out = np.broadcast_to(out, (idx.shape[0], out.shape[1]))
            val = np.zeros((want, out.shape[1]))
            np.add.at(val, idx, out)
        elif want == out.shape[0]:
            val = out
        elif want == 1:
            val = out.sum(axis=0, keepdims=True)
        elif out.shape[0] == 1:
            val = np.broadcast_to(out, (want, out.shape[1])).copy()
        else:
            raise ValueError("batch mismatch")
        results[j] = val if results[j] is None else results[j] + val
    for j, r in enumerate(results):
        if r is None:
            results[j] = np.zeros((output_rows.get(j, batch), poly.outputs[j].size))
    return results

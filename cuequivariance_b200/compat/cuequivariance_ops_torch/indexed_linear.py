"""``indexed_linear`` of the closed package, on this library.

The reference front-end reaches it from ``method="indexed_linear"``
(cuequivariance_torch/primitives/segmented_polynomial_indexed_linear.py:116-156): after sorting rows by class
it calls

    indexed_linear(input1, input2, counts, u, v, C, Z, subscripts, coefficient)

where exactly one of the three tensors (two inputs, the result) is a stack of ``C`` matrices and the other two
are ``Z`` rows; ``counts[c]`` consecutive rows belong to class ``c``; ``subscripts`` names the axes of
(input1, input2, result) with the letters ``u`` and ``v`` (the table of the six accepted triples is at :345-398
of that file and, with the argument order spelled out, in
cuequivariance_jax/segmented_polynomials/segmented_polynomial_indexed_linear.py:218-400):

    ("uv", "u", "v") / ("uv", "v", "u")    result[z] = coefficient * input1[class(z)] contracted with input2[z]
    ("u", "uv", "v") / ("u", "vu", "v")    result[z] = coefficient * input1[z] contracted with input2[class(z)]
    ("u", "v", "uv") / ("u", "v", "vu")    result[c] = coefficient * sum over the rows of class c of input1[z] (x) input2[z]

The result is differentiable to any order: each case is one bilinear polynomial evaluated by this library's
``SegmentedPolynomial`` (``uv,iu,iv`` with the class index on the matrix operand, or its transpose with the class
index on the result), so derivatives are again polynomials on the same CUDA kernels.  float32 and float64.
"""
from __future__ import annotations

from functools import lru_cache
from typing import Sequence

import torch

from cuequivariance_b200.polynomial import Polynomial
from cuequivariance_b200.stp import SegmentedTensorProduct


@lru_cache(maxsize=64)
def _rows_times_matrices(k: int, n: int, coefficient: float):
    """``(W [C, k*n], x [Z, k], class ids) -> [Z, n]``."""
    from cuequivariance_b200.segmented_polynomial import SegmentedPolynomial

    d = SegmentedTensorProduct.from_subscripts("uv,iu,iv")
    d.add_segment(1, (1, k))
    d.add_segment(2, (1, n))
    d.add_path(None, 0, 0, c=coefficient, dims={"u": k, "v": n})
    return SegmentedPolynomial(Polynomial.eval_last_operand(d), method="fused_tp", name="indexed_linear")


@lru_cache(maxsize=64)
def _rows_outer(a: int, b: int, coefficient: float):
    """``(x [Z, a], y [Z, b], class ids, C) -> [C, a*b]``: per class the sum of the rows' outer products."""
    from cuequivariance_b200.segmented_polynomial import SegmentedPolynomial

    d = SegmentedTensorProduct.from_subscripts("iu,iv,uv")
    d.add_segment(0, (1, a))
    d.add_segment(1, (1, b))
    d.add_path(0, 0, None, c=coefficient, dims={"u": a, "v": b})
    return SegmentedPolynomial(Polynomial.eval_last_operand(d), method="fused_tp", name="indexed_linear_outer")


def _class_ids(counts: torch.Tensor, rows: int) -> torch.Tensor:
    counts = counts.to(torch.int64)
    ids = torch.repeat_interleave(torch.arange(counts.shape[0], device=counts.device, dtype=torch.int32), counts)
    if ids.shape[0] != rows:
        raise ValueError(f"indexed_linear: counts sum to {ids.shape[0]} but there are {rows} rows")
    return ids


def indexed_linear(input1: torch.Tensor, input2: torch.Tensor, counts: torch.Tensor, u: int, v: int, C: int, Z: int,
                   subscripts: Sequence[str], coefficient, math_dtype=None) -> torch.Tensor:
    sa, sb, so = (str(s) for s in subscripts)
    if sorted(map(len, (sa, sb, so))) != [1, 1, 2] or set(sa + sb + so) != {"u", "v"}:
        raise ValueError(f"indexed_linear: unsupported subscripts {tuple(subscripts)}")
    if not (input1.is_cuda and input2.is_cuda):
        raise RuntimeError("indexed_linear needs CUDA tensors (there is no CPU fallback)")
    dim = {"u": int(u), "v": int(v)}
    c = float(coefficient)
    C, Z = int(C), int(Z)
    if counts.shape[0] != C:
        raise ValueError(f"indexed_linear: {C} classes but {counts.shape[0]} counts")
    ids = _class_ids(counts, Z)
    if len(so) == 2:                                    # rows (x) rows -> one matrix per class
        x, y = input1.reshape(Z, dim[sa]), input2.reshape(Z, dim[sb])
        first, second = (x, y) if so == sa + sb else (y, x)
        f = _rows_outer(first.shape[1], second.shape[1], c)
        (out,) = f([first, second], {}, {0: torch.empty((C, 1), device=x.device)}, {0: ids})
        return out.reshape(C, dim[so[0]], dim[so[1]])
    mats, rows, sm, sr = (input1, input2, sa, sb) if len(sa) == 2 else (input2, input1, sb, sa)
    if sr == so or sr not in sm:
        raise ValueError(f"indexed_linear: unsupported subscripts {tuple(subscripts)}")
    W = mats.reshape(C, dim[sm[0]], dim[sm[1]])
    if sm != sr + so:                                   # bring the contracted axis first
        W = W.transpose(1, 2)
    k, n = dim[sr], dim[so]
    f = _rows_times_matrices(k, n, c)
    (out,) = f([W.reshape(C, k * n), rows.reshape(Z, k)], {0: ids}, {}, {})
    return out

"""``FusedTensorProductOp3`` / ``FusedTensorProductOp4`` of the closed package, on this library.

The reference front-end builds one of these per operation of a polynomial
(cuequivariance_torch/primitives/segmented_polynomial_fused_tp.py:27-72) after its ``dispatch``
step has brought the tensor product into one of eleven mode patterns (:114-129; algorithm in
cuequivariance/segmented_polynomials/dispatch.py:23-92).  Constructor arguments, as passed at
that call site: the mode string of every operand (output last), per operand the element offset
and the shape of every segment, ``path_indices`` ``[num_paths, num_operands]`` and
``path_coefficients`` (scalars after dispatch, stacked ``[num_paths]``), and ``math_dtype``
(float32 or float64).  ``op(in0, in1[, in2])`` returns ``[batch, output size]``; inputs with
one row are shared over the batch.

Here the lists become a one-operation polynomial evaluated by ``method="fused_tp"`` of this
library, so all eleven patterns run on its CUDA kernels: multi-mode operands are flattened
onto the generic uniform-1d kernel, and the dense ``u,v,uvw,w`` pattern at sizes where that
flattening explodes is first re-coupled into ``uvw,iu,jv,kw+ijk`` (the scalar paths that share
a weight segment are the non-zero entries of one coupling tensor) and then takes the
tensor-core kernels.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from cuequivariance_b200.polynomial import Operation, Polynomial
from cuequivariance_b200.stp import Operand, Path, SegmentedTensorProduct


def _product(modes, offsets, shapes, indices, coefficients) -> SegmentedTensorProduct:
    modes = tuple(str(m) for m in modes)
    operands = []
    for m, offs, shp in zip(modes, offsets, shapes):
        op = Operand(len(m), tuple(tuple(int(v) for v in s) for s in shp))
        if [int(o) for o in offs] != op.offsets():
            raise ValueError("FusedTensorProductOp: segments must be stored back to back in operand order")
        operands.append(op)
    indices = np.asarray(indices, dtype=np.int64).reshape(-1, len(modes))
    coefficients = np.asarray(coefficients, dtype=np.float64)
    if coefficients.shape != (indices.shape[0],):
        raise ValueError("FusedTensorProductOp: one scalar coefficient per path is expected")
    paths = [Path(tuple(int(i) for i in row), np.float64(c)) for row, c in zip(indices, coefficients)]
    return SegmentedTensorProduct(modes, "", operands, paths)


def _blocks(groups: Sequence[frozenset], n: int) -> Optional[List[List[int]]]:
    """The partition of segments 0..n-1 induced by ``groups`` if every group is a run of
    consecutive segments and two groups are equal or disjoint; segments in no group stay alone."""
    owner = {}
    for g in set(groups):
        s = sorted(g)
        if s != list(range(s[0], s[0] + len(s))) or any(i in owner for i in s):
            return None
        for i in s:
            owner[i] = s[0]
    out, i = [], 0
    while i < n:
        blk = [j for j in range(n) if owner.get(j, j) == owner.get(i, i)] if i in owner else [i]
        out.append(blk)
        i = blk[-1] + 1
    return out


def recouple_dense(d: SegmentedTensorProduct) -> Optional[SegmentedTensorProduct]:
    """``u,v,uvw,w`` with scalar coefficients -> ``uvw,iu,jv,kw+ijk`` (operands w, x1, x2, out),
    or None when the paths do not have that structure."""
    if d.operand_subscripts != ("u", "v", "uvw", "w") or d.coefficient_subscripts:
        return None
    x1, x2, w, out = d.operands
    by_w: dict = {}
    for p in d.paths:
        by_w.setdefault(p.indices[2], []).append(p)
    b1 = _blocks([frozenset(p.indices[0] for p in ps) for ps in by_w.values()], x1.num_segments)
    b2 = _blocks([frozenset(p.indices[1] for p in ps) for ps in by_w.values()], x2.num_segments)
    b3 = _blocks([frozenset(p.indices[3] for p in ps) for ps in by_w.values()], out.num_segments)
    if b1 is None or b2 is None or b3 is None:
        return None

    def merged(op, blocks):
        segs = []
        for blk in blocks:
            shapes = {op.segments[i] for i in blk}
            if len(shapes) != 1:
                return None
            segs.append((len(blk),) + tuple(shapes.pop()))
        return Operand(2, tuple(segs))

    m1, m2, m3 = merged(x1, b1), merged(x2, b2), merged(out, b3)
    if m1 is None or m2 is None or m3 is None:
        return None
    where = [{i: (n, blk.index(i)) for n, blk in enumerate(bl) for i in blk} for bl in (b1, b2, b3)]
    paths = []
    for sw, ps in sorted(by_w.items()):
        n1, n2, n3 = where[0][ps[0].indices[0]][0], where[1][ps[0].indices[1]][0], where[2][ps[0].indices[3]][0]
        c = np.zeros((len(b1[n1]), len(b2[n2]), len(b3[n3])))
        for p in ps:
            (a, i), (b, j), (o, k) = where[0][p.indices[0]], where[1][p.indices[1]], where[2][p.indices[3]]
            if (a, b, o) != (n1, n2, n3):
                return None
            c[i, j, k] += float(p.coefficients)
        if w.segments[sw] != (m1.segments[n1][1], m2.segments[n2][1], m3.segments[n3][1]):
            return None
        paths.append(Path((sw, n1, n2, n3), c))
    return SegmentedTensorProduct(("uvw", "iu", "jv", "kw"), "ijk", [w, m1, m2, m3], paths)


class _FusedTensorProductOp(torch.nn.Module):
    def __init__(self, operand_segment_modes, operand_segment_offsets, operand_segment_shapes, path_indices,
                 path_coefficients, math_dtype: torch.dtype = torch.float32):
        super().__init__()
        import cuequivariance_b200 as cb
        from cuequivariance_b200.fused_tp import FLATTEN_LIMIT, flattened_path_count

        d = _product(operand_segment_modes, operand_segment_offsets, operand_segment_shapes, path_indices, path_coefficients)
        n = d.num_operands
        if n != self.NUM_OPERANDS:
            raise ValueError(f"{type(self).__name__} takes {self.NUM_OPERANDS} operands, got {n}")
        self.order = list(range(n - 1))
        poly = Polynomial(d.operands[:-1], d.operands[-1:], [(Operation(tuple(range(n))), d)])
        if n == 4 and flattened_path_count(poly) > FLATTEN_LIMIT:
            dense = recouple_dense(d)
            if dense is not None:
                poly = Polynomial(dense.operands[:3], dense.operands[3:], [(Operation((0, 1, 2, 3)), dense)])
                self.order = [2, 0, 1]   # this library's operand order is (w, x1, x2)
        self.f = cb.SegmentedPolynomial(poly, method="fused_tp", math_dtype=math_dtype)

    def forward(self, *inputs: torch.Tensor) -> torch.Tensor:
        return self.f([inputs[i] for i in self.order])[0]


class FusedTensorProductOp3(_FusedTensorProductOp):
    NUM_OPERANDS = 3


class FusedTensorProductOp4(_FusedTensorProductOp):
    NUM_OPERANDS = 4

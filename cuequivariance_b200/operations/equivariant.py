"""`EquivariantTensorProduct`: evaluates an `EquivariantPolynomial` with layout handling.

The reference removed its torch class of this name (its stub raises with migration
advice, cuequivariance_torch/primitives/deprecated.py:25-96); this thin working version
wraps `SegmentedPolynomial` with the layout transpositions of every operand, which is what
the operation modules do individually.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..descriptors import EquivariantPolynomial
from ..irreps import IrrepsLayout
from ..segmented_polynomial import SegmentedPolynomial
from ..transpose import TransposeIrrepsLayout


class EquivariantTensorProduct(torch.nn.Module):
    def __init__(self, e: EquivariantPolynomial, *, layout=None, layout_in: Optional[Sequence] = None,
                 layout_out=None, device=None, math_dtype=None, method: str = "uniform_1d"):
        super().__init__()
        self.e = e
        n_in = len(e.inputs)
        if layout_in is None or not isinstance(layout_in, (list, tuple)):
            layout_in = [layout_in or layout] * n_in
        self.transpose_in = torch.nn.ModuleList(
            TransposeIrrepsLayout(r.irreps, source=IrrepsLayout.parse(l), target=r.layout, device=device)
            for r, l in zip(e.inputs, layout_in)
        )
        self.transpose_out = torch.nn.ModuleList(
            TransposeIrrepsLayout(r.irreps, source=r.layout, target=IrrepsLayout.parse(layout_out or layout), device=device)
            for r in e.outputs
        )
        self.f = SegmentedPolynomial(e.polynomial, method=method, math_dtype=math_dtype)

    def forward(self, *inputs, indices=None, indices_out=None, size_out=None):
        xs = [t(x) for t, x in zip(self.transpose_in, inputs)]
        kw = {}
        if indices:
            kw["input_indices"] = dict(indices)
        if indices_out is not None:
            kw["output_indices"] = {0: indices_out}
            kw["output_shapes"] = {0: torch.empty(size_out, 1, device=xs[0].device)}
        outs = self.f(xs, **kw)
        outs = [t(o) for t, o in zip(self.transpose_out, outs)]
        return outs[0] if len(outs) == 1 else outs

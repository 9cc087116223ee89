"""`SymmetricContraction`: same surface as the reference module
(cuequivariance_torch/operations/symmetric_contraction.py:32-242)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import descriptors
from ..irreps import Irreps, IrrepsLayout
from ..segmented_polynomial import SegmentedPolynomial
from ..transpose import TransposeIrrepsLayout


class SymmetricContraction(torch.nn.Module):
    """Weighted sum of symmetric powers ``x, x(x)x, ..., x^(x)degree`` of the input,
    projected on ``irreps_out``, with one weight set per element (species).

    ``forward(x[batch, irreps_in.dim], indices[batch]) -> [batch, irreps_out.dim]``.
    ``weight`` has shape ``(num_elements, weight_numel // mul, mul)``.
    """

    def __init__(
        self,
        irreps_in,
        irreps_out,
        contraction_degree: int,
        num_elements: int,
        *,
        layout=None,
        layout_in=None,
        layout_out=None,
        device: Optional[torch.device] = None,
        dtype: Optional[torch.dtype] = None,
        math_dtype=None,
        original_mace: bool = False,
        use_fallback: Optional[bool] = None,
        method: Optional[str] = None,
    ):
        super().__init__()
        if use_fallback:
            raise ValueError("cuequivariance_b200 has no fallback implementation (use_fallback must be None or False)")
        irreps_in = irreps_in if isinstance(irreps_in, Irreps) else Irreps(irreps_in)
        irreps_out = irreps_out if isinstance(irreps_out, Irreps) else Irreps(irreps_in.group, irreps_out)
        if len(set(irreps_in.muls) | set(irreps_out.muls)) != 1:
            raise ValueError("Input/Output irreps must have the same mul")
        mul = irreps_in.muls[0]
        self.irreps_in, self.irreps_out = irreps_in, irreps_out
        self.contraction_degree = contraction_degree
        self.etp, p = descriptors.symmetric_contraction(irreps_in, irreps_out, tuple(range(1, contraction_degree + 1)))
        if original_mace:
            if p is None:
                raise NotImplementedError("original_mace=True needs the projection from original-MACE weights, which exists only "
                                          "for the shapes with a reference table (inputs 0e[+1o[+2e[+3o]]], outputs 0e[+1o[+2e]], degree <= 3)")
            self.register_buffer("projection", torch.tensor(p, dtype=dtype, device=device))
            self.weight_shape = (p.shape[0], mul)
        else:
            self.projection = None
            self.weight_shape = (self.etp.inputs[0].dim // mul, mul)
        self.num_elements = num_elements
        self.weight = torch.nn.Parameter(torch.randn(num_elements, *self.weight_shape, device=device, dtype=dtype))
        if method not in (None, "uniform_1d"):
            raise ValueError(f"method {method!r} is not available for SymmetricContraction (only 'uniform_1d')")
        self.method = "uniform_1d"
        self.transpose_in = TransposeIrrepsLayout(irreps_in, source=IrrepsLayout.parse(layout_in or layout), target=self.etp.inputs[1].layout, device=device)
        self.transpose_out = TransposeIrrepsLayout(irreps_out, source=self.etp.outputs[0].layout, target=IrrepsLayout.parse(layout_out or layout), device=device)
        self.f = SegmentedPolynomial(self.etp.polynomial, method=self.method, math_dtype=math_dtype, name="symmetric_contraction")

    def extra_repr(self) -> str:
        return f"contraction_degree={self.contraction_degree}, weight_shape={self.weight_shape}"

    def forward(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        if self.projection is not None:
            weight = torch.einsum("zau,ab->zbu", self.weight, self.projection)
        else:
            weight = self.weight
        out = self.f([weight.flatten(1), self.transpose_in(x)], input_indices={0: indices})
        return self.transpose_out(out[0])

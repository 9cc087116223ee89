"""`Linear`: same surface as the reference module
(cuequivariance_torch/operations/linear.py:30-191) - an equivariant linear map with one dense
``[mul_in, mul_out]`` block per irrep present on both sides, optionally one weight set per class
selected by ``weight_indices``."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import descriptors
from ..irreps import Irreps, IrrepsLayout
from ..segmented_polynomial import SegmentedPolynomial
from ..transpose import TransposeIrrepsLayout


class Linear(torch.nn.Module):
    """``forward(x, weight=None, weight_indices=None)``; ``x``: ``[batch, irreps_in.dim]``;
    ``weight``: ``[1 or weight_classes, weight_numel]`` when shared (the module's own parameter
    when ``internal_weights``), ``[batch, weight_numel]`` otherwise; ``weight_indices``:
    ``[batch]`` class ids, required when ``weight_classes > 1``.

    Executed by the CUDA executor on the polynomial ``uv,iu,iv`` flattened over ``u`` (the generic
    kernel; a dense tensor-core route for large multiplicities is not written yet).  There is no
    ``naive`` method and no fallback."""

    def __init__(
        self,
        irreps_in,
        irreps_out,
        *,
        layout=None,
        layout_in=None,
        layout_out=None,
        shared_weights: bool = True,
        internal_weights: bool = None,
        weight_classes: Optional[int] = 1,
        device: Optional[torch.device] = None,
        dtype: Optional[torch.dtype] = None,
        math_dtype=None,
        use_fallback: Optional[bool] = None,
        method: Optional[str] = None,
    ):
        super().__init__()
        if use_fallback:
            raise ValueError("cuequivariance_b200 has no fallback implementation (use_fallback must be None or False)")
        irreps_in = irreps_in if isinstance(irreps_in, Irreps) else Irreps(irreps_in)
        irreps_out = irreps_out if isinstance(irreps_out, Irreps) else Irreps(irreps_in.group, irreps_out)
        e = descriptors.linear(irreps_in, irreps_out)
        self.irreps_in, self.irreps_out = irreps_in, irreps_out
        self.weight_numel = e.polynomial.inputs[0].size
        self.weight_classes = weight_classes
        self.shared_weights = shared_weights
        if weight_classes > 1 and not shared_weights:
            raise ValueError("Weight classes require shared weights.")
        self.internal_weights = internal_weights if internal_weights is not None else shared_weights
        if self.internal_weights:
            if not self.shared_weights:
                raise ValueError("Internal weights should be shared")
            self.weight = torch.nn.Parameter(torch.randn(weight_classes, self.weight_numel, device=device, dtype=dtype))
        else:
            self.weight = None
        if method not in (None, "fused_tp"):
            raise ValueError(f"method {method!r} is not available for Linear (only 'fused_tp')")
        self.method = "fused_tp"
        self.transpose_in = TransposeIrrepsLayout(irreps_in, source=IrrepsLayout.parse(layout_in or layout), target=e.inputs[1].layout, device=device)
        self.transpose_out = TransposeIrrepsLayout(irreps_out, source=e.outputs[0].layout, target=IrrepsLayout.parse(layout_out or layout), device=device)
        if math_dtype is None and dtype in (torch.float32, torch.float64):
            math_dtype = dtype
        self.f = SegmentedPolynomial(e.polynomial, method=self.method, math_dtype=math_dtype, name="linear")

    def extra_repr(self) -> str:
        return (f"shared_weights={self.shared_weights}, internal_weights={self.internal_weights}, "
                f"weight_numel={self.weight_numel}, weight_classes={self.weight_classes}")

    def forward(self, x: torch.Tensor, weight: Optional[torch.Tensor] = None, weight_indices: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.weight is not None:
            if weight is not None:
                raise ValueError("Internal weights are used, weight should be None")
            weight = self.weight
        input_indices: Dict[int, torch.Tensor] = {}
        if self.weight_classes > 1:
            if weight_indices is None:
                raise ValueError("weight_indices should be provided if weight_classes > 1")
            input_indices[0] = weight_indices
        if weight is None:
            raise ValueError("Weights should not be None")
        out = self.f([weight, self.transpose_in(x)], input_indices=input_indices)
        return self.transpose_out(out[0])

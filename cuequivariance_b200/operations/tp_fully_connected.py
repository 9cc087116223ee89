"""`FullyConnectedTensorProduct`: same surface as the reference module
(cuequivariance_torch/operations/tp_fully_connected.py:30-207)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import descriptors
from ..irreps import Irreps, IrrepsLayout
from ..segmented_polynomial import SegmentedPolynomial
from ..transpose import TransposeIrrepsLayout


class FullyConnectedTensorProduct(torch.nn.Module):
    """Fully connected ("uvw") tensor product ``x1 (x) x2 -> out`` with a weight per
    (u, v, w) and allowed irrep triple."""

    def __init__(
        self,
        irreps_in1,
        irreps_in2,
        irreps_out,
        *,
        layout=None,
        layout_in1=None,
        layout_in2=None,
        layout_out=None,
        shared_weights: bool = True,
        internal_weights: bool = None,
        device: Optional[torch.device] = None,
        dtype: Optional[torch.dtype] = None,
        math_dtype=None,
        use_fallback: Optional[bool] = None,
        method: Optional[str] = None,
        options: Optional[dict] = None,
    ):
        """``options={"tensor_cores": True}`` sends float32 inputs through the bf16 tensor-core
        route as well (bf16/fp16 inputs always take it when the shapes allow)."""
        super().__init__()
        if use_fallback:
            raise ValueError("cuequivariance_b200 has no fallback implementation (use_fallback must be None or False)")
        irreps_in1 = irreps_in1 if isinstance(irreps_in1, Irreps) else Irreps(irreps_in1)
        irreps_in2 = irreps_in2 if isinstance(irreps_in2, Irreps) else Irreps(irreps_in1.group, irreps_in2)
        irreps_out = irreps_out if isinstance(irreps_out, Irreps) else Irreps(irreps_in1.group, irreps_out)
        e = descriptors.fully_connected_tensor_product(irreps_in1, irreps_in2, irreps_out)
        self.irreps_in1, self.irreps_in2, self.irreps_out = irreps_in1, irreps_in2, irreps_out
        self.weight_numel = e.polynomial.inputs[0].size
        self.shared_weights = shared_weights
        self.internal_weights = internal_weights if internal_weights is not None else shared_weights
        if self.internal_weights:
            if not self.shared_weights:
                raise ValueError("Internal weights should be shared")
            self.weight = torch.nn.Parameter(torch.randn(1, self.weight_numel, device=device, dtype=dtype))
        else:
            self.weight = None
        if method not in (None, "fused_tp"):
            raise ValueError(f"method {method!r} is not available for FullyConnectedTensorProduct (only 'fused_tp')")
        self.method = "fused_tp"
        self.transpose_in1 = TransposeIrrepsLayout(irreps_in1, source=IrrepsLayout.parse(layout_in1 or layout), target=e.inputs[1].layout, device=device)
        self.transpose_in2 = TransposeIrrepsLayout(irreps_in2, source=IrrepsLayout.parse(layout_in2 or layout), target=e.inputs[2].layout, device=device)
        self.transpose_out = TransposeIrrepsLayout(irreps_out, source=e.outputs[0].layout, target=IrrepsLayout.parse(layout_out or layout), device=device)
        if math_dtype is None and dtype in (torch.float32, torch.float64):
            math_dtype = dtype
        self.f = SegmentedPolynomial(e.polynomial, method=self.method, math_dtype=math_dtype, name="fully_connected_tensor_product",
                                     options=options)

    def extra_repr(self) -> str:
        return f"shared_weights={self.shared_weights}, internal_weights={self.internal_weights}, weight_numel={self.weight_numel}"

    def forward(self, x1: torch.Tensor, x2: torch.Tensor, weight: Optional[torch.Tensor] = None) -> torch.Tensor:
        x1 = self.transpose_in1(x1)
        x2 = self.transpose_in2(x2)
        if self.weight is not None:
            if weight is not None:
                raise ValueError("Internal weights are used, weight should be None")
            weight = self.weight
        elif weight is None:
            raise ValueError("Internal weights are not used, weight should not be None")
        return self.transpose_out(self.f([weight, x1, x2])[0])

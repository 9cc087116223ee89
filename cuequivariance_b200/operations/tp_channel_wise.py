"""`ChannelWiseTensorProduct`: same surface as the reference module
(cuequivariance_torch/operations/tp_channel_wise.py:30-258)."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import descriptors
from ..irreps import Irreps, IrrepsLayout
from ..segmented_polynomial import SegmentedPolynomial


class ChannelWiseTensorProduct(torch.nn.Module):
    """Channel-wise ("uvu") tensor product with optional fused gather of ``x1``/``x2`` and
    scatter-add of the output.

    Args mirror the reference: ``irreps_in1``, ``irreps_in2``, ``filter_irreps_out``,
    ``layout`` (+ per-operand overrides, default ``mul_ir``), ``shared_weights`` (default
    True), ``internal_weights`` (default = ``shared_weights``), ``device``, ``dtype``,
    ``math_dtype``, ``method`` (``"uniform_1d"`` only).
    """

    def __init__(
        self,
        irreps_in1,
        irreps_in2,
        filter_irreps_out: Sequence = None,
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
    ):
        super().__init__()
        if use_fallback:
            raise ValueError("cuequivariance_b200 has no fallback implementation (use_fallback must be None or False)")
        irreps_in1 = irreps_in1 if isinstance(irreps_in1, Irreps) else Irreps(irreps_in1)
        irreps_in2 = irreps_in2 if isinstance(irreps_in2, Irreps) else Irreps(irreps_in1.group, irreps_in2)
        if irreps_in1.group != irreps_in2.group:
            raise ValueError("irreps_in1 and irreps_in2 must belong to the same group")
        e = descriptors.channelwise_tensor_product(irreps_in1, irreps_in2, filter_irreps_out)
        self.irreps_in1, self.irreps_in2 = irreps_in1, irreps_in2
        self.irreps_out = e.outputs[0].irreps
        self.weight_numel = e.polynomial.inputs[0].size
        self.shared_weights = shared_weights
        self.internal_weights = internal_weights if internal_weights is not None else shared_weights
        if self.internal_weights:
            if not self.shared_weights:
                raise ValueError("Internal weights should be shared")
            self.weight = torch.nn.Parameter(torch.randn(1, self.weight_numel, device=device, dtype=dtype))
        else:
            self.weight = None
        if method not in (None, "uniform_1d"):
            raise ValueError(f"method {method!r} is not available for ChannelWiseTensorProduct (only 'uniform_1d')")
        self.method = "uniform_1d"
        # layouts are handed to the executor, which folds them into kernel addressing when it
        # can and transposes explicitly otherwise (the reference always transposes,
        # tp_channel_wise.py:221-222,258)
        self._layouts = {}
        for b, (irreps, lay) in {1: (irreps_in1, layout_in1 or layout), 2: (irreps_in2, layout_in2 or layout),
                                 3: (self.irreps_out, layout_out or layout)}.items():
            if IrrepsLayout.parse(lay) is IrrepsLayout.mul_ir:
                self._layouts[b] = tuple((mul, ir.dim) for mul, ir in irreps)
        self.f = SegmentedPolynomial(e.polynomial, method=self.method, math_dtype=math_dtype, name="channelwise_tensor_product")

    def extra_repr(self) -> str:
        return f"shared_weights={self.shared_weights}, internal_weights={self.internal_weights}, weight_numel={self.weight_numel}"

    def forward(
        self,
        x1: torch.Tensor,
        x2: torch.Tensor,
        weight: Optional[torch.Tensor] = None,
        indices_1: Optional[torch.Tensor] = None,
        indices_2: Optional[torch.Tensor] = None,
        indices_out: Optional[torch.Tensor] = None,
        size_out: Optional[int] = None,
    ) -> torch.Tensor:
        indices_in: Dict[int, torch.Tensor] = {}
        if indices_1 is not None:
            indices_in[1] = indices_1
        if indices_2 is not None:
            indices_in[2] = indices_2
        idx_out: Dict[int, torch.Tensor] = {}
        sizes_out: Dict[int, torch.Tensor] = {}
        if indices_out is not None:
            if size_out is None:
                raise ValueError("size_out should be provided if indices_out is provided")
            idx_out = {0: indices_out}
            sizes_out = {0: torch.empty(size_out, 1, device=x1.device)}
        if self.weight is not None:
            if weight is not None:
                raise ValueError("Internal weights are used, weight should be None")
            weight = self.weight
        elif weight is None:
            raise ValueError("Internal weights are not used, weight should not be None")
        out = self.f([weight, x1, x2], input_indices=indices_in, output_shapes=sizes_out, output_indices=idx_out,
                     layouts=self._layouts)
        return out[0]

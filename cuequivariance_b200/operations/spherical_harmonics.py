"""`SphericalHarmonics`: same surface as the reference module
(cuequivariance_torch/operations/spherical_harmonics.py:26-93)."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from .. import descriptors
from ..irreps import Irrep
from ..segmented_polynomial import SegmentedPolynomial


class SphericalHarmonics(nn.Module):
    """Real spherical harmonics of 3-vectors, component-normalised (|Y_l|^2 = 2l+1 on the
    unit sphere); with ``normalize=True`` the vectors are first divided by their norm."""

    def __init__(self, ls: List[int], normalize: bool = True, device: Optional[torch.device] = None,
                 math_dtype=None, use_fallback: Optional[bool] = None, method: Optional[str] = None):
        super().__init__()
        if use_fallback or method not in (None, "uniform_1d"):
            raise ValueError("SphericalHarmonics runs with method 'uniform_1d' only")
        self.ls = list(ls)
        if self.ls != sorted(set(self.ls)):
            raise ValueError("ls must be sorted and unique")
        self.normalize = normalize
        e = descriptors.spherical_harmonics(Irrep(1, -1), self.ls)
        self.f = SegmentedPolynomial(e.polynomial, method="uniform_1d", math_dtype=math_dtype, name="spherical_harmonics")

    def forward(self, vectors: torch.Tensor) -> torch.Tensor:
        torch._assert(vectors.ndim == 2, "input must have shape (batch, 3)")
        if self.normalize:
            vectors = torch.nn.functional.normalize(vectors, dim=1)
        return self.f([vectors])[0]


def spherical_harmonics(ls: List[int], vectors: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    return SphericalHarmonics(ls, normalize)(vectors)

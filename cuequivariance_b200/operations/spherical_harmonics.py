"""`SphericalHarmonics`: same surface as the reference module
(cuequivariance_torch/operations/spherical_harmonics.py:26-93)."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from .. import descriptors
from ..irreps import Irrep
from ..segmented_polynomial import SegmentedPolynomial


FUSED = True       # degrees 0..4, float32/float64 CUDA tensors: the fused kernels (normalisation included)
FUSED_LMAX = 4


def _launch(which: str, vec, y, gvec, mask: int, normalize: bool):
    import ctypes as C

    from .. import _lib, profiling

    a = _lib.ShArgs()
    a.vec, a.y = vec.data_ptr(), y.data_ptr()
    a.gvec = gvec.data_ptr() if gvec is not None else None
    a.rows, a.ld_vec, a.ld_y = vec.shape[0], vec.stride(0), y.stride(0)
    a.ld_gvec = gvec.stride(0) if gvec is not None else 0
    a.ls_mask, a.normalize = mask, 1 if normalize else 0
    a.dtype = _lib.F32 if vec.dtype == torch.float32 else _lib.F64
    fn = _lib.lib().cueq_b200_sh_forward if which == "forward" else _lib.lib().cueq_b200_sh_backward
    with torch.cuda.device(vec.device), profiling.kernel(f"sh_fused_{which}"):
        _lib.check(fn(C.byref(a), C.c_void_p(torch.cuda.current_stream(vec.device).cuda_stream)))


class _FusedSH(torch.autograd.Function):
    """Forward and first derivative on the fused kernels.  When the derivative itself has to be
    differentiable (``create_graph=True``, e.g. forces inside a training loss) the backward pass is
    evaluated through the polynomial executor instead, which is differentiable to any order."""

    @staticmethod
    def forward(ctx, module, vec):
        vec_c = vec.contiguous()
        out = torch.empty((vec.shape[0], module.width), dtype=vec.dtype, device=vec.device)
        _launch("forward", vec_c, out, None, module.mask, module.normalize)
        ctx.module = module
        ctx.save_for_backward(vec)
        return out

    @staticmethod
    def backward(ctx, g):
        (vec,) = ctx.saved_tensors
        module = ctx.module
        if torch.is_grad_enabled():
            with torch.enable_grad():
                y = module._polynomial_route(vec)
                (gv,) = torch.autograd.grad(y, vec, g, create_graph=True)
            return None, gv
        gv = torch.empty((vec.shape[0], 3), dtype=vec.dtype, device=vec.device)
        _launch("backward", vec.contiguous(), g.contiguous(), gv, module.mask, module.normalize)
        return None, gv


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
        self.math_dtype = self.f.math_dtype
        self.mask = sum(1 << l for l in self.ls) if self.ls and max(self.ls) <= FUSED_LMAX else 0  # noqa: E741
        self.width = sum(2 * l + 1 for l in self.ls)  # noqa: E741

    def _polynomial_route(self, vectors: torch.Tensor) -> torch.Tensor:
        if self.normalize:
            vectors = torch.nn.functional.normalize(vectors, dim=1)
        return self.f([vectors])[0]

    def forward(self, vectors: torch.Tensor) -> torch.Tensor:
        torch._assert(vectors.ndim == 2, "input must have shape (batch, 3)")
        if (FUSED and self.mask and vectors.is_cuda and vectors.shape[1] == 3 and vectors.dtype in (torch.float32, torch.float64)
                and self.math_dtype in (None, vectors.dtype)):
            return _FusedSH.apply(self, vectors)
        return self._polynomial_route(vectors)


def spherical_harmonics(ls: List[int], vectors: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    return SphericalHarmonics(ls, normalize)(vectors)

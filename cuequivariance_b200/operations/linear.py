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


DENSE_ROUTE = True      # float32, one weight set, multiplicities that are multiples of 32: tensor-core GEMMs
DENSE_MIN_ROWS = 256    # below this the generic kernel is used


class _DenseLinear(torch.autograd.Function):
    """``uv,iu,iv`` with one shared weight set as one float32-accurate tensor-core GEMM per
    (path, component): ``out[:, i-th block of the output irrep] = c * x[:, i-th block] @ W``.
    Inputs and outputs are in the descriptor's ir_mul layout, so every block is a column slice."""

    @staticmethod
    def forward(ctx, plan, weight, x):
        from ..dense import gemm_f32x3

        out = torch.zeros((x.shape[0], plan["out_size"]), dtype=torch.float32, device=x.device)
        seen = set()
        for (wo, u, v, xo, oo, d, c) in plan["paths"]:
            wt = (weight[0, wo : wo + u * v].reshape(u, v).t() * c).contiguous()       # [N = v][K = u]
            for i in range(d):
                dst = out[:, oo + i * v : oo + (i + 1) * v]
                if oo in seen:
                    dst += gemm_f32x3(x[:, xo + i * u : xo + (i + 1) * u], wt, name="linear_f32x3")
                else:
                    gemm_f32x3(x[:, xo + i * u : xo + (i + 1) * u], wt, name="linear_f32x3", out=dst)
            seen.add(oo)
        ctx.plan = plan
        ctx.save_for_backward(weight, x)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gout):
        from ..dense import gemm_f32x3, gemm_f32x3_tn

        plan = ctx.plan
        weight, x = ctx.saved_tensors
        gout = gout.contiguous()
        gw = torch.zeros_like(weight) if ctx.needs_input_grad[1] else None
        gx = torch.zeros_like(x) if ctx.needs_input_grad[2] else None
        seen = set()
        for (wo, u, v, xo, oo, d, c) in plan["paths"]:
            if gx is not None:
                wc = (weight[0, wo : wo + u * v].reshape(u, v) * c).contiguous()        # [N = u][K = v]
                for i in range(d):
                    dst = gx[:, xo + i * u : xo + (i + 1) * u]
                    if xo in seen:
                        dst += gemm_f32x3(gout[:, oo + i * v : oo + (i + 1) * v], wc, name="linear_f32x3_gx")
                    else:
                        gemm_f32x3(gout[:, oo + i * v : oo + (i + 1) * v], wc, name="linear_f32x3_gx", out=dst)
                seen.add(xo)
            if gw is not None:
                acc = torch.zeros((u, v), dtype=torch.float32, device=x.device)
                for i in range(d):   # reduction over the rows, component by component, into one accumulator
                    gemm_f32x3_tn(x[:, xo + i * u : xo + (i + 1) * u], gout[:, oo + i * v : oo + (i + 1) * v], out=acc,
                                  name="linear_f32x3_gw")
                gw[0, wo : wo + u * v] += (acc * c).reshape(-1)
        return None, gw, gx


_BOUNDS: list = []   # small cache: (index tensor, version, classes) -> row ranges of the classes


def class_bounds(indices: torch.Tensor, classes: int):
    """Row ranges of the weight classes when ``indices`` is sorted ascending (``[classes + 1]`` python ints),
    else None.  One device-to-host read, cached on the tensor's identity and version counter."""
    for ref, ver, c, val in _BOUNDS:
        if ref is indices and ver == indices._version and c == classes:
            return val
    idx = indices.contiguous()
    edges = torch.searchsorted(idx, torch.arange(classes + 1, device=idx.device, dtype=idx.dtype))
    ok = (idx[1:] >= idx[:-1]).all() if idx.numel() > 1 else torch.ones((), dtype=torch.bool, device=idx.device)
    host = torch.cat([edges.to(torch.int64), ok.to(torch.int64).reshape(1)]).tolist()
    val = host[:-1] if host[-1] else None
    _BOUNDS.append((indices, indices._version, classes, val))
    if len(_BOUNDS) > 8:
        _BOUNDS.pop(0)
    return val


class _GroupedDenseLinear(torch.autograd.Function):
    """Linear map with one weight set per class and rows sorted by class - the counterpart of the reference's
    ``indexed_linear`` method (cuequivariance_torch/primitives/segmented_polynomial_indexed_linear.py:116-156,
    247-339: sorted indices -> counts -> grouped GEMM): class ``c`` owns the contiguous rows
    ``bounds[c] : bounds[c + 1]`` and gets its own GEMM against its own weight block.  Per irrep pair the ``d``
    components of a row are folded into the row axis (``[Z, d, u] -> [Z * d, u]``), so one float32-accurate
    tensor-core GEMM per (class, irrep pair) does the forward, one the input gradient and one (a reduction over
    the class's rows) the weight gradient."""

    @staticmethod
    def forward(ctx, plan, bounds, weight, x):
        from ..dense import gemm_f32x3

        Z = x.shape[0]
        out = torch.zeros((Z, plan["out_size"]), dtype=torch.float32, device=x.device)
        for (wo, u, v, xo, oo, d, c) in plan["paths"]:
            xp = x[:, xo : xo + d * u].reshape(Z * d, u)
            wt = (weight[:, wo : wo + u * v].reshape(-1, u, v).transpose(1, 2) * c).contiguous()     # [class][N = v][K = u]
            op = torch.zeros((Z * d, v), dtype=torch.float32, device=x.device)
            for k in range(len(bounds) - 1):
                r0, r1 = bounds[k] * d, bounds[k + 1] * d
                if r1 > r0:
                    gemm_f32x3(xp[r0:r1], wt[k], name="indexed_linear_f32x3", out=op[r0:r1])
            out[:, oo : oo + d * v] += op.view(Z, d * v)
        ctx.plan, ctx.bounds = plan, bounds
        ctx.save_for_backward(weight, x)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gout):
        from ..dense import gemm_f32x3, gemm_f32x3_tn

        plan, bounds = ctx.plan, ctx.bounds
        weight, x = ctx.saved_tensors
        Z = x.shape[0]
        gw = torch.zeros_like(weight) if ctx.needs_input_grad[2] else None
        gx = torch.zeros_like(x) if ctx.needs_input_grad[3] else None
        for (wo, u, v, xo, oo, d, c) in plan["paths"]:
            gp = gout[:, oo : oo + d * v].reshape(Z * d, v)
            if gx is not None:
                wc = (weight[:, wo : wo + u * v].reshape(-1, u, v) * c).contiguous()                 # [class][N = u][K = v]
                gxp = torch.zeros((Z * d, u), dtype=torch.float32, device=x.device)
            if gw is not None:
                xp = x[:, xo : xo + d * u].reshape(Z * d, u)
            for k in range(len(bounds) - 1):
                r0, r1 = bounds[k] * d, bounds[k + 1] * d
                if r1 <= r0:
                    continue
                if gx is not None:
                    gemm_f32x3(gp[r0:r1], wc[k], name="indexed_linear_f32x3_gx", out=gxp[r0:r1])
                if gw is not None:
                    acc = torch.zeros((u, v), dtype=torch.float32, device=x.device)
                    gemm_f32x3_tn(xp[r0:r1], gp[r0:r1], out=acc, name="indexed_linear_f32x3_gw")
                    gw[k, wo : wo + u * v] += (acc * c).reshape(-1)
            if gx is not None:
                gx[:, xo : xo + d * u] += gxp.view(Z, d * u)
        return None, None, gw, gx


class Linear(torch.nn.Module):
    """``forward(x, weight=None, weight_indices=None)``; ``x``: ``[batch, irreps_in.dim]``;
    ``weight``: ``[1 or weight_classes, weight_numel]`` when shared (the module's own parameter
    when ``internal_weights``), ``[batch, weight_numel]`` otherwise; ``weight_indices``:
    ``[batch]`` class ids, required when ``weight_classes > 1``.

    float32 with one weight set and multiplicities that are multiples of 32 runs as float32-accurate
    tensor-core GEMMs (``dense.gemm_f32x3`` / ``gemm_f32x3_tn``; first derivatives only); everything else
    runs on the generic kernel over the polynomial ``uv,iu,iv``
    flattened over ``u``.  There is no ``naive`` method and no fallback."""

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
        if method not in (None, "fused_tp", "indexed_linear"):
            raise ValueError(f"method {method!r} is not available for Linear ('fused_tp' or 'indexed_linear')")
        # "indexed_linear" (weight classes, rows sorted by class) insists on the grouped tensor-core GEMMs and
        # raises where they do not apply; with the default the grouped route is taken when it applies and the
        # generic kernel otherwise
        self.require_grouped = method == "indexed_linear"
        self.method = "fused_tp"
        self.transpose_in = TransposeIrrepsLayout(irreps_in, source=IrrepsLayout.parse(layout_in or layout), target=e.inputs[1].layout, device=device)
        self.transpose_out = TransposeIrrepsLayout(irreps_out, source=e.outputs[0].layout, target=IrrepsLayout.parse(layout_out or layout), device=device)
        if math_dtype is None and dtype in (torch.float32, torch.float64):
            math_dtype = dtype
        # dense route: every multiplicity a multiple of 32 (K of the forward and of the input gradient)
        _, d = e.polynomial.operations[0]
        offs = [op.offsets() for op in d.operands]
        paths = []
        for p in d.paths:
            sw, si, so = p.indices
            u, v = d.operands[0].segments[sw]
            dim = d.operands[1].segments[si][0]
            paths.append((offs[0][sw], u, v, offs[1][si], offs[2][so], dim, float(p.coefficients)))
        self._dense_plan = None
        if paths and all(u % 32 == 0 and v % 32 == 0 for (_, u, v, _, _, _, _) in paths):
            self._dense_plan = {"paths": paths, "out_size": d.operands[2].size}
        try:
            self.f = SegmentedPolynomial(e.polynomial, method=self.method, math_dtype=math_dtype, name="linear")
            self._generic_error = None
        except ValueError as err:   # mixed large multiplicities: only the dense route can run this shape
            if self._dense_plan is None:
                raise
            self.f, self._generic_error = None, str(err)

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
        xin = self.transpose_in(x)
        if (self._dense_plan is not None and DENSE_ROUTE and not input_indices and weight.shape[0] == 1 and xin.is_cuda
                and xin.dtype == torch.float32 and weight.dtype == torch.float32 and xin.shape[0] >= DENSE_MIN_ROWS):
            return self.transpose_out(_DenseLinear.apply(self._dense_plan, weight, xin.contiguous()))
        if self._dense_plan is not None and DENSE_ROUTE and input_indices and xin.is_cuda and xin.dtype == torch.float32 \
                and weight.dtype == torch.float32 and weight.shape[0] == self.weight_classes \
                and (self.require_grouped or xin.shape[0] >= DENSE_MIN_ROWS):
            bounds = class_bounds(weight_indices, self.weight_classes)
            if bounds is not None:
                return self.transpose_out(_GroupedDenseLinear.apply(self._dense_plan, bounds, weight, xin.contiguous()))
            if self.require_grouped:
                raise ValueError("Linear(method='indexed_linear') does not support non-sorted indices")
        elif self.require_grouped:
            raise ValueError("Linear(method='indexed_linear') needs float32 CUDA tensors, weight classes selected by sorted "
                             "weight_indices and multiplicities that are multiples of 32")
        if self.f is None:
            raise ValueError("Linear: this shape runs only on the dense route (float32 CUDA tensors, one weight set, at least "
                             f"{DENSE_MIN_ROWS} rows); the generic kernel cannot take it: {self._generic_error}")
        out = self.f([weight, xin], input_indices=input_indices)
        return self.transpose_out(out[0])

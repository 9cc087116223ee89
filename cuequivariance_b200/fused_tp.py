"""Execution of dense multi-mode tensor products (method ``"fused_tp"``).

Counterpart of the reference's ``SegmentedPolynomialFusedTP``
(cuequivariance_torch/primitives/segmented_polynomial_fused_tp.py:74-262), which hands 3-
and 4-operand products with up to three modes to a closed kernel.

Two routes:

* small products: every mode but the innermost one of the output is flattened into
  segments, which turns the product into a uniform-1d polynomial for the generic CUDA kernel
  (`FusedTPProgram`);
* the fully connected pattern ``uvw,iu,jv,kw+ijk`` with shared weights at sizes where that
  flattening explodes (u*v*nnz paths): INTERIM composite of device-side torch ops
  (`dense_uvw`): per path the coupled operand ``Z[z,k,(u,v)] = sum_ij C[ijk] x1[z,i,u] x2[z,j,v]``
  is formed and contracted with the weight block by a library GEMM in float32 (TF32 off), and
  autograd differentiates the composite.  It exists so that the configuration runs and is
  checked at full size; the tensor-core kernel that should replace it (weights through TMA,
  ``Z`` tiles built in shared memory, tcgen05 accumulation in TMEM) is not written yet.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from .executor import Uniform1dProgram
from .polynomial import Polynomial

FLATTEN_LIMIT = 20000  # flattened paths above which the composite route is taken


def _flatten_all_but_inner(poly: Polynomial) -> Polynomial:
    def fn(d):
        out_sub = d.operand_subscripts[-1] if d.operand_subscripts else ""
        keep = out_sub[-1:] if out_sub else ""
        modes = "".join(m for m in d.modes() if m != keep)
        return d.flatten_modes(modes)

    return poly.map_tensor_products(fn)


def flattened_path_count(poly: Polynomial) -> int:
    n = 0
    for _, d in poly.operations:
        keep = d.operand_subscripts[-1][-1:] if d.operand_subscripts and d.operand_subscripts[-1] else ""
        for p in d.paths:
            dims = d.path_dims(p)
            extra = int(np.prod([v for k, v in dims.items() if k != keep and k not in d.coefficient_subscripts] or [1]))
            n += extra * int(np.count_nonzero(p.coefficients)) if d.coefficient_subscripts else extra
    return n


class FusedTPProgram(Uniform1dProgram):
    def __init__(self, polynomial: Polynomial, math_dtype, output_dtype_map=None, name="segmented_polynomial"):
        super().__init__(_flatten_all_but_inner(polynomial), math_dtype, output_dtype_map, name)


def is_fully_connected(poly: Polynomial) -> bool:
    if len(poly.operations) != 1 or poly.num_inputs != 3 or poly.num_outputs != 1:
        return False
    ope, d = poly.operations[0]
    return d.subscripts == "uvw,iu,jv,kw+ijk" and tuple(ope.buffers) == (0, 1, 2, 3)


class DenseUVW:
    """INTERIM composite for ``uvw,iu,jv,kw+ijk`` (see the module docstring)."""

    def __init__(self, polynomial: Polynomial, math_dtype: Optional[torch.dtype]):
        _, d = polynomial.operations[0]
        self.d = d
        self.math_dtype = math_dtype
        self.offsets = [op.offsets() for op in d.operands]
        self.out_size = d.operands[3].size
        self._coef = {}

    def _c(self, k, device, dtype):
        key = (k, device, dtype)
        t = self._coef.get(key)
        if t is None:
            t = torch.tensor(self.d.paths[k].coefficients, dtype=dtype, device=device)
            self._coef[key] = t
        return t

    def __call__(self, inputs: List[torch.Tensor]) -> List[torch.Tensor]:
        w, x1, x2 = inputs
        if w.device.type != "cuda":
            raise RuntimeError("cuequivariance_b200 executes on CUDA devices only (there is no CPU fallback)")
        io = x1.dtype
        md = self.math_dtype or (io if io in (torch.float32, torch.float64) else torch.float32)
        d, off = self.d, self.offsets
        B = max(x1.shape[0], x2.shape[0], w.shape[0])
        pieces = [None] * d.operands[3].num_segments
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            for k, p in enumerate(d.paths):
                sw, s1, s2, so = p.indices
                u, v, wd = d.operands[0].segments[sw]
                d1, d2, d3 = p.coefficients.shape
                a = x1[:, off[1][s1] : off[1][s1] + d1 * u].reshape(-1, d1, u).to(md)
                b = x2[:, off[2][s2] : off[2][s2] + d2 * v].reshape(-1, d2, v).to(md)
                z = torch.einsum("ijk,ziu,zjv->zkuv", self._c(k, x1.device, md), a, b)
                wk = w[:, off[0][sw] : off[0][sw] + u * v * wd].to(md)
                if wk.shape[0] == 1:
                    r = (z.reshape(-1, u * v) @ wk.reshape(u * v, wd)).reshape(-1, d3 * wd)
                else:
                    r = torch.einsum("zkq,zqw->zkw", z.reshape(z.shape[0], d3, u * v), wk.reshape(-1, u * v, wd)).reshape(-1, d3 * wd)
                pieces[so] = r if pieces[so] is None else pieces[so] + r
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        cols = []
        for s, seg in enumerate(d.operands[3].segments):
            cols.append(pieces[s] if pieces[s] is not None else x1.new_zeros(B, int(np.prod(seg)), dtype=md))
        return [torch.cat(cols, dim=1).to(io)]

"""Execution of dense multi-mode tensor products (method ``"fused_tp"``).

Counterpart of the reference's ``SegmentedPolynomialFusedTP``
(cuequivariance_torch/primitives/segmented_polynomial_fused_tp.py:74-262), which hands 3-
and 4-operand products with up to three modes to a closed kernel.  Here every mode but the
innermost one of the output is flattened into segments, which turns the product into a
uniform-1d polynomial executed by the generic CUDA kernel.
"""
from __future__ import annotations

from .executor import Uniform1dProgram
from .polynomial import Polynomial


def _flatten_all_but_inner(poly: Polynomial) -> Polynomial:
    def fn(d):
        out_sub = d.operand_subscripts[-1] if d.operand_subscripts else ""
        keep = out_sub[-1:] if out_sub else ""
        modes = "".join(m for m in d.modes() if m != keep)
        return d.flatten_modes(modes)

    return poly.map_tensor_products(fn)


class FusedTPProgram(Uniform1dProgram):
    def __init__(self, polynomial: Polynomial, math_dtype, output_dtype_map=None, name="segmented_polynomial"):
        super().__init__(_flatten_all_but_inner(polynomial), math_dtype, output_dtype_map, name)

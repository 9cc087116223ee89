"""`SegmentedPolynomial`: the torch module that evaluates a polynomial on a B200.

Same constructor and ``forward`` signature as the reference module
(cuequivariance_torch/primitives/segmented_polynomial.py:141-149,259-265); the execution
methods are the CUDA ones only (``"uniform_1d"``; ``"fused_tp"`` for dense three-mode
products).  There is no ``"naive"`` method and no fallback: a polynomial that does not fit
the requested method raises at construction, and CPU tensors raise at call time.
"""
from __future__ import annotations

import warnings
from typing import Any, Dict, List, Optional

import numpy as np
import torch
import torch.nn as nn

from .executor import Uniform1dProgram, evaluate
from .polynomial import Operation, Polynomial
from .stp import Operand, Path, SegmentedTensorProduct


def as_polynomial(p) -> Polynomial:
    """Accepts this package's `Polynomial` or a ``cue.SegmentedPolynomial`` (duck-typed:
    ``inputs``/``outputs`` with ``segments``/``ndim``, ``operations`` of (operation, stp))."""
    if isinstance(p, Polynomial):
        return p
    if hasattr(p, "polynomial") and not hasattr(p, "operations"):
        raise ValueError(
            f"The polynomial is not a segmented polynomial, but a {type(p)}. "
            "Did you forget to call `.polynomial` on the descriptor?"
        )
    try:
        def cv(o):
            return Operand(int(o.ndim), tuple(tuple(s) for s in o.segments))

        ops = []
        for ope, d in p.operations:
            subs = d.subscripts
            stp = SegmentedTensorProduct(
                tuple(str(s) for s in subs.operands), str(subs.coefficients),
                [cv(o) for o in d.operands],
                [Path(tuple(q.indices), np.asarray(q.coefficients, dtype=np.float64)) for q in d.paths],
            )
            ops.append((Operation(tuple(ope.buffers)), stp))
        return Polynomial([cv(o) for o in p.inputs], [cv(o) for o in p.outputs], ops)
    except AttributeError as e:
        raise ValueError(f"The polynomial is not a segmented polynomial, but a {type(p)}") from e


def _resolve_math_dtype(math_dtype, method: str):
    if isinstance(math_dtype, str):
        try:
            math_dtype = getattr(torch, math_dtype)
        except AttributeError:
            raise ValueError(
                f"Invalid math_dtype '{math_dtype}' for method '{method}'. Expected 'float32', 'float64', or None."
            ) from None
    if math_dtype not in (None, torch.float32, torch.float64):
        raise ValueError(f"For method '{method}', math_dtype must be 'float32', 'float64', or None; got {math_dtype}")
    return math_dtype


class SegmentedPolynomial(nn.Module):
    """Evaluates ``polynomial`` with the CUDA executor.

    Args:
        polynomial: `cuequivariance_b200.Polynomial` or ``cue.SegmentedPolynomial``.
        method: ``"uniform_1d"`` (default when empty, with the reference's warning text
            shortened) or ``"fused_tp"``.
        math_dtype: ``float32``/``float64`` (or their names); ``None`` = the dtype of the
            first input if it is one of those, else float32.
        output_dtype_map: per output, the input whose dtype it takes (-1: math dtype);
            default 0.
        name, options: kept for signature compatibility; ``options`` is stored.
    """

    def __init__(
        self,
        polynomial,
        method: str = "",
        math_dtype=None,
        output_dtype_map: List[int] = None,
        name: str = "segmented_polynomial",
        options: Optional[Dict[str, Any]] = None,
    ):
        super().__init__()
        self._polynomial_orig = polynomial
        self._math_dtype_orig = math_dtype
        self._output_dtype_map_orig = output_dtype_map
        self.options = options if options is not None else {}
        self.name = name
        if method == "":
            warnings.warn("No `method` given to SegmentedPolynomial(); defaulting to 'uniform_1d'.")
            method = "uniform_1d"
        if method == "naive":
            raise ValueError(
                "method 'naive' is not provided by cuequivariance_b200: it ships CUDA execution only "
                "(use 'uniform_1d' or 'fused_tp')"
            )
        if method not in ("uniform_1d", "fused_tp"):
            raise ValueError(f"Invalid method: {method}")
        self.method = method
        self.polynomial = as_polynomial(polynomial)
        self.num_inputs = self.polynomial.num_inputs
        self.num_outputs = self.polynomial.num_outputs
        self.math_dtype = _resolve_math_dtype(math_dtype, method)
        self.output_dtype_map = output_dtype_map
        self.repr = repr(self.polynomial)
        self._programs: Dict[torch.dtype, Any] = {}
        # validate eagerly so that an unsuitable polynomial fails at construction
        self._program(self.math_dtype or torch.float32)

    def _program(self, math_dtype: torch.dtype):
        prog = self._programs.get(math_dtype)
        if prog is None:
            if self.method == "uniform_1d":
                prog = Uniform1dProgram(self.polynomial, math_dtype, self.output_dtype_map, self.name)
                from .channelwise import attach_specialisation
                from .executor import attach_static

                attach_specialisation(prog)
                attach_static(prog)
            else:
                from .fused_tp import FLATTEN_LIMIT, DenseUVW, FusedTPProgram, flattened_path_count, is_fully_connected

                if is_fully_connected(self.polynomial) and flattened_path_count(self.polynomial) > FLATTEN_LIMIT:
                    prog = DenseUVW(self.polynomial, self.math_dtype, self.options)
                else:
                    prog = FusedTPProgram(self.polynomial, math_dtype, self.output_dtype_map, self.name)
            self._programs[math_dtype] = prog
        return prog

    def __reduce__(self):
        return (
            SegmentedPolynomial,
            (self._polynomial_orig, self.method, self._math_dtype_orig, self._output_dtype_map_orig, self.name, self.options),
        )

    def __repr__(self):
        return self.repr + f"\n{super().__repr__()}"

    def forward(
        self,
        inputs: List[torch.Tensor],
        input_indices: Optional[Dict[int, torch.Tensor]] = None,
        output_shapes: Optional[Dict[int, torch.Tensor]] = None,
        output_indices: Optional[Dict[int, torch.Tensor]] = None,
        layouts: Optional[Dict[int, tuple]] = None,
    ) -> List[torch.Tensor]:
        """Reference signature plus ``layouts``: {buffer id (inputs, then outputs):
        ((mul, dim), ...)} for buffers the caller holds channel-major (mul_ir)."""
        input_indices = dict(input_indices or {})
        output_shapes = dict(output_shapes or {})
        output_indices = dict(output_indices or {})
        inputs = list(inputs)
        torch._assert(len(inputs) == self.num_inputs, "the number of inputs must match the number of inputs of the polynomial")
        for k, v in input_indices.items():
            torch._assert(0 <= k < self.num_inputs, "input index must be in range")
            torch._assert(v.ndim == 1, "input index must be one-dimensional")
            torch._assert(v.dtype in (torch.int32, torch.int64), "input index must be integral")
        for k, v in output_indices.items():
            torch._assert(0 <= k < self.num_outputs, "output index must be in range")
            torch._assert(v.ndim == 1, "input index must be one-dimensional")
            torch._assert(v.dtype in (torch.int32, torch.int64), "input index must be integral")
        for k, v in output_shapes.items():
            torch._assert(0 <= k < self.num_outputs, "output index must be in range")
            torch._assert(v.ndim == 2, "output shape must be two-dimensional")
        if self.math_dtype is not None:
            md = self.math_dtype
        elif inputs and inputs[0].dtype in (torch.float32, torch.float64):
            md = inputs[0].dtype
        else:
            md = torch.float32
        prog = self._program(md)
        if not hasattr(prog, "run"):  # composite route (dense uvw): no index support, batch semantics of the inputs
            if input_indices or output_indices or output_shapes or layouts:
                raise ValueError("the dense fully connected route takes plain batched (or shared-weight) inputs")
            return prog(inputs)
        return evaluate(prog, inputs, input_indices, output_shapes, output_indices, layouts)

"""Polynomials of segmented tensor products and their reverse-mode derivatives.

A polynomial has ``num_inputs`` input buffers and ``num_outputs`` output buffers and a
list of operations.  Each operation binds the operands of one segmented tensor product
to buffers (``buffers[k]`` = buffer id of operand ``k``; ids ``>= num_inputs`` are
outputs, exactly one per operation; an input buffer may be bound to several operands,
which is how powers such as ``x*x*x`` are written).  The value of output ``j`` is the
sum over the operations bound to it.  Same model as the reference's
``cue.SegmentedPolynomial`` / ``cue.Operation``
(cuequivariance/segmented_polynomials/segmented_polynomial.py:34-51, operation.py:50-81).

Derivatives are again polynomials over the same segmented tensor products: the
cotangent takes the place of the output operand and the differentiated operand becomes
the output.  The reference derives them as jvp-then-transpose
(segmented_polynomial.py:1003-1133, operation.py:149-261); here the two steps are fused
into one direct rule, which yields the same function (checked in the tests against the
reference-generated tables and against autograd of the naive evaluation).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np

from .stp import Operand, Path, SegmentedTensorProduct


@dataclass(frozen=True)
class Operation:
    buffers: tuple[int, ...]

    def __post_init__(self):
        object.__setattr__(self, "buffers", tuple(int(b) for b in self.buffers))

    def output_operand(self, num_inputs: int) -> int:
        outs = [k for k, b in enumerate(self.buffers) if b >= num_inputs]
        if len(outs) != 1:
            raise ValueError(f"operation {self.buffers} must bind exactly one output buffer")
        return outs[0]

    def output_buffer(self, num_inputs: int) -> int:
        return self.buffers[self.output_operand(num_inputs)]

    def input_operands(self, num_inputs: int) -> list[tuple[int, int]]:
        return [(k, b) for k, b in enumerate(self.buffers) if b < num_inputs]


class Polynomial:
    """Host-side polynomial: ``inputs``/``outputs`` are `Operand` layouts of the buffers."""

    def __init__(
        self,
        inputs: Sequence[Operand],
        outputs: Sequence[Operand],
        operations: Sequence[tuple[Operation, SegmentedTensorProduct]],
    ):
        self.inputs = tuple(inputs)
        self.outputs = tuple(outputs)
        ops = []
        for ope, stp in operations:
            if not isinstance(ope, Operation):
                ope = Operation(tuple(ope))
            if len(ope.buffers) != stp.num_operands:
                raise ValueError("operation arity does not match its tensor product")
            for k, b in enumerate(ope.buffers):
                want = self.operands[b]
                if stp.operands[k].size != want.size:
                    raise ValueError(
                        f"operand {k} (size {stp.operands[k].size}) bound to buffer {b} (size {want.size})"
                    )
            ope.output_operand(self.num_inputs)
            ops.append((ope, stp))
        self.operations = tuple(ops)

    # -- basic facts --------------------------------------------------------------
    @property
    def num_inputs(self) -> int:
        return len(self.inputs)

    @property
    def num_outputs(self) -> int:
        return len(self.outputs)

    @property
    def operands(self) -> tuple[Operand, ...]:
        return self.inputs + self.outputs

    @classmethod
    def eval_last_operand(cls, stp: SegmentedTensorProduct) -> "Polynomial":
        """Polynomial whose inputs are all operands but the last and whose output is the last."""
        n = stp.num_operands
        return cls(stp.operands[:-1], stp.operands[-1:], [(Operation(tuple(range(n))), stp)])

    def __repr__(self) -> str:
        lines = [f"Polynomial(inputs={list(self.inputs)} -> outputs={list(self.outputs)})"]
        for ope, stp in self.operations:
            lines.append(f"  {ope.buffers}: {stp.subscripts} num_paths={stp.num_paths}")
        return "\n".join(lines)

    # -- transformations that keep the function -------------------------------------------
    def map_tensor_products(self, fn) -> "Polynomial":
        new_ops = [(ope, fn(stp)) for ope, stp in self.operations]
        operands = list(self.operands)
        for ope, stp in new_ops:
            for k, b in enumerate(ope.buffers):
                operands[b] = stp.operands[k]
        return Polynomial(operands[: self.num_inputs], operands[self.num_inputs :], new_ops)

    def flatten_coefficient_modes(self) -> "Polynomial":
        return self.map_tensor_products(lambda d: d.flatten_coefficient_modes())

    def squeeze_modes(self) -> "Polynomial":
        return self.map_tensor_products(lambda d: d.squeeze_modes())

    @classmethod
    def stack(cls, polys: Sequence["Polynomial"], stacked: Sequence[bool]) -> "Polynomial":
        """Concatenate the buffers flagged in ``stacked`` (one flag per buffer) and share the
        others; segment indices of stacked operands are shifted (reference:
        segmented_polynomial.py ``stack``)."""
        n_in, n_out = polys[0].num_inputs, polys[0].num_outputs
        nb = n_in + n_out
        assert len(stacked) == nb and all(p.num_inputs == n_in and p.num_outputs == n_out for p in polys)
        shift = [[0] * nb for _ in polys]
        operands = []
        for b in range(nb):
            if stacked[b]:
                segs, nd = [], polys[0].operands[b].ndim
                for pi, p in enumerate(polys):
                    shift[pi][b] = len(segs)
                    segs += list(p.operands[b].segments)
                operands.append(Operand(nd, tuple(segs)))
            else:
                cands = [p.operands[b] for p in polys]
                assert all(c == cands[0] for c in cands), "shared buffers must agree"
                operands.append(cands[0])
        new_ops = []
        for pi, p in enumerate(polys):
            for ope, stp in p.operations:
                d = stp.copy()
                d.operands = [operands[b] for b in ope.buffers]
                d.paths = [
                    Path(tuple(s + shift[pi][b] for s, b in zip(path.indices, ope.buffers)), path.coefficients)
                    for path in stp.paths
                ]
                new_ops.append((ope, d))
        return cls(operands[:n_in], operands[n_in:], new_ops)

    # -- differentiation ------------------------------------------------------------------
    def backward(self, requires_gradient: Sequence[bool], has_cotangent: Sequence[bool]) -> "Polynomial":
        """Vector-Jacobian product as a polynomial.

        New inputs : the original inputs, then one cotangent per output with
                     ``has_cotangent`` set (in output order).
        New outputs: one gradient per input with ``requires_gradient`` set (in input order).
        """
        requires_gradient, has_cotangent = list(requires_gradient), list(has_cotangent)
        assert len(requires_gradient) == self.num_inputs and len(has_cotangent) == self.num_outputs
        n_in = self.num_inputs
        cot_buffer, nxt = {}, n_in
        for j, has in enumerate(has_cotangent):
            if has:
                cot_buffer[j] = nxt
                nxt += 1
        new_n_in = nxt
        grad_buffer = {}
        for i, req in enumerate(requires_gradient):
            if req:
                grad_buffer[i] = nxt
                nxt += 1
        new_inputs = list(self.inputs) + [self.outputs[j] for j in cot_buffer]
        new_outputs = [self.inputs[i] for i in grad_buffer]
        new_ops = []
        for ope, stp in self.operations:
            k_out = ope.output_operand(n_in)
            j = ope.buffers[k_out] - n_in
            if j not in cot_buffer:
                continue
            for k, b in ope.input_operands(n_in):
                if b not in grad_buffer:
                    continue
                bufs = list(ope.buffers)
                bufs[k_out] = cot_buffer[j]
                bufs[k] = grad_buffer[b]
                new_ops.append((Operation(tuple(bufs)), stp))
        return Polynomial(new_inputs, new_outputs, _merge_identical(new_ops, new_n_in))


def _merge_identical(operations, num_inputs: int):
    """Fold operations that bind the same buffers and whose path lists coincide after
    the operand permutation relating them (this is what turns the three derivative terms
    of ``w*x*x*x`` with a symmetric coefficient table into one term of weight 3)."""
    out: list[list] = []
    for ope, stp in operations:
        merged = False
        for entry in out:
            ope0, stp0, mult = entry
            if sorted(ope0.buffers) != sorted(ope.buffers) or stp0.num_paths != stp.num_paths:
                continue
            perm = _matching_permutation(ope0, ope)
            if perm is None:
                continue
            cand = stp.permute_operands(perm)
            if _same_paths(stp0, cand):
                entry[2] = mult + 1
                merged = True
                break
        if not merged:
            out.append([ope, stp, 1])
    return [(ope, stp if m == 1 else stp.scaled(float(m))) for ope, stp, m in out]


def _matching_permutation(ope0: Operation, ope: Operation):
    """Permutation ``perm`` with ``ope.buffers[perm[i]] == ope0.buffers[i]`` that keeps the
    relative order of operands bound to the same buffer, or None."""
    used, perm = set(), []
    for b in ope0.buffers:
        for k, bb in enumerate(ope.buffers):
            if bb == b and k not in used:
                used.add(k)
                perm.append(k)
                break
        else:
            return None
    return perm


def _same_paths(a: SegmentedTensorProduct, b: SegmentedTensorProduct) -> bool:
    if a.operand_subscripts != b.operand_subscripts or a.coefficient_subscripts != b.coefficient_subscripts:
        return False
    if a.operands != b.operands:
        return False

    def canon(d):
        return sorted((p.indices, p.coefficients.tobytes()) for p in d.paths)

    return canon(a) == canon(b)

"""Descriptors: the polynomials of the equivariant operations, built from irreps.

Each function returns an `EquivariantPolynomial` = a `Polynomial` plus the irreps and
layout of every buffer.  Construction follows the reference descriptors so that segment
order, path order, Clebsch-Gordan convention and normalisation agree with
``cue.descriptors.*`` (cuequivariance/group_theory/descriptors/irreps_tp.py:22-91 fully
connected, :232-321 channelwise, :505-545 linear; spherical_harmonics_.py:23-156).
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass
from functools import lru_cache
from typing import Optional, Sequence

import numpy as np

from .cg import clebsch_gordan
from .irreps import Irrep, Irreps, IrrepsLayout, ir_mul, parse_irrep_list
from .polynomial import Operation, Polynomial
from .stp import Operand, SegmentedTensorProduct


@dataclass(frozen=True)
class IrrepsAndLayout:
    irreps: Irreps
    layout: IrrepsLayout

    @property
    def dim(self) -> int:
        return self.irreps.dim


@dataclass(frozen=True)
class EquivariantPolynomial:
    inputs: tuple[IrrepsAndLayout, ...]
    outputs: tuple[IrrepsAndLayout, ...]
    polynomial: Polynomial

    @property
    def operands(self) -> tuple[IrrepsAndLayout, ...]:
        return self.inputs + self.outputs

    def __repr__(self) -> str:
        a = " ".join(f"{r.irreps}" for r in self.inputs)
        b = " ".join(f"{r.irreps}" for r in self.outputs)
        return f"EquivariantPolynomial({a} -> {b})\n{self.polynomial}"


def _as_irreps(x, group: Optional[str] = None) -> Irreps:
    return x if isinstance(x, Irreps) else Irreps(group, x) if group else Irreps(x)


def channelwise_tensor_product(
    irreps1, irreps2, irreps3_filter=None, simplify_irreps3: bool = False
) -> EquivariantPolynomial:
    """``weights[uv], lhs[iu], rhs[jv] -> output[kuv]`` with coefficient ``[ijk]``.

    One path, one weight segment ``(u, v)`` and one output segment ``(k, u, v)`` per
    allowed triple (ir1, ir2, ir3); output blocks are then sorted by irrep (stable) and
    the weight segments follow the same order; paths are normalised for the output.
    """
    irreps1 = _as_irreps(irreps1)
    irreps2 = _as_irreps(irreps2, irreps1.group)
    keep = parse_irrep_list(irreps1.group, irreps3_filter)

    d = SegmentedTensorProduct.from_subscripts("uv,iu,jv,kuv+ijk")
    for mul, ir in irreps1:
        d.add_segment(1, (ir.dim, mul))
    for mul, ir in irreps2:
        d.add_segment(2, (ir.dim, mul))

    blocks = []
    for (i1, (mul1, ir1)), (i2, (mul2, ir2)) in itertools.product(enumerate(irreps1), enumerate(irreps2)):
        for ir3 in ir1 * ir2:
            if keep is not None and ir3 not in keep:
                continue
            for cg in clebsch_gordan(ir1, ir2, ir3):
                d.add_path(None, i1, i2, None, c=cg, dims={"u": mul1, "v": mul2})
                blocks.append((mul1 * mul2, ir3))

    irreps3, _, inv = Irreps(irreps1.group, blocks).sort()
    d = d.permute_segments(0, inv).permute_segments(3, inv)
    d = d.normalize_paths_for_operand(-1)

    if simplify_irreps3:
        d = d.flatten_coefficient_modes()
        comps = [(ir._key(), k, sid) for sid, (ir, k) in enumerate((ir, k) for _, ir in irreps3 for k in range(ir.dim))]
        d = d.permute_segments(3, [sid for _, _, sid in sorted(comps)])
        irreps3 = irreps3.simplify()

    poly = Polynomial.eval_last_operand(d)
    return EquivariantPolynomial(
        (
            IrrepsAndLayout(irreps1.new_scalars(poly.inputs[0].size), ir_mul),
            IrrepsAndLayout(irreps1, ir_mul),
            IrrepsAndLayout(irreps2, ir_mul),
        ),
        (IrrepsAndLayout(irreps3, ir_mul),),
        poly,
    )


def fully_connected_tensor_product(irreps1, irreps2, irreps3) -> EquivariantPolynomial:
    """``weights[uvw], lhs[iu], rhs[jv] -> output[kw]`` with coefficient ``[ijk]``."""
    irreps1 = _as_irreps(irreps1)
    irreps2 = _as_irreps(irreps2, irreps1.group)
    irreps3 = _as_irreps(irreps3, irreps1.group)

    d = SegmentedTensorProduct.from_subscripts("uvw,iu,jv,kw+ijk")
    for mul, ir in irreps1:
        d.add_segment(1, (ir.dim, mul))
    for mul, ir in irreps2:
        d.add_segment(2, (ir.dim, mul))
    for mul, ir in irreps3:
        d.add_segment(3, (ir.dim, mul))
    for (i1, (mul1, ir1)), (i2, (mul2, ir2)), (i3, (mul3, ir3)) in itertools.product(
        enumerate(irreps1), enumerate(irreps2), enumerate(irreps3)
    ):
        if ir3 not in ir1 * ir2:
            continue
        for cg in clebsch_gordan(ir1, ir2, ir3):
            d.add_path(None, i1, i2, i3, c=cg, dims={"u": mul1, "v": mul2, "w": mul3})
    d = d.normalize_paths_for_operand(-1)
    poly = Polynomial.eval_last_operand(d)
    return EquivariantPolynomial(
        (
            IrrepsAndLayout(irreps1.new_scalars(poly.inputs[0].size), ir_mul),
            IrrepsAndLayout(irreps1, ir_mul),
            IrrepsAndLayout(irreps2, ir_mul),
        ),
        (IrrepsAndLayout(irreps3, ir_mul),),
        poly,
    )


def linear(irreps_in, irreps_out) -> EquivariantPolynomial:
    """``weights[uv], input[iu] -> output[iv]``: one dense block per matching irrep pair."""
    irreps_in = _as_irreps(irreps_in)
    irreps_out = _as_irreps(irreps_out, irreps_in.group)
    d = SegmentedTensorProduct.from_subscripts("uv,iu,iv")
    for mul, ir in irreps_in:
        d.add_segment(1, (ir.dim, mul))
    for mul, ir in irreps_out:
        d.add_segment(2, (ir.dim, mul))
    for (i1, (mul1, ir1)), (i2, (mul2, ir2)) in itertools.product(enumerate(irreps_in), enumerate(irreps_out)):
        if ir1 == ir2:
            d.add_path(None, i1, i2, c=1.0, dims={"u": mul1, "v": mul2})
    d = d.normalize_paths_for_operand(-1)
    poly = Polynomial.eval_last_operand(d)
    return EquivariantPolynomial(
        (
            IrrepsAndLayout(irreps_in.new_scalars(poly.inputs[0].size), ir_mul),
            IrrepsAndLayout(irreps_in, ir_mul),
        ),
        (IrrepsAndLayout(irreps_out, ir_mul),),
        poly,
    )


# ---------------------------------------------------------------------------------------
# spherical harmonics: polynomials in (x0, x1, x2) held as {(a, b, c): coefficient}
# ---------------------------------------------------------------------------------------
def _poly_mul(p: dict, q: dict) -> dict:
    out: dict = {}
    for (a1, b1, c1), v1 in p.items():
        for (a2, b2, c2), v2 in q.items():
            k = (a1 + a2, b1 + b2, c1 + c2)
            out[k] = out.get(k, 0.0) + v1 * v2
    return out


def _poly_eval(p: dict, x) -> float:
    return sum(v * x[0] ** a * x[1] ** b * x[2] ** c for (a, b, c), v in p.items())


@lru_cache(maxsize=None)
def _sh_polynomials(l: int) -> tuple:  # noqa: E741
    """Components of Y_l as homogeneous polynomials of degree l; ``|Y_l(n)|^2 = 2l+1`` on
    unit vectors ("component" normalisation).  Built by coupling Y_{ceil(l/2)} with
    Y_{floor(l/2)} through the Clebsch-Gordan tensor and rescaling at the point (0,1,0),
    as the reference does symbolically (spherical_harmonics_.py:107-156)."""
    if l == 0:
        return ({(0, 0, 0): 1.0},)
    if l == 1:
        s = math.sqrt(3.0)
        return ({(1, 0, 0): s}, {(0, 1, 0): s}, {(0, 0, 1): s})
    lb = l // 2
    la = l - lb
    ya, yb = _sh_polynomials(la), _sh_polynomials(lb)
    cg = clebsch_gordan(Irrep(la, 0), Irrep(lb, 0), Irrep(l, 0))[0]
    comps = []
    for k in range(2 * l + 1):
        acc: dict = {}
        for i in range(2 * la + 1):
            for j in range(2 * lb + 1):
                c = cg[i, j, k]
                if c == 0.0:
                    continue
                for mono, v in _poly_mul(ya[i], yb[j]).items():
                    acc[mono] = acc.get(mono, 0.0) + c * v
        comps.append(acc)
    at_y = [_poly_eval(p, (0.0, 1.0, 0.0)) for p in comps]
    scale = math.sqrt(2 * l + 1) / math.sqrt(sum(v * v for v in at_y))
    out = []
    for p in comps:
        mx = max((abs(v) for v in p.values()), default=0.0)
        out.append({m: v * scale for m, v in sorted(p.items(), reverse=True) if abs(v) > 1e-12 * max(mx, 1.0)})
    return tuple(out)


def spherical_harmonics(ir_vec, ls: Sequence[int], layout=ir_mul) -> EquivariantPolynomial:
    """``vector[] x l -> Y_l[]`` for every ``l`` in ``ls``; all segments are scalars."""
    ir_vec = Irrep.parse("O3", ir_vec) if not isinstance(ir_vec, Irrep) else ir_vec
    if ir_vec.l != 1:
        raise ValueError("the vector irrep must have l=1")
    vec = Operand(0, ((),) * 3)
    pieces, blocks = [], []
    for l in ls:  # noqa: E741
        ir = Irrep(l, ir_vec.p**l if ir_vec.p != 0 else 0)
        d = SegmentedTensorProduct.empty_segments([3] * l + [ir.dim])
        for k, comp in enumerate(_sh_polynomials(l)):
            for (a, b, c), v in comp.items():
                # the monomial x0^a x1^b x2^c is spread evenly over its distinct orderings so
                # that the table is symmetric under exchange of the vector operands
                base = (0,) * a + (1,) * b + (2,) * c
                perms = sorted(set(itertools.permutations(base)))
                for idx in perms:
                    d.add_path(*idx, k, c=v / len(perms))
        d = d.sort_paths(0) if l > 0 else d
        d.paths = sorted(d.paths, key=lambda p: p.indices)
        pieces.append(Polynomial([vec], [Operand(0, ((),) * ir.dim)], [(Operation((0,) * l + (1,)), d)]))
        blocks.append((1, ir))
    poly = Polynomial.stack(pieces, [False, True])
    group = "SO3" if ir_vec.p == 0 else "O3"
    return EquivariantPolynomial(
        (IrrepsAndLayout(Irreps(group, [(1, ir_vec)]), ir_mul),),
        (IrrepsAndLayout(Irreps(group, blocks), IrrepsLayout.parse(layout)),),
        poly,
    )


# ---------------------------------------------------------------------------------------
# symmetric contraction (MACE): tables generated from the reference, see data/
# ---------------------------------------------------------------------------------------
def _symmetric_contraction_degree(irreps_in: Irreps, irreps_out: Irreps, degree: int, mul: int) -> Polynomial:
    """One degree of the symmetric contraction built from this package's own symmetric-power basis:
    ``w_a_b_.._i+ab..iw`` with one path per output irrep carrying ``U[a, b, .., i, w]``, normalised for the
    output, coefficient modes flattened, and the channel mode ``u`` appended to every operand (the
    construction of cuequivariance/group_theory/descriptors/symmetric_contractions.py:47-88)."""
    from .stp import Path
    from .symmetric_basis import symmetric_power_basis

    blocks = [ir for _, ir in irreps_in]
    letters = "abcdefgh"[:degree]
    d = SegmentedTensorProduct.from_subscripts("w," + ",".join(letters) + ",i+" + letters + "iw")
    for k in range(1, degree + 1):
        d.add_segment(k, (irreps_in.set_mul(1).dim,))
    for _, ir in irreps_out:
        U = symmetric_power_basis(blocks, degree, ir)
        if U.shape[-1] == 0:
            d.add_segment(degree + 1, (ir.dim,))
        else:
            d.add_path(None, *(0,) * degree, None, c=U)
    d = d.normalize_paths_for_operand(-1).flatten_coefficient_modes()
    # every operand is now a list of scalar segments: give each the channel axis
    operands = [Operand(1, ((mul,),) * op.num_segments) for op in d.operands]
    du = SegmentedTensorProduct(("u",) * len(operands), "", operands, [Path(p.indices, p.coefficients) for p in d.paths])
    return Polynomial([operands[0], operands[1]], [operands[-1]], [(Operation((0,) + (1,) * degree + (2,)), du)])


def symmetric_contraction(irreps_in, irreps_out, degrees: Sequence[int], basis: str = "auto"):
    """``weights[u], input[u] (x degree) -> output[u]`` for each degree in ``degrees``
    (which must be ``1..n``).  Returns ``(EquivariantPolynomial, projection)`` like the
    reference's ``experimental.mace.symmetric_contraction``; ``projection`` maps original-MACE
    weights to this basis.

    The basis of the symmetric powers is not unique (any invertible mixing of the weights gives another
    valid one).  ``basis``:

    * ``"reference"``: the reference's own path tables, shipped under ``cuequivariance_b200/data`` for
      input irreps ``0e[+1o[+2e[+3o]]]``, output ``0e[+1o[+2e]]`` and degree up to 3 (any multiplicity), so
      that weights trained with the reference keep their meaning;
    * ``"constructed"``: this package's own basis (``symmetric_basis.symmetric_power_basis``), for any
      O3/SO3 irreps and degree; the projection from original-MACE weights is not available (``None``);
    * ``"auto"``: the table when there is one, else the constructed basis.
    """
    import os

    irreps_in = _as_irreps(irreps_in)
    irreps_out = _as_irreps(irreps_out, irreps_in.group)
    degrees = tuple(degrees)
    if degrees != tuple(range(1, len(degrees) + 1)):
        raise ValueError("degrees must be (1, 2, ..., n)")
    muls = set(irreps_in.muls) | set(irreps_out.muls)
    if len(muls) != 1:
        raise ValueError("Input/Output irreps must have the same mul")
    (mul,) = muls
    if basis not in ("auto", "reference", "constructed"):
        raise ValueError("basis must be 'auto', 'reference' or 'constructed'")
    key_in = "_".join(repr(ir) for _, ir in irreps_in)
    key_out = "_".join(repr(ir) for _, ir in irreps_out)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", f"sc__{key_in}__{key_out}__deg{len(degrees)}.npz")
    if basis == "constructed" or (basis == "auto" and not os.path.exists(path)):
        polys = [_symmetric_contraction_degree(irreps_in, irreps_out, deg, mul) for deg in degrees]
        poly = Polynomial.stack(polys, [True, False, False])
        e = EquivariantPolynomial(
            (IrrepsAndLayout(irreps_in.new_scalars(poly.inputs[0].size), ir_mul), IrrepsAndLayout(irreps_in, ir_mul)),
            (IrrepsAndLayout(irreps_out, ir_mul),),
            poly,
        )
        return e, None
    if not os.path.exists(path):
        raise NotImplementedError(
            f"no reference table for {irreps_in} -> {irreps_out} degree {len(degrees)}; "
            "tables exist for inputs 0e[+1o[+2e[+3o]]], outputs 0e[+1o[+2e]], degree <= 3 "
            "(data/make_symmetric_contraction_tables.py generates more from the reference); basis='constructed' covers any shape"
        )
    t = np.load(path)
    nseg = [int(n) for n in t["num_segments"]]
    operands = [Operand(1, ((mul,),) * n) for n in nseg]
    ops = []
    for k in range(int(t["num_operations"])):
        buffers = tuple(int(b) for b in t[f"op{k}_buffers"])
        d = SegmentedTensorProduct(("u",) * len(buffers), "", [operands[b] for b in buffers], [])
        from .stp import Path

        d.paths = [Path(tuple(int(i) for i in idx), np.float64(c)) for idx, c in zip(t[f"op{k}_indices"], t[f"op{k}_coefficients"])]
        ops.append((Operation(buffers), d))
    poly = Polynomial(operands[:2], operands[2:], ops)
    e = EquivariantPolynomial(
        (IrrepsAndLayout(irreps_in.new_scalars(poly.inputs[0].size), ir_mul), IrrepsAndLayout(irreps_in, ir_mul)),
        (IrrepsAndLayout(irreps_out, ir_mul),),
        poly,
    )
    return e, np.array(t["projection"])

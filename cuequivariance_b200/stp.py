"""Segmented tensor products: the host-side description the CUDA plans are compiled from.

A *segmented operand* is a flat vector cut into segments, each segment a small dense
tensor whose axes are named by one-letter modes.  A *path* picks one segment per
operand and carries a coefficient tensor; the product contracts, for every path,
``coefficient x segment_0 x ... x segment_{n-2}`` into ``segment_{n-1}`` following the
subscripts (einsum semantics, repeated modes are shared, modes missing from the last
operand are summed).  Same model as the reference's
``cue.SegmentedTensorProduct`` (cuequivariance/segmented_polynomials/
segmented_tensor_product.py:46-65, segmented_operand.py:23-54, path.py:32-51); this is an
independent, much smaller implementation holding only what the executor needs:
construction, path normalisation (:1243-1284), flattening of coefficient modes
(:1472-1637), squeezing of extent-1 modes and operand/segment permutations.
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np


@dataclass(frozen=True)
class Operand:
    """Flat vector split into segments of shape ``segments[i]`` (all of rank ``ndim``)."""

    ndim: int
    segments: tuple[tuple[int, ...], ...] = ()

    def __post_init__(self):
        object.__setattr__(self, "segments", tuple(tuple(int(d) for d in s) for s in self.segments))
        for s in self.segments:
            if len(s) != self.ndim:
                raise ValueError(f"segment {s} does not have {self.ndim} axes")

    @property
    def num_segments(self) -> int:
        return len(self.segments)

    @property
    def size(self) -> int:
        return sum(math.prod(s) for s in self.segments)

    def offsets(self) -> list[int]:
        out, off = [], 0
        for s in self.segments:
            out.append(off)
            off += math.prod(s)
        return out

    def slices(self) -> list[slice]:
        return [slice(o, o + math.prod(s)) for o, s in zip(self.offsets(), self.segments)]

    def uniform_shape(self) -> Optional[tuple[int, ...]]:
        """The common segment shape, or None if segments differ (or there are none)."""
        if not self.segments:
            return None
        first = self.segments[0]
        return first if all(s == first for s in self.segments) else None

    def __repr__(self) -> str:
        u = self.uniform_shape()
        if u is not None:
            return f"[{self.size}:{self.num_segments}x{u}]"
        return f"[{self.size}:{self.num_segments} segments]"


@dataclass(frozen=True, eq=False)
class Path:
    indices: tuple[int, ...]
    coefficients: np.ndarray

    def __post_init__(self):
        object.__setattr__(self, "indices", tuple(int(i) for i in self.indices))
        c = np.asarray(self.coefficients, dtype=np.float64)
        object.__setattr__(self, "coefficients", c)


def _parse_subscripts(s: str) -> tuple[tuple[str, ...], str]:
    """``"uv,iu,jv,kuv+ijk"`` -> (("uv","iu","jv","kuv"), "ijk").  ``_`` also separates operands."""
    if "+" in s:
        ops, coeff = s.split("+")
    else:
        ops, coeff = s, ""
    ops = tuple(ops.replace("_", ",").split(","))
    for t in ops + (coeff,):
        if not all(ch.islower() and ch.isalpha() for ch in t):
            raise ValueError(f"invalid subscripts {s!r}")
    return ops, coeff


@dataclass(eq=False)
class SegmentedTensorProduct:
    operand_subscripts: tuple[str, ...]
    coefficient_subscripts: str
    operands: list[Operand] = field(default_factory=list)
    paths: list[Path] = field(default_factory=list)

    # -- construction -------------------------------------------------------------
    @classmethod
    def from_subscripts(cls, subscripts: str) -> "SegmentedTensorProduct":
        ops, coeff = _parse_subscripts(subscripts)
        return cls(ops, coeff, [Operand(len(s)) for s in ops], [])

    @classmethod
    def empty_segments(cls, num_segments: Sequence[int]) -> "SegmentedTensorProduct":
        """All-scalar operands (no modes) with the given segment counts."""
        n = len(num_segments)
        return cls(("",) * n, "", [Operand(0, ((),) * k) for k in num_segments], [])

    @property
    def subscripts(self) -> str:
        s = ",".join(self.operand_subscripts)
        return s + ("+" + self.coefficient_subscripts if self.coefficient_subscripts else "")

    @property
    def num_operands(self) -> int:
        return len(self.operands)

    @property
    def num_paths(self) -> int:
        return len(self.paths)

    def modes(self) -> list[str]:
        seen: list[str] = []
        for s in self.operand_subscripts + (self.coefficient_subscripts,):
            for ch in s:
                if ch not in seen:
                    seen.append(ch)
        return seen

    def copy(self) -> "SegmentedTensorProduct":
        return SegmentedTensorProduct(
            self.operand_subscripts, self.coefficient_subscripts, list(self.operands), list(self.paths)
        )

    def add_segment(self, operand: int, shape) -> int:
        operand %= self.num_operands
        if isinstance(shape, dict):
            shape = tuple(shape[ch] for ch in self.operand_subscripts[operand])
        op = self.operands[operand]
        self.operands[operand] = Operand(op.ndim, op.segments + (tuple(shape),))
        return op.num_segments

    def path_dims(self, path: Path) -> dict[str, int]:
        dims: dict[str, int] = {}
        for oid, sid in enumerate(path.indices):
            for ch, d in zip(self.operand_subscripts[oid], self.operands[oid].segments[sid]):
                if dims.setdefault(ch, d) != d:
                    raise ValueError(f"mode {ch} has conflicting extents {dims[ch]} and {d}")
        for ch, d in zip(self.coefficient_subscripts, path.coefficients.shape):
            if dims.setdefault(ch, d) != d:
                raise ValueError(f"mode {ch} has conflicting extents {dims[ch]} and {d}")
        return dims

    def add_path(self, *segments, c, dims: Optional[dict[str, int]] = None) -> int:
        """Append a path.  ``None`` in place of a segment index creates a new segment whose
        shape is deduced from the other operands, the coefficient shape and ``dims``."""
        if len(segments) != self.num_operands:
            raise ValueError("one segment index (or None) per operand is required")
        c = np.asarray(c, dtype=np.float64)
        if c.ndim != len(self.coefficient_subscripts):
            raise ValueError("coefficient rank does not match its subscripts")
        known = dict(dims or {})
        for ch, d in zip(self.coefficient_subscripts, c.shape):
            known[ch] = d
        for oid, sid in enumerate(segments):
            if sid is not None:
                for ch, d in zip(self.operand_subscripts[oid], self.operands[oid].segments[sid]):
                    known[ch] = d
        idx = []
        for oid, sid in enumerate(segments):
            if sid is None:
                sid = self.add_segment(oid, tuple(known[ch] for ch in self.operand_subscripts[oid]))
            idx.append(sid)
        p = Path(tuple(idx), c)
        self.path_dims(p)  # consistency check
        self.paths.append(p)
        return len(self.paths) - 1

    # -- rearrangements -------------------------------------------------------------
    def permute_segments(self, operand: int, order: Sequence[int]) -> "SegmentedTensorProduct":
        """New segment ``i`` of ``operand`` is old segment ``order[i]``."""
        operand %= self.num_operands
        op = self.operands[operand]
        order = list(order)
        if sorted(order) != list(range(op.num_segments)):
            raise ValueError("order must be a permutation of the segments")
        new_of_old = {old: new for new, old in enumerate(order)}
        out = self.copy()
        out.operands[operand] = Operand(op.ndim, tuple(op.segments[i] for i in order))
        out.paths = [
            Path(tuple(new_of_old[s] if o == operand else s for o, s in enumerate(p.indices)), p.coefficients)
            for p in self.paths
        ]
        return out

    def permute_operands(self, order: Sequence[int]) -> "SegmentedTensorProduct":
        """New operand ``i`` is old operand ``order[i]``."""
        order = [o % self.num_operands for o in order]
        return SegmentedTensorProduct(
            tuple(self.operand_subscripts[o] for o in order),
            self.coefficient_subscripts,
            [self.operands[o] for o in order],
            [Path(tuple(p.indices[o] for o in order), p.coefficients) for p in self.paths],
        )

    def move_operand_last(self, operand: int) -> "SegmentedTensorProduct":
        operand %= self.num_operands
        order = [o for o in range(self.num_operands) if o != operand] + [operand]
        return self.permute_operands(order)

    def sort_paths(self, operand: int = -1) -> "SegmentedTensorProduct":
        """Stable sort by the segment index of ``operand`` first, then the other indices."""
        operand %= self.num_operands
        out = self.copy()
        out.paths = sorted(self.paths, key=lambda p: (p.indices[operand],) + p.indices)
        return out

    def scaled(self, factor: float) -> "SegmentedTensorProduct":
        out = self.copy()
        out.paths = [Path(p.indices, p.coefficients * factor) for p in self.paths]
        return out

    # -- normalisation ---------------------------------------------------------------
    def normalize_paths_for_operand(self, operand: int) -> "SegmentedTensorProduct":
        """Divide every path by sqrt(variance of its segment of ``operand``), the variance
        being ``sum_paths mean(c**2) * prod(extents of the modes contracted away)`` under
        unit-variance inputs (reference: segmented_tensor_product.py:1243-1284)."""
        operand %= self.num_operands
        kept = set(self.operand_subscripts[operand])
        var = [0.0] * self.operands[operand].num_segments
        for p in self.paths:
            dims = self.path_dims(p)
            contracted = math.prod(d for ch, d in dims.items() if ch not in kept)
            var[p.indices[operand]] += float(np.mean(p.coefficients**2)) * contracted
        out = self.copy()
        out.paths = []
        for p in self.paths:
            v = var[p.indices[operand]]
            c = p.coefficients / math.sqrt(v) if v > 0 else 0.0 * p.coefficients
            out.paths.append(Path(p.indices, c))
        return out

    # -- mode surgery -------------------------------------------------------------------
    def flatten_modes(self, modes: str, skip_zeros: bool = True) -> "SegmentedTensorProduct":
        """Turn the listed modes into explicit segments: a segment of shape ``(i, u)`` with
        ``i`` flattened becomes ``i`` consecutive segments of shape ``(u,)``; each path is
        split accordingly.  The flattened modes must lead in every operand that has them, so
        the operand's memory order is unchanged.  Zero coefficients are dropped."""
        modes = "".join(ch for ch in self.modes() if ch in set(modes))
        if not modes:
            return self
        lead = []
        for s in self.operand_subscripts:
            n = 0
            while n < len(s) and s[n] in modes:
                n += 1
            if any(ch in modes for ch in s[n:]):
                raise ValueError(f"modes {modes} must lead in operand subscripts {s!r}")
            lead.append(n)

        new_ops, first_new = [], []
        for op, n in zip(self.operands, lead):
            segs, starts, off = [], [], 0
            for s in op.segments:
                starts.append(off)
                k = math.prod(s[:n])
                segs += [s[n:]] * k
                off += k
            new_ops.append(Operand(op.ndim - n, tuple(segs)))
            first_new.append(starts)

        cs = self.coefficient_subscripts
        c_flat_axes = [a for a, ch in enumerate(cs) if ch in modes]
        new_cs = "".join(ch for ch in cs if ch not in modes)
        new_paths = []
        for p in self.paths:
            dims = self.path_dims(p)
            for combo in itertools.product(*(range(dims[m]) for m in modes)):
                at = dict(zip(modes, combo))
                sel = tuple(at[ch] if a in c_flat_axes else slice(None) for a, ch in enumerate(cs))
                c = p.coefficients[sel]
                if skip_zeros and not np.any(c != 0):
                    continue
                idx = []
                for oid, sid in enumerate(p.indices):
                    n = lead[oid]
                    shp = self.operands[oid].segments[sid][:n]
                    sub = 0
                    for ch, d in zip(self.operand_subscripts[oid][:n], shp):
                        sub = sub * d + at[ch]
                    idx.append(first_new[oid][sid] + sub)
                new_paths.append(Path(tuple(idx), c))
        return SegmentedTensorProduct(
            tuple(s[n:] for s, n in zip(self.operand_subscripts, lead)), new_cs, new_ops, new_paths
        )

    def flatten_coefficient_modes(self) -> "SegmentedTensorProduct":
        return self.flatten_modes(self.coefficient_subscripts)

    def squeeze_modes(self) -> "SegmentedTensorProduct":
        """Drop every mode whose extent is 1 in all segments that carry it."""
        extents: dict[str, set] = {}
        for s, op in zip(self.operand_subscripts, self.operands):
            for seg in op.segments:
                for ch, d in zip(s, seg):
                    extents.setdefault(ch, set()).add(d)
        for p in self.paths:
            for ch, d in zip(self.coefficient_subscripts, p.coefficients.shape):
                extents.setdefault(ch, set()).add(d)
        drop = {ch for ch, e in extents.items() if e == {1}}
        if not drop:
            return self
        new_subs = tuple("".join(ch for ch in s if ch not in drop) for s in self.operand_subscripts)
        new_ops = [
            Operand(len(ns), tuple(tuple(d for ch, d in zip(s, seg) if ch not in drop) for seg in op.segments))
            for s, ns, op in zip(self.operand_subscripts, new_subs, self.operands)
        ]
        cs = self.coefficient_subscripts
        axes = tuple(a for a, ch in enumerate(cs) if ch in drop)
        new_paths = [Path(p.indices, np.squeeze(p.coefficients, axis=axes) if axes else p.coefficients) for p in self.paths]
        return SegmentedTensorProduct(new_subs, "".join(ch for ch in cs if ch not in drop), new_ops, new_paths)

    def remove_zero_paths(self) -> "SegmentedTensorProduct":
        out = self.copy()
        out.paths = [p for p in self.paths if np.any(p.coefficients != 0)]
        return out

    # -- tables -----------------------------------------------------------------------
    def index_table(self) -> np.ndarray:
        return np.array([p.indices for p in self.paths], dtype=np.int64).reshape(self.num_paths, self.num_operands)

    def coefficient_table(self) -> np.ndarray:
        """Stacked coefficients ``[num_paths, ...]``; requires equal shapes across paths."""
        if not self.paths:
            return np.zeros((0,))
        return np.stack([p.coefficients for p in self.paths])

    def __repr__(self) -> str:
        return f"STP({self.subscripts} operands={self.operands} num_paths={self.num_paths})"

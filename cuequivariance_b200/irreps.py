"""Irreducible representations of O(3)/SO(3) and the `Irreps` container.

Host-side bookkeeping only: which (multiplicity, irrep) blocks an operand holds, in
which order, and in which memory layout.  Conventions follow the reference so that a
descriptor built here lines up segment for segment with one built there:

* ordering of O3 irreps: by ``l`` first, then the "natural" parity ``(-1)**l`` before
  the other one (reference: cuequivariance/group_theory/representations/irrep_o3.py:86-88);
* product rule ``ir1 * ir2`` enumerates ``|l1-l2| .. l1+l2`` ascending with parity
  ``p1*p2`` (irrep_o3.py:61-67, irrep_so3.py:68-72);
* string syntax ``"128x0e + 3x1o"`` (group_theory/irreps_array/irreps.py:39-120);
* layouts ``mul_ir`` (channel-major) / ``ir_mul`` (component-major)
  (group_theory/irreps_array/irreps_layout.py:23-89).
"""
from __future__ import annotations

import enum
import re
from dataclasses import dataclass
from typing import Iterable, Iterator, Sequence, Union


@dataclass(frozen=True)
class Irrep:
    """One irrep of O(3) (``p`` = +1/-1) or of SO(3) (``p`` = 0, no parity label)."""

    l: int  # noqa: E741
    p: int = 0

    def __post_init__(self):
        if self.l < 0 or self.p not in (-1, 0, 1):
            raise ValueError(f"invalid irrep l={self.l} p={self.p}")

    # -- identity ---------------------------------------------------------------
    @property
    def group(self) -> str:
        return "SO3" if self.p == 0 else "O3"

    @property
    def dim(self) -> int:
        return 2 * self.l + 1

    def is_scalar(self) -> bool:
        return self.l == 0 and self.p in (0, 1)

    def __repr__(self) -> str:
        if self.p == 0:
            return f"{self.l}"
        return f"{self.l}{'e' if self.p > 0 else 'o'}"

    # -- ordering ---------------------------------------------------------------
    def _key(self):
        if self.p == 0:
            return (self.l, 0)
        return (self.l, -self.p * (-1) ** self.l)

    def __lt__(self, other: "Irrep") -> bool:
        return self._key() < other._key()

    # -- selection rule ---------------------------------------------------------
    def __mul__(self, other: "Irrep") -> list["Irrep"]:
        if (self.p == 0) != (other.p == 0):
            raise ValueError("cannot mix O3 and SO3 irreps")
        return [
            Irrep(l, self.p * other.p)
            for l in range(abs(self.l - other.l), self.l + other.l + 1)  # noqa: E741
        ]

    @staticmethod
    def parse(group: str, s: Union[str, "Irrep"]) -> "Irrep":
        if isinstance(s, Irrep):
            return s
        if hasattr(s, "l"):  # duck-typed cue.O3 / cue.SO3
            return Irrep(int(s.l), int(getattr(s, "p", 0)))
        s = s.strip()
        if group == "O3":
            m = re.fullmatch(r"(\d+)([eo])", s)
            if not m:
                raise ValueError(f"cannot parse O3 irrep {s!r}")
            return Irrep(int(m.group(1)), 1 if m.group(2) == "e" else -1)
        if group == "SO3":
            if not re.fullmatch(r"\d+", s):
                raise ValueError(f"cannot parse SO3 irrep {s!r}")
            return Irrep(int(s), 0)
        raise ValueError(f"unsupported group {group!r} (O3 and SO3 are available)")


class IrrepsLayout(enum.Enum):
    """``mul_ir``: index = channel*dim + component;  ``ir_mul``: component*mul + channel."""

    mul_ir = "mul_ir"
    ir_mul = "ir_mul"

    def shape(self, mul: int, dim: int) -> tuple[int, int]:
        return (mul, dim) if self is IrrepsLayout.mul_ir else (dim, mul)

    @staticmethod
    def parse(x) -> "IrrepsLayout":
        if x is None:
            return IrrepsLayout.mul_ir
        if isinstance(x, IrrepsLayout):
            return x
        name = getattr(x, "name", x)  # cue.IrrepsLayout members have .name
        return IrrepsLayout[str(name)]


mul_ir = IrrepsLayout.mul_ir
ir_mul = IrrepsLayout.ir_mul


class Irreps:
    """Ordered list of ``(mul, Irrep)`` blocks, all of one group."""

    __slots__ = ("group", "blocks")

    def __init__(self, group: str = None, blocks=None):
        if blocks is None and not (isinstance(group, str) and group in ("O3", "SO3")):
            group, blocks = None, group
        if isinstance(blocks, Irreps):
            group = group or blocks.group
            blocks = list(blocks.blocks)
        elif hasattr(blocks, "irrep_class") and not isinstance(blocks, str):
            # duck-typed cue.Irreps
            group = blocks.irrep_class.__name__
            blocks = [(int(m), Irrep.parse(group, ir)) for m, ir in blocks]
        if group is not None and not isinstance(group, str):
            group = getattr(group, "__name__", str(group))
        if isinstance(blocks, str):
            if group is None:
                group = "O3" if re.search(r"\d[eo]", blocks) else "SO3"
            parsed = []
            for term in blocks.split("+"):
                term = term.strip()
                if not term:
                    continue
                if "x" in term:
                    m, ir = term.split("x")
                    parsed.append((int(m), Irrep.parse(group, ir)))
                else:
                    parsed.append((1, Irrep.parse(group, term)))
            blocks = parsed
        else:
            out = []
            for b in blocks or []:
                if isinstance(b, (tuple, list)):
                    m, ir = b
                else:
                    m, ir = 1, b
                if group is None and isinstance(ir, Irrep):
                    group = ir.group
                out.append((int(m), Irrep.parse(group or "O3", ir)))
            blocks = out
        self.group = group or "O3"
        self.blocks = tuple((m, ir) for m, ir in blocks)
        for _, ir in self.blocks:
            if ir.group != self.group:
                raise ValueError(f"irrep {ir} does not belong to {self.group}")

    # -- container protocol -----------------------------------------------------
    def __iter__(self) -> Iterator[tuple[int, Irrep]]:
        return iter(self.blocks)

    def __len__(self) -> int:
        return len(self.blocks)

    def __getitem__(self, i):
        if isinstance(i, slice):
            return Irreps(self.group, self.blocks[i])
        return self.blocks[i]

    def __eq__(self, other) -> bool:
        return isinstance(other, Irreps) and (self.group, self.blocks) == (other.group, other.blocks)

    def __hash__(self):
        return hash((self.group, self.blocks))

    def __repr__(self) -> str:
        return "+".join(f"{m}x{ir}" if m != 1 else f"{ir}" for m, ir in self.blocks)

    def __rmul__(self, k: int) -> "Irreps":
        return Irreps(self.group, [(k * m, ir) for m, ir in self.blocks])

    def __add__(self, other: "Irreps") -> "Irreps":
        return Irreps(self.group, self.blocks + Irreps(self.group, other).blocks)

    # -- queries ----------------------------------------------------------------
    @property
    def dim(self) -> int:
        return sum(m * ir.dim for m, ir in self.blocks)

    @property
    def muls(self) -> list[int]:
        return [m for m, _ in self.blocks]

    @property
    def num_irreps(self) -> int:
        return sum(self.muls)

    def slices(self) -> list[slice]:
        out, off = [], 0
        for m, ir in self.blocks:
            out.append(slice(off, off + m * ir.dim))
            off += m * ir.dim
        return out

    def sort(self):
        """Stable sort by irrep.  Returns ``(sorted, perm, inv)`` with
        ``sorted[perm[i]] = self[i]`` and ``sorted[j] = self[inv[j]]``."""
        order = sorted(range(len(self.blocks)), key=lambda i: (self.blocks[i][1]._key(), i))
        inv = tuple(order)
        perm = tuple(inv.index(i) for i in range(len(inv)))
        return Irreps(self.group, [self.blocks[i] for i in order]), perm, inv

    def simplify(self) -> "Irreps":
        out: list[list] = []
        for m, ir in self.blocks:
            if m == 0:
                continue
            if out and out[-1][1] == ir:
                out[-1][0] += m
            else:
                out.append([m, ir])
        return Irreps(self.group, [(m, ir) for m, ir in out])

    def set_mul(self, mul: int) -> "Irreps":
        return Irreps(self.group, [(mul, ir) for _, ir in self.blocks])

    def new_scalars(self, mul: int) -> "Irreps":
        return Irreps(self.group, [(mul, Irrep(0, 1 if self.group == "O3" else 0))])

    def filter(self, keep: Iterable) -> "Irreps":
        keep = parse_irrep_list(self.group, keep)
        return Irreps(self.group, [(m, ir) for m, ir in self.blocks if ir in keep])

    def is_scalar(self) -> bool:
        return all(ir.is_scalar() for _, ir in self.blocks)


def parse_irrep_list(group: str, items) -> list[Irrep]:
    """Accepts an `Irreps`, a string ``"0e+1o"``, or a sequence of irreps/strings."""
    if items is None:
        return None
    if isinstance(items, Irreps):
        return [ir for _, ir in items]
    if isinstance(items, str):
        return [ir for _, ir in Irreps(group, items)]
    if hasattr(items, "irrep_class"):
        return [ir for _, ir in Irreps(items)]
    return [Irrep.parse(group, x) for x in items]


IrrepsLike = Union[Irreps, str, Sequence]

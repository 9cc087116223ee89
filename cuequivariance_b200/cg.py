"""Clebsch-Gordan tensors for real irreps of SO(3)/O(3).

The coupling tensor ``C[i, j, k]`` maps ``x1[i] * x2[j]`` (components of irreps l1, l2 in
the real basis) onto component ``k`` of irrep l3.  Convention = the reference's
(cuequivariance/group_theory/representations/irrep_su2.py:188-279 for the complex SU(2)
coefficients, which are the textbook Condon-Shortley ones and are NOT divided by
``sqrt(2*l3+1)``; irrep_so3.py:29-41,81-96 for the change to the real basis, which carries
an extra phase ``(-i)**l`` so that the real-basis tensor is real; irrep_o3.py:70-77 for
the parity rule).  The arithmetic here is a restatement: Racah's closed form evaluated
with exact rationals, then one change of basis in complex128.
"""
from __future__ import annotations

from fractions import Fraction
from functools import lru_cache
from math import factorial, sqrt

import numpy as np

from .irreps import Irrep


def _su2_coefficient(j1: int, m1: int, j2: int, m2: int, j3: int, m3: int) -> float:
    """<j1 m1 j2 m2 | j3 m3> for integer spins (Racah's formula, exact until the last sqrt)."""
    if m1 + m2 != m3 or not (abs(j1 - j2) <= j3 <= j1 + j2):
        return 0.0
    if abs(m1) > j1 or abs(m2) > j2 or abs(m3) > j3:
        return 0.0
    f = factorial
    tri = Fraction(
        f(j1 + j2 - j3) * f(j1 - j2 + j3) * f(-j1 + j2 + j3), f(j1 + j2 + j3 + 1)
    )
    pref = (2 * j3 + 1) * tri * (
        f(j3 + m3) * f(j3 - m3) * f(j1 - m1) * f(j1 + m1) * f(j2 - m2) * f(j2 + m2)
    )
    kmin = max(0, j2 - j3 - m1, j1 - j3 + m2)
    kmax = min(j1 + j2 - j3, j1 - m1, j2 + m2)
    s = Fraction(0)
    for k in range(kmin, kmax + 1):
        den = (
            f(k) * f(j1 + j2 - j3 - k) * f(j1 - m1 - k) * f(j2 + m2 - k)
            * f(j3 - j2 + m1 + k) * f(j3 - j1 - m2 + k)
        )
        s += Fraction((-1) ** k, den)
    val = sqrt(pref * s * s)  # Fraction -> float only here
    return val if s > 0 else -val


def su2_clebsch_gordan(j1: int, j2: int, j3: int) -> np.ndarray:
    """Complex-basis coupling array indexed ``[j1+m1, j2+m2, j3+m3]`` (m ascending)."""
    out = np.zeros((2 * j1 + 1, 2 * j2 + 1, 2 * j3 + 1))
    for m1 in range(-j1, j1 + 1):
        for m2 in range(-j2, j2 + 1):
            m3 = m1 + m2
            if abs(m3) <= j3:
                out[j1 + m1, j2 + m2, j3 + m3] = _su2_coefficient(j1, m1, j2, m2, j3, m3)
    return out


def real_to_complex(l: int) -> np.ndarray:  # noqa: E741
    """Unitary ``Q[complex m, real component]`` of the real spherical basis, times ``(-i)**l``."""
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    r = 1.0 / sqrt(2.0)
    q[l, l] = 1.0
    for m in range(1, l + 1):
        sgn = (-1.0) ** m
        # negative m row
        q[l - m, l + m] = r
        q[l - m, l - m] = -1j * r
        # positive m row
        q[l + m, l + m] = sgn * r
        q[l + m, l - m] = 1j * sgn * r
    return q * (-1j) ** l


@lru_cache(maxsize=None)
def so3_clebsch_gordan(l1: int, l2: int, l3: int) -> np.ndarray:
    """Real-basis coupling tensor of shape ``(n_solutions, 2l1+1, 2l2+1, 2l3+1)``;
    ``n_solutions`` is 1 inside the triangle rule, else 0."""
    if not (abs(l1 - l2) <= l3 <= l1 + l2):
        return np.zeros((0, 2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1))
    c = su2_clebsch_gordan(l1, l2, l3).astype(np.complex128)
    q1, q2, q3 = real_to_complex(l1), real_to_complex(l2), real_to_complex(l3)
    # real[a,b,c] = sum_{i,k,n} q1[i,a] q2[k,b] conj(q3[n,c]) c[i,k,n]
    t = np.tensordot(q1, c, axes=([0], [0]))            # a,k,n
    t = np.tensordot(q2, t, axes=([0], [1]))            # b,a,n
    t = np.tensordot(t, np.conj(q3), axes=([2], [0]))   # b,a,c
    t = np.transpose(t, (1, 0, 2))
    if np.abs(t.imag).max() > 1e-9:
        raise AssertionError("real-basis Clebsch-Gordan tensor has an imaginary part")
    out = np.ascontiguousarray(t.real)[None]
    out.setflags(write=False)
    return out


def clebsch_gordan(ir1: Irrep, ir2: Irrep, ir3: Irrep) -> np.ndarray:
    """``(n_solutions, dim1, dim2, dim3)`` coupling tensors for O3 or SO3 irreps."""
    if ir1.p * ir2.p != ir3.p:
        return np.zeros((0, ir1.dim, ir2.dim, ir3.dim))
    return so3_clebsch_gordan(ir1.l, ir2.l, ir3.l)

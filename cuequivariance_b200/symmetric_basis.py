"""Basis of the symmetric powers of a representation, restricted to given output irreps.

``symmetric_power_basis(irreps, n, ir)`` returns ``U[a_1, .., a_n, i, w]``: for every ``w`` an
equivariant map from the ``n``-fold tensor power of ``V = irreps`` (multiplicity one per block) to the
irrep ``ir`` that is symmetric under every permutation of ``a_1 .. a_n``; the ``w`` together span all of
them.  This is what the symmetric contraction of MACE contracts with its weights; the reference builds it
with ``cue.reduced_symmetric_tensor_product_basis`` (cuequivariance/group_theory/irreps_array/
reduced_tensor_product.py:147, used by descriptors/symmetric_contractions.py:62-72).

Construction used here (independent of the reference's):

1. couple step by step with Clebsch-Gordan tensors: every chain
   ``(((ir_1 x ir_2 -> j_2) x ir_3 -> j_3) ... x ir_n -> ir)`` over the blocks of ``V`` gives one equivariant
   map of the full tensor power onto ``ir``, and the chains together span all of them;
2. symmetrise each chain tensor over the ``n`` input slots (average over the permutations);
3. keep a maximal linearly independent subset, orthonormalised by modified Gram-Schmidt in chain order
   (deterministic: no eigen-decomposition whose degenerate subspaces could rotate between machines).

The basis of such a space is not unique: two valid bases differ by an invertible mixing of the ``w``
axis, i.e. by a linear change of the weights.  The number of basis elements is an invariant and equals the
reference's.
"""
from __future__ import annotations

import itertools
from typing import Sequence

import numpy as np

from .cg import clebsch_gordan
from .irreps import Irrep


def _block_offsets(blocks: Sequence[Irrep]):
    offs, o = [], 0
    for ir in blocks:
        offs.append(o)
        o += ir.dim
    return offs, o


def _coupled_chains(blocks: Sequence[Irrep], degree: int, target: Irrep):
    """Yields tensors ``[D]*degree + [target.dim]``, one per coupling chain that ends in ``target``."""
    offs, D = _block_offsets(blocks)
    # level 1: the embedding of every block
    level = []
    for ir, o in zip(blocks, offs):
        t = np.zeros((D, ir.dim))
        t[o : o + ir.dim] = np.eye(ir.dim)
        level.append((ir, t))
    for k in range(2, degree + 1):
        nxt = []
        last = k == degree
        for irA, tA in level:
            for irB, o in zip(blocks, offs):
                for irC in irA * irB:
                    if last and irC != target:
                        continue
                    if not last and not _can_reach(irC, blocks, degree - k, target):
                        continue
                    for cg in clebsch_gordan(irA, irB, irC):
                        # t[..., a_k, mC] = sum_{mA, mB} tA[..., mA] * [a_k = o + mB] * cg[mA, mB, mC]
                        part = np.tensordot(tA, cg, axes=([tA.ndim - 1], [0]))        # [..., dB, dC]
                        t = np.zeros(tA.shape[:-1] + (D, irC.dim))
                        t[..., o : o + irB.dim, :] = part
                        nxt.append((irC, t))
        level = nxt
    for ir, t in level:
        if ir == target:
            yield t


def _can_reach(j: Irrep, blocks: Sequence[Irrep], steps: int, target: Irrep) -> bool:
    """Can ``steps`` further couplings with blocks of V turn ``j`` into ``target``?  (|l| triangle rule and
    parity: each step changes l by at most the block's l and multiplies the parity.)"""
    if steps == 0:
        return j == target
    lmax = max(b.l for b in blocks)
    if abs(j.l - target.l) > steps * lmax:
        return False
    frontier = {j}
    for _ in range(steps):
        frontier = {c for a in frontier for b in blocks for c in a * b}
    return target in frontier


def _symmetrise(t: np.ndarray, degree: int) -> np.ndarray:
    acc = np.zeros_like(t)
    perms = list(itertools.permutations(range(degree)))
    for perm in perms:
        acc += np.transpose(t, perm + (degree,))
    return acc / len(perms)


def symmetric_power_basis(blocks: Sequence[Irrep], degree: int, target: Irrep, tol: float = 1e-9) -> np.ndarray:
    """``U[a_1..a_degree, i, w]`` (may have zero columns ``w`` when the target does not occur)."""
    blocks = tuple(blocks)
    _, D = _block_offsets(blocks)
    shape = (D,) * degree + (target.dim,)
    basis = []          # orthonormal, flattened
    for t in _coupled_chains(blocks, degree, target):
        v = _symmetrise(t, degree).reshape(-1)
        n0 = np.linalg.norm(v)
        if n0 < tol:
            continue
        v = v / n0
        for _ in range(2):                      # modified Gram-Schmidt, twice for stability
            for b in basis:
                v = v - np.dot(b, v) * b
        n1 = np.linalg.norm(v)
        if n1 > 1e-6:
            basis.append(v / n1)
    if not basis:
        return np.zeros(shape + (0,))
    U = np.stack(basis, axis=-1).reshape(shape + (len(basis),))
    U[np.abs(U) < 1e-12] = 0.0
    return U

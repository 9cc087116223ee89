"""Polynomials that have a kernel written out at build time ("static" kernels).

For a polynomial whose path list is known when the library is built, the whole evaluation
of one (row, channel) pair can be emitted as straight-line FP32 code: every operand segment
is loaded into a register once, every path is a couple of multiplies, and permutation-
equivalent paths of repeated operands (x*x*x) are merged.  The reference obtains the same
effect by JIT-compiling one kernel per polynomial with NVRTC (CHANGELOG.md:38,49); here the
source is generated ahead of time by ``csrc/gen_u1d_static.py`` for the polynomials listed in
`registered_polynomials` and matched at run time by a digest of the serialised tables.
"""
from __future__ import annotations

import hashlib
import struct
from typing import Dict, List, Tuple

import numpy as np

from .polynomial import Operation, Polynomial
from .stp import Path, SegmentedTensorProduct


def merge_symmetric_paths(poly: Polynomial) -> Polynomial:
    """Within each operation, paths that differ only by a permutation of the segment indices
    of operands bound to the same buffer describe the same monomial; they are merged (their
    coefficients added).  The polynomial function is unchanged."""
    new_ops = []
    for ope, stp in poly.operations:
        groups: Dict[int, List[int]] = {}
        for k, b in enumerate(ope.buffers):
            groups.setdefault(b, []).append(k)
        acc: Dict[Tuple[int, ...], float] = {}
        order: List[Tuple[int, ...]] = []
        for p in stp.paths:
            idx = list(p.indices)
            for ks in groups.values():
                if len(ks) > 1:
                    vals = sorted(idx[k] for k in ks)
                    for k, v in zip(ks, vals):
                        idx[k] = v
            key = tuple(idx)
            if key not in acc:
                acc[key] = 0.0
                order.append(key)
            acc[key] += float(p.coefficients)
        d = stp.copy()
        d.paths = [Path(k, np.float64(acc[k])) for k in order if acc[k] != 0.0]
        new_ops.append((ope, d))
    return Polynomial(poly.inputs, poly.outputs, new_ops)


def digest(poly: Polynomial) -> str:
    """Digest of the structure a static kernel depends on: segment counts, scalar/vector kind,
    operations, path indices and coefficients (float64 bit patterns) - not the extent."""
    h = hashlib.sha1()
    h.update(struct.pack("<ii", poly.num_inputs, poly.num_outputs))
    for o in poly.operands:
        h.update(struct.pack("<ii", o.ndim, o.num_segments))
    for ope, stp in poly.operations:
        h.update(struct.pack(f"<{len(ope.buffers) + 1}i", len(ope.buffers), *ope.buffers))
        for p in stp.paths:
            h.update(struct.pack(f"<{len(p.indices)}i", *p.indices))
            h.update(struct.pack("<d", float(p.coefficients)))
    return h.hexdigest()[:16]


def registered_polynomials() -> List[Tuple[str, Polynomial]]:
    """(name, flattened polynomial) of everything that gets a static kernel: the MACE
    symmetric contraction 0e+1o+2e+3o -> 0e+1o of degree 3 and its first derivatives."""
    from . import descriptors

    out = []
    e, _ = descriptors.symmetric_contraction("4x0e+4x1o+4x2e+4x3o", "4x0e+4x1o", (1, 2, 3))
    fwd = e.polynomial.flatten_coefficient_modes().squeeze_modes()
    out.append(("sc_l3_l1_d3_fwd", fwd))
    out.append(("sc_l3_l1_d3_bwd_wx", fwd.backward([True, True], [True])))
    out.append(("sc_l3_l1_d3_bwd_x", fwd.backward([False, True], [True])))
    out.append(("sc_l3_l1_d3_bwd_w", fwd.backward([True, False], [True])))
    return out

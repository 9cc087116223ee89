"""Writes the symmetric-contraction path tables shipped in this directory.

The basis of the symmetric powers (which linear combinations of x(x)x(x)x transform as a
given irrep) is not unique; to be a drop-in for the reference the tables must be the
reference's own.  This script runs the reference's descriptor
(cuequivariance/group_theory/experimental/mace/symmetric_contractions.py:27-130) for the
usual MACE shapes and stores segment counts, path indices, coefficients and the
projection matrix.  The tables do not depend on the multiplicity.

    python cuequivariance_b200/data/make_symmetric_contraction_tables.py /path/to/reference
"""
import itertools
import os
import sys
import types

import numpy as np


def main(root, outdir):
    import torch  # noqa: F401  (before the stub, so torch.einsum keeps its own contraction order)

    if "opt_einsum" not in sys.modules:
        m = types.ModuleType("opt_einsum")
        m.contract_path = lambda s, *shapes, **kw: ([(0, 1)] * (len(shapes) - 1), types.SimpleNamespace(naive_cost=1, opt_cost=1))
        sys.modules["opt_einsum"] = m
    sys.path.insert(0, f"{root}/cuequivariance")
    import cuequivariance as cue
    from cuequivariance.group_theory.experimental.mace import symmetric_contraction

    ins = ["0e", "0e+1o", "0e+1o+2e", "0e+1o+2e+3o"]
    outs = ["0e", "0e+1o", "0e+1o+2e"]
    for s_in, s_out, deg in itertools.product(ins, outs, [1, 2, 3]):
        if s_out.count("+") > s_in.count("+"):
            continue
        ir_in = cue.Irreps("O3", "+".join("2x" + t for t in s_in.split("+")))
        ir_out = cue.Irreps("O3", "+".join("2x" + t for t in s_out.split("+")))
        e, proj = symmetric_contraction(ir_in, ir_out, tuple(range(1, deg + 1)))
        poly = e.polynomial
        t = {"projection": proj, "num_operations": np.int64(len(poly.operations)),
             "num_segments": np.array([o.num_segments for o in poly.operands], dtype=np.int64)}
        for k, (ope, d) in enumerate(poly.operations):
            t[f"op{k}_buffers"] = np.array(ope.buffers, dtype=np.int64)
            t[f"op{k}_indices"] = np.array([p.indices for p in d.paths], dtype=np.int32).reshape(d.num_paths, d.num_operands)
            t[f"op{k}_coefficients"] = np.array([float(p.coefficients) for p in d.paths])
        name = f"sc__{s_in.replace('+', '_')}__{s_out.replace('+', '_')}__deg{deg}.npz"
        np.savez_compressed(os.path.join(outdir, name), **t)
        print(name, [d.num_paths for _, d in poly.operations])


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(f"usage: python {sys.argv[0]} <path of the cuEquivariance reference checkout>")
    main(sys.argv[1], os.path.dirname(os.path.abspath(__file__)))

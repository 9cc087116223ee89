"""Makes the staged reference (``baseline/_ref``, see ``stage_reference.py``) importable.

``activate()`` must run after ``import torch``: the reference imports ``opt_einsum`` (only
its ``flop()`` helper uses it) and that package is not installed; a stand-in module is put
into ``sys.modules`` here.  If such a module were importable *before* torch is imported,
torch would route every ``einsum`` through it, which is why the stand-in is created in
memory instead of being a file on ``sys.path``.  With ``with_kernels=True`` this library's
replacement for the closed ``cuequivariance_ops_torch`` package is installed as well, so the
reference front-end dispatches ``uniform_1d`` / ``fused_tp`` to the CUDA kernels of this
repository; without it the reference only has its ``naive`` method.
"""
from __future__ import annotations

import math
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.isdir(os.path.join(REF, "cuequivariance")) and os.path.isdir(os.path.join(REF, "cuequivariance_torch"))


def activate(with_kernels: bool = False):
    import torch  # noqa: F401  (before the stand-in, see above)

    if not available():
        raise RuntimeError("the reference is not staged under baseline/_ref (run baseline/stage_reference.py where the checkout exists)")
    if "opt_einsum" not in sys.modules:
        m = types.ModuleType("opt_einsum")

        def contract_path(subscripts, *shapes, **kw):
            dims = {}
            ins = subscripts.split("->")[0].split(",")
            for s, shp in zip(ins, shapes):
                for ch, d in zip(s, shp):
                    dims[ch] = d
            cost = math.prod(dims.values())
            return [(0, 1)] * (len(ins) - 1), types.SimpleNamespace(naive_cost=cost, opt_cost=cost)

        m.contract_path = contract_path
        sys.modules["opt_einsum"] = m
    if REF not in sys.path:
        sys.path.insert(0, REF)
    if with_kernels:
        root = os.path.dirname(HERE)
        if root not in sys.path:
            sys.path.insert(0, root)
        from cuequivariance_b200 import compat

        compat.install()
    import cuequivariance as cue
    import cuequivariance_torch as cuet

    return cue, cuet

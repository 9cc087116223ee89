"""Drop-in for the closed ``cuequivariance_ops_torch`` package.

The open reference front-end (``cuequivariance_torch``) looks for a module of that name and,
if it is importable, sends its polynomials to ``torch.ops.cuequivariance.uniform_1d`` and its
layout changes to ``segmented_transpose`` (cuequivariance_torch/primitives/
segmented_polynomial.py:37-42, segmented_polynomial_uniform_1d.py:24-77, transpose.py:171-183).
``install()`` makes the package in this directory importable under that name, so an
unmodified ``cuequivariance_torch`` runs on the B200 kernels of this repository.
"""
import os
import sys


def install() -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    if here not in sys.path:
        sys.path.insert(0, here)
    import cuequivariance_ops_torch  # noqa: F401

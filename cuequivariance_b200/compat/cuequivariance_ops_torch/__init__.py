"""Stand-in for the closed ``cuequivariance_ops_torch`` package, backed by cuequivariance_b200.

Provides what the open front-end imports for the segmented-polynomial path:
``uniform_1d`` (constants + the registered op ``torch.ops.cuequivariance.uniform_1d``),
``FusedTensorProductOp3`` / ``FusedTensorProductOp4``, ``indexed_linear`` and ``segmented_transpose``.
The triangle ops are not provided; asking for them raises ImportError/AttributeError, which the
front-end turns into its documented fallback.
"""
from . import uniform_1d  # noqa: F401  (registers the op)
from .fused_tensor_product import FusedTensorProductOp3, FusedTensorProductOp4  # noqa: F401
from .indexed_linear import indexed_linear  # noqa: F401
from .uniform_1d import segmented_transpose  # noqa: F401

__version__ = "0.0.0+cueq_b200"

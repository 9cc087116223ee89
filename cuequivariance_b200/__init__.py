"""cuequivariance_b200: a B200-native (sm_100a) executor for cuEquivariance's
segmented-polynomial operations, behind the ``cuequivariance_torch`` module surface."""
from .irreps import Irrep, Irreps, IrrepsLayout, mul_ir, ir_mul
from .cg import clebsch_gordan
from .stp import Operand, Path, SegmentedTensorProduct
from .polynomial import Operation, Polynomial
from . import descriptors
from .descriptors import EquivariantPolynomial, IrrepsAndLayout
from .segmented_polynomial import SegmentedPolynomial
from .transpose import TransposeIrrepsLayout, TransposeSegments
from .operations import (
    ChannelWiseTensorProduct,
    FullyConnectedTensorProduct,
    SymmetricContraction,
    SphericalHarmonics,
    spherical_harmonics,
    EquivariantTensorProduct,
    Linear,
)

from ._lib import check_status  # noqa: E402  (raises if a kernel reported a bounded wait that ran out)

__version__ = "0.1.0"

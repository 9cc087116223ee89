from .tp_channel_wise import ChannelWiseTensorProduct
from .tp_fully_connected import FullyConnectedTensorProduct
from .symmetric_contraction import SymmetricContraction
from .spherical_harmonics import SphericalHarmonics, spherical_harmonics
from .equivariant import EquivariantTensorProduct
from .linear import Linear

__all__ = [
    "ChannelWiseTensorProduct", "FullyConnectedTensorProduct", "SymmetricContraction",
    "SphericalHarmonics", "spherical_harmonics", "EquivariantTensorProduct", "Linear",
]

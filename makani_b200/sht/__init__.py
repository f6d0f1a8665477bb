from .legendre import legendre_table
from .quadrature import clenshaw_curtiss_weights, legendre_gauss_weights, lobatto_weights, precompute_latitudes
from .sht import InverseRealSHT, RealSHT
from .distributed import DistributedInverseRealSHT, DistributedRealSHT

__all__ = [
    "legendre_table", "clenshaw_curtiss_weights", "legendre_gauss_weights", "lobatto_weights",
    "precompute_latitudes", "RealSHT", "InverseRealSHT", "DistributedRealSHT", "DistributedInverseRealSHT",
]

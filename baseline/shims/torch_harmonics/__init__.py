"""Stand-in for `torch_harmonics` (absent from this image): real spherical harmonic transforms as
`torch.fft` along longitude + `torch.einsum` against a precomputed associated-Legendre table."""

from .sht import RealSHT, InverseRealSHT  # noqa: F401
from . import quadrature  # noqa: F401

__version__ = "0.6.5+standin"

"""Stand-in for the part of NVIDIA Modulus that `makani` imports (the package is absent from this image)."""

from .module import Module  # noqa: F401

__version__ = "0.0.0+standin"

from .activations import ComplexActivation, ComplexReLU
from .layers import MLP, DropPath, EncoderDecoder, InverseRealFFT2, PatchEmbed, RealFFT2
from .spectral_convolution import FactorizedSpectralConv, SpectralAttention, SpectralConv

__all__ = ["ComplexActivation", "ComplexReLU", "MLP", "DropPath", "EncoderDecoder", "InverseRealFFT2", "PatchEmbed",
           "RealFFT2", "FactorizedSpectralConv", "SpectralAttention", "SpectralConv"]

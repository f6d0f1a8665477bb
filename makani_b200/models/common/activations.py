"""Activations for complex spectral coefficients (behaviour of makani/models/common/activations.py:20-100)."""

from __future__ import annotations

import torch
import torch.nn as nn


class ComplexReLU(nn.Module):
    """ReLU-like non-linearities on complex tensors.

    mode "cartesian": ReLU on real and imaginary parts separately; "real": ReLU on the real part only;
    "modulus": ReLU(|z| + b) with the phase kept; "halfplane": negative_slope outside the right half plane.
    """

    def __init__(self, negative_slope: float = 0.0, mode: str = "real", bias_shape=None, scale: float = 1.0):
        super().__init__()
        self.mode = mode
        self.negative_slope = negative_slope
        if mode in ("modulus", "halfplane"):
            if bias_shape is not None:
                self.bias = nn.Parameter(scale * torch.ones(bias_shape, dtype=torch.float32))
            else:
                self.bias = nn.Parameter(scale * torch.ones(1, dtype=torch.float32))
        else:
            self.bias = None
        self.act = nn.LeakyReLU(negative_slope=negative_slope)

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        if self.mode == "cartesian":
            return torch.view_as_complex(self.act(torch.view_as_real(z)))
        if self.mode == "modulus":
            zabs = torch.sqrt(torch.square(z.real) + torch.square(z.imag))
            return z * (self.act(zabs + self.bias) / (zabs + 1e-12)).to(z.dtype)
        if self.mode == "halfplane":
            modified_angle = torch.angle(z) - self.bias
            cond = torch.logical_and((0.0 <= modified_angle), (modified_angle < torch.pi / 2.0))
            return torch.where(cond, z, self.negative_slope * z)
        if self.mode == "real":
            return torch.complex(self.act(z.real), z.imag)
        raise ValueError(f"unknown complex activation mode {self.mode}")


class ComplexActivation(nn.Module):
    """Wrap a real activation for complex input (same three placement modes)."""

    def __init__(self, activation: nn.Module, mode: str = "cartesian", bias_shape=None):
        super().__init__()
        self.mode = mode
        self.act = activation
        if mode == "modulus":
            self.bias = nn.Parameter(torch.zeros(bias_shape if bias_shape is not None else 1, dtype=torch.float32))
        else:
            # an unused one-element buffer, part of the state dict exactly as in makani/models/common/activations.py:81-83
            self.register_buffer("bias", torch.zeros(1, dtype=torch.float32))

    def forward(self, z):
        if self.mode == "cartesian":
            return torch.view_as_complex(torch.stack([self.act(z.real), self.act(z.imag)], dim=-1))
        if self.mode == "modulus":
            zabs = torch.sqrt(torch.square(z.real) + torch.square(z.imag))
            return z * (self.act(zabs + self.bias) / (zabs + 1e-12)).to(z.dtype)
        return z

"""Small elementwise helpers shared by the fused ops (torch fallbacks on CPU)."""

from __future__ import annotations

import torch


def dgelu_mul(dy: torch.Tensor, pre: torch.Tensor) -> torch.Tensor:
    """dy * GELU'(pre) (erf form, or the tanh form when that approximation is selected), computed in fp32 and returned
    in dy's dtype."""
    from . import _ext

    x = pre.float()
    if _ext.gelu_approximation() == "tanh":
        t = torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3))
        d = 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * 0.7978845608028654 * (1.0 + 3 * 0.044715 * x * x)
        return (dy.float() * d).to(dy.dtype)
    cdf = 0.5 * (1.0 + torch.erf(x * 0.7071067811865476))
    pdf = torch.exp(-0.5 * x * x) * 0.3989422804014327
    return (dy.float() * (cdf + x * pdf)).to(dy.dtype)

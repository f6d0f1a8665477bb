"""Small elementwise helpers shared by the fused ops (torch fallbacks on CPU)."""

from __future__ import annotations

import torch


def dgelu_mul(dy: torch.Tensor, pre: torch.Tensor) -> torch.Tensor:
    """dy * GELU'(pre) with the exact (erf) GELU, computed in fp32 and returned in dy's dtype."""
    x = pre.float()
    cdf = 0.5 * (1.0 + torch.erf(x * 0.7071067811865476))
    pdf = torch.exp(-0.5 * x * x) * 0.3989422804014327
    return (dy.float() * (cdf + x * pdf)).to(dy.dtype)

"""Low-rank parametrisations of the spectral weight tensor (dense / CP / Tucker / tensor-train).

The reference delegates these to tensorly / tltorch `FactorizedTensor`
(makani/models/common/factorizations.py:33-247, spectral_convolution.py:151-265).  Neither package is needed
here: each factorisation stores its factors as complex parameters, can be reconstructed to the dense weight
(`to_tensor`) and contracted directly with the input without reconstruction (`contract`).
"""

from __future__ import annotations

import math
from typing import List, Sequence

import torch
import torch.nn as nn

_LETTERS = "ioxyzuvw"


class FactorizedWeight(nn.Module):
    """Complex weight of shape `shape` = [Cin, (Cout), modes...] in a chosen factorisation."""

    def __init__(self, shape: Sequence[int], rank: float = 0.5, factorization: str = "cp", init_std: float = 0.02):
        super().__init__()
        self.shape = list(shape)
        self.factorization = factorization.lower()
        nd = len(self.shape)
        dense_numel = math.prod(self.shape)
        if self.factorization in ("dense", "complexdense"):
            self.factors = nn.ParameterList([nn.Parameter(init_std * torch.randn(*self.shape, dtype=torch.complex64))])
        elif self.factorization in ("cp", "complexcp"):
            r = max(1, int(rank * dense_numel / sum(self.shape))) if rank <= 1.0 else int(rank)
            self.rank = r
            scale = init_std ** (1.0 / nd)
            self.weights = nn.Parameter(torch.ones(r, dtype=torch.complex64))
            self.factors = nn.ParameterList([nn.Parameter(scale * torch.randn(s, r, dtype=torch.complex64)) for s in self.shape])
        elif self.factorization in ("tucker", "complextucker"):
            frac = rank ** (1.0 / nd) if rank <= 1.0 else None
            ranks = [max(1, int(round(s * frac))) if frac is not None else int(rank) for s in self.shape]
            self.ranks = ranks
            scale = init_std ** (1.0 / (nd + 1))
            self.core = nn.Parameter(scale * torch.randn(*ranks, dtype=torch.complex64))
            self.factors = nn.ParameterList([nn.Parameter(scale * torch.randn(s, r, dtype=torch.complex64) / math.sqrt(r))
                                             for s, r in zip(self.shape, ranks)])
        elif self.factorization in ("tt", "complextt"):
            rr = max(1, int(rank * min(self.shape))) if rank <= 1.0 else int(rank)
            ranks = [1] + [rr] * (nd - 1) + [1]
            self.ranks = ranks
            scale = init_std ** (1.0 / nd)
            self.factors = nn.ParameterList([
                nn.Parameter(scale * torch.randn(ranks[k], s, ranks[k + 1], dtype=torch.complex64) / math.sqrt(ranks[k]))
                for k, s in enumerate(self.shape)])
        else:
            raise ValueError(f"unknown factorization {factorization}")

    def to_tensor(self) -> torch.Tensor:
        nd = len(self.shape)
        idx = _LETTERS[:nd]
        f = self.factorization
        if f in ("dense", "complexdense"):
            return self.factors[0]
        if f in ("cp", "complexcp"):
            eq = ",".join(f"{c}r" for c in idx) + ",r->" + idx
            return torch.einsum(eq, *self.factors, self.weights)
        if f in ("tucker", "complextucker"):
            core_idx = "".join(chr(ord("A") + k) for k in range(nd))
            eq = core_idx + "," + ",".join(f"{c}{C}" for c, C in zip(idx, core_idx)) + "->" + idx
            return torch.einsum(eq, self.core, *self.factors)
        # tensor train
        out = self.factors[0]  # [1, s0, r1]
        for k in range(1, nd):
            out = torch.einsum("...a,abc->...bc", out, self.factors[k])
        return out.reshape(self.shape)

    def forward(self):
        return self.to_tensor()

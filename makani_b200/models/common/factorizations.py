"""Low-rank parametrisations of the spectral weight tensor (dense / CP / Tucker / tensor-train).

The reference delegates these to tensorly / tltorch `FactorizedTensor`
(makani/models/common/factorizations.py:33-247, spectral_convolution.py:151-265).  Neither package is needed
here: each factorisation stores its factors as complex parameters and is reconstructed to the dense weight
(`to_tensor`) before the contraction.
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


def get_contract_fun(weight, implementation: str = "reconstructed", separable: bool = False, operator_type: str = "diagonal",
                     complex: bool = True):
    """`(x, weight) -> x * weight` in spectral space for a dense or factorised weight, by the calling convention of
    makani/models/common/factorizations.py:212-247.  Both implementations ("reconstructed", "factorized") form the
    dense weight from the factors and apply the contraction of `operator_type`: reconstructing costs less than the
    contraction itself at the ranks and mode counts of these models, so no factor-by-factor path is kept."""
    from .contractions import get_contract_fun as dense_contraction

    if implementation not in ("reconstructed", "factorized"):
        raise ValueError(f"implementation must be 'reconstructed' or 'factorized', got {implementation!r}")
    if not (torch.is_tensor(weight) or isinstance(weight, FactorizedWeight)):
        raise ValueError(f"unexpected weight type {type(weight).__name__}")
    dense = dense_contraction(operator_type, separable)

    def as_complex(t):
        return torch.view_as_complex(t) if (complex and not t.is_complex() and t.shape[-1] == 2) else t

    def contract(x, w):
        w = w.to_tensor() if isinstance(w, FactorizedWeight) else w
        return dense(as_complex(x), as_complex(w))

    return contract

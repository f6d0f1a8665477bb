"""Stand-in for `tltorch.factorized_tensors.core.FactorizedTensor`: parameter containers for dense / CP / Tucker / TT
weights with the attributes the reference's contractions read (`weights`, `factors`, `core`, `to_tensor`)."""

import math

import torch
import torch.nn as nn


class FactorizedTensor(nn.Module):
    def __init__(self, shape, name):
        super().__init__()
        self.shape = tuple(shape)
        self.name = name

    @classmethod
    def new(cls, shape, rank="same", factorization="Dense", fixed_rank_modes=False, dtype=None, **kwargs):
        kind = factorization.lower()
        if kind in ("dense", "complexdense"):
            return _Dense(shape, dtype)
        if kind in ("cp", "complexcp"):
            return _CP(shape, rank, dtype)
        if kind in ("tucker", "complextucker"):
            return _Tucker(shape, rank, dtype)
        if kind in ("tt", "complextt"):
            return _TT(shape, rank, dtype)
        raise ValueError(f"unknown factorization {factorization}")

    def normal_(self, mean=0.0, std=1.0):
        with torch.no_grad():
            for p in self.parameters():
                p.normal_(mean, std)
        return self

    @property
    def is_complex(self):
        return next(self.parameters()).is_complex()


def _rank(shape, rank):
    if isinstance(rank, (int,)):
        return rank
    frac = 1.0 if rank == "same" else float(rank)
    return max(1, int(frac * math.prod(shape) / sum(shape)))


class _Dense(FactorizedTensor):
    def __init__(self, shape, dtype):
        super().__init__(shape, "Dense")
        self.tensor = nn.Parameter(torch.empty(*shape, dtype=dtype))

    def to_tensor(self):
        return self.tensor


class _CP(FactorizedTensor):
    def __init__(self, shape, rank, dtype):
        super().__init__(shape, "CP")
        r = _rank(shape, rank)
        self.rank = r
        self.weights = nn.Parameter(torch.ones(r, dtype=dtype))
        self.factors = nn.ParameterList([nn.Parameter(torch.empty(s, r, dtype=dtype)) for s in shape])

    def to_tensor(self):
        sub = "abcdefgh"[: len(self.shape)]
        eq = "r," + ",".join(c + "r" for c in sub) + "->" + sub
        return torch.einsum(eq, self.weights, *self.factors)


class _Tucker(FactorizedTensor):
    def __init__(self, shape, rank, dtype):
        super().__init__(shape, "Tucker")
        frac = 1.0 if rank == "same" else float(rank)
        ranks = [max(1, int(round(s * frac ** (1.0 / len(shape))))) for s in shape] if not isinstance(rank, (list, tuple)) else list(rank)
        self.rank = ranks
        self.core = nn.Parameter(torch.empty(*ranks, dtype=dtype))
        self.factors = nn.ParameterList([nn.Parameter(torch.empty(s, r, dtype=dtype)) for s, r in zip(shape, ranks)])

    def to_tensor(self):
        sub, rs = "abcdefgh"[: len(self.shape)], "ijklmnop"[: len(self.shape)]
        eq = rs + "," + ",".join(c + r for c, r in zip(sub, rs)) + "->" + sub
        return torch.einsum(eq, self.core, *self.factors)


class _TT(FactorizedTensor):
    def __init__(self, shape, rank, dtype):
        super().__init__(shape, "TT")
        r = _rank(shape, rank) if not isinstance(rank, (list, tuple)) else None
        ranks = [1] + ([r] * (len(shape) - 1) if r is not None else list(rank)[1:-1]) + [1]
        self.rank = ranks
        self.factors = nn.ParameterList(
            [nn.Parameter(torch.empty(ranks[i], s, ranks[i + 1], dtype=dtype)) for i, s in enumerate(shape)])

    def to_tensor(self):
        out = self.factors[0]
        for f in self.factors[1:]:
            out = torch.tensordot(out, f, dims=([-1], [0]))
        return out.squeeze(0).squeeze(-1)

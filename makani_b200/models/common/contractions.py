"""Complex tensor contractions used by the spectral filters (torch formulations).

Index convention: b batch, i input channel, o output channel, x degree l (or first mode index), y order m.
Hot variant on GPUs: "dhconv" (`bixy,iox->boxy`), which `makani_b200.ops.spectral` runs on the tensor cores; the
"diagonal" and the separable operators run as streaming kernels (`makani_b200.ops.spectral_modes`) on CUDA complex64
tensors; the einsum forms below serve CPU, other dtypes and the spectral-MLP products
(behaviour of makani/models/common/contractions.py:19-178).
"""

from __future__ import annotations

import torch

from ...ops import spectral_modes as _modes


def contract_diagonal(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return _modes.contract_diagonal(a, b)


def contract_dhconv(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.einsum("bixy,iox->boxy", a, b)


def contract_sep_diagonal(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return _modes.contract_sep_diagonal(a, b)


def contract_sep_dhconv(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return _modes.contract_sep_dhconv(a, b)


# spectral MLP products: weights are shared over all modes ("io") or depend on the degree ("xio")
def compl_mul2d_fwd(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a: real view [b,i,x,y,2], b: complex [i,o] -> real view [b,o,x,y,2]."""
    return torch.view_as_real(torch.einsum("bixy,io->boxy", torch.view_as_complex(a), b))


def compl_muladd2d_fwd(a, b, c):
    return torch.view_as_real(torch.einsum("bixy,io->boxy", torch.view_as_complex(a), b) + c)


def compl_exp_mul2d_fwd(a, b):
    return torch.view_as_real(torch.einsum("bixy,xio->boxy", torch.view_as_complex(a), b))


def compl_exp_muladd2d_fwd(a, b, c):
    return torch.view_as_real(torch.einsum("bixy,xio->boxy", torch.view_as_complex(a), b) + c)


def get_contract_fun(operator_type: str, separable: bool = False):
    table = {
        ("diagonal", False): contract_diagonal,
        ("diagonal", True): contract_sep_diagonal,
        ("dhconv", False): contract_dhconv,
        ("dhconv", True): contract_sep_dhconv,
    }
    try:
        return table[(operator_type, separable)]
    except KeyError:
        raise ValueError(f"unknown operator type {operator_type}")

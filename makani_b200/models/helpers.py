"""Model bookkeeping helpers (parameter counting across model-parallel shards; makani/models/helpers.py:22-44)."""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..utils import comm


def count_parameters(model: torch.nn.Module, device) -> int:
    """Global number of trainable parameters: every shard counted once, replicated tensors not multiplied."""
    with torch.no_grad():
        total = torch.zeros(1, dtype=torch.float64, device=device)
        for p in model.parameters():
            if not p.requires_grad:
                continue
            n = float(p.numel())
            for g in getattr(p, "is_shared_mp", ["model"]):
                n /= comm.get_size(g)
            total += n
        if comm.get_size("model") > 1:
            dist.all_reduce(total, group=comm.get_group("model"))
    return int(round(total.item()))


def check_parameters(model: torch.nn.Module) -> None:
    """Debug print of every trainable parameter's shape, strides and contiguity (makani/models/helpers.py:41-44)."""
    for name, p in model.named_parameters():
        if p.requires_grad:
            print(name, tuple(p.shape), p.stride(), p.is_contiguous())

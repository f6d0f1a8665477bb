"""Checkpoint formats.

"legacy": one file per model-parallel rank, `<path>.format(mp_rank=r)`, holding
    {iters, epoch, model_state (state_dict of the local shards), optimizer_state_dict, params[, scheduler_state_dict]}.
"flexible": one file (`mp_rank=0`) whose `model_state` holds *full* parameters, gathered along every dimension
    listed in `param.sharded_dims_mp`; on load each rank re-slices with the ceil-split rule, so a checkpoint can
    be restored under any (h, w, fin, fout) layout.
Format contract: makani/utils/trainer.py:890-1064.  Files written by the reference load here too: its pickled
`makani.utils.YParams.YParams` objects are mapped to this package's class and `module.` prefixes are stripped.
"""

from __future__ import annotations

import gc
import io
import logging
import pickle
from collections import OrderedDict

import torch
import torch.distributed as dist

from ..parallel.helpers import gather_uneven
from . import comm


class _RenamingUnpickler(pickle.Unpickler):
    """Resolves classes pickled under the reference's package name to this package."""

    def find_class(self, module, name):
        if module == "makani" or module.startswith("makani."):
            module = "makani_b200" + module[len("makani"):]
        return super().find_class(module, name)


class _PickleModule:
    Unpickler = _RenamingUnpickler
    __name__ = "pickle"

    @staticmethod
    def load(f, **kwargs):
        return _RenamingUnpickler(f, **kwargs).load()

    loads = staticmethod(pickle.loads)
    dump = staticmethod(pickle.dump)
    dumps = staticmethod(pickle.dumps)


def load_file(path: str):
    try:
        return torch.load(path, map_location="cpu", weights_only=False)
    except (ModuleNotFoundError, AttributeError):
        return torch.load(path, map_location="cpu", weights_only=False, pickle_module=_PickleModule)


def gather_full_state(model: torch.nn.Module) -> "OrderedDict[str, torch.Tensor]":
    """Full (un-sharded) parameters on the CPU; collective over the model-parallel groups."""
    state = OrderedDict()
    with torch.no_grad():
        for k, v in model.named_parameters():
            w = v.detach().clone()
            for d, group in enumerate(getattr(v, "sharded_dims_mp", [])):
                if group is not None and comm.get_size(group) > 1:
                    w = gather_uneven(w, d, group)
            state[k] = w.to("cpu")
    return state


def scatter_full_state(model: torch.nn.Module, state_dict, logger=None) -> None:
    """Copy this rank's shard of every full parameter in `state_dict` into the model."""
    state_dict = dict(state_dict)
    torch.nn.modules.utils.consume_prefix_in_state_dict_if_present(state_dict, "module.")
    with torch.no_grad():
        for k, v in model.named_parameters():
            if k not in state_dict:
                (logger or logging).warning(f"missing {k}")
                continue
            w = state_dict[k]
            for d, group in enumerate(getattr(v, "sharded_dims_mp", [])):
                if group is None or comm.get_size(group) == 1:
                    continue
                shard = (w.shape[d] + comm.get_size(group) - 1) // comm.get_size(group)
                w = torch.split(w, shard, dim=d)[comm.get_rank(group)]
            v.copy_(w)


def save_checkpoint(path_template: str, model, optimizer=None, scheduler=None, params=None, iters=0, epoch=0,
                    mode="flexible", world_rank=0, device=None) -> None:
    with torch.no_grad():
        if mode == "legacy":
            store = {"iters": iters, "epoch": epoch, "model_state": model.state_dict(), "params": params}
            if optimizer is not None:
                store["optimizer_state_dict"] = optimizer.state_dict()
            if scheduler is not None:
                store["scheduler_state_dict"] = scheduler.state_dict()
            torch.save(store, path_template.format(mp_rank=comm.get_rank("model")))
        elif mode == "flexible":
            store = {"iters": iters, "epoch": epoch, "model_state": gather_full_state(model), "params": params}
            if optimizer is not None:
                store["optimizer_state_dict"] = optimizer.state_dict()
            if scheduler is not None:
                store["scheduler_state_dict"] = scheduler.state_dict()
            if world_rank == 0:
                torch.save(store, path_template.format(mp_rank=0))
            if dist.is_initialized() and comm.get_size("model") > 1:
                dist.barrier(group=comm.get_group("model"))
        else:
            raise ValueError(f"Unknown checkpoint mode {mode}.")


def restore_checkpoint(path_template: str, model, optimizer=None, scheduler=None, mode="flexible", load_optimizer=False,
                       load_scheduler=False, load_counters=False, logger=None):
    """Returns (iters, epoch) from the file when `load_counters`, else (None, None)."""
    if mode == "legacy":
        ckpt = load_file(path_template.format(mp_rank=comm.get_rank("model")))
        state = ckpt["model_state"]
        torch.nn.modules.utils.consume_prefix_in_state_dict_if_present(state, "module.")
        model.load_state_dict(state, strict=True)
        if load_optimizer and optimizer is not None:
            optimizer.load_state_dict(ckpt["optimizer_state_dict"])
    elif mode == "flexible":
        ckpt = load_file(path_template.format(mp_rank=0))
        scatter_full_state(model, ckpt["model_state"], logger)
        if load_optimizer:
            raise NotImplementedError("restoring the optimizer is not supported for the flexible checkpoint format")
    else:
        raise ValueError(f"Unknown checkpoint mode {mode}.")
    if load_scheduler and scheduler is not None and "scheduler_state_dict" in ckpt:
        scheduler.load_state_dict(ckpt["scheduler_state_dict"])
    out = (ckpt.get("iters"), ckpt.get("epoch")) if load_counters else (None, None)
    del ckpt
    gc.collect()
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        torch.cuda.empty_cache()
        torch.cuda.synchronize()
    return out

"""Process topology: data x (h x w spatial) x (fin x fout channel) groups on top of torch.distributed.

API contract of the reference's `makani.utils.comm` (makani/utils/comm.py:32-153): `init(sizes, names)`
builds the group tree world -> {model -> {spatial -> {h, w}, matmul -> {fin, fout}}, data}; `get_size`,
`get_rank`, `get_group`, `get_root` by name; sizes/ranks are 1/0 when not distributed.

Rank order (the reference leaves it to an external package): the model block is contiguous in world rank
and inside it `fout` varies fastest, i.e.
    world_rank = (((d * H + h) * W + w) * Fin + fin) * Fout + fout
so that the ranks of one model instance sit on neighbouring GPUs of the NVSwitch domain.

Initialisation reads torchrun / SLURM / OpenMPI environment variables; backend is NCCL when CUDA is available
and gloo otherwise.
"""

from __future__ import annotations

import datetime
import math
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

_INITIALIZED = False
_WORLD_SIZE = 1
_WORLD_RANK = 0
_LOCAL_RANK = 0
_GROUPS: Dict[str, Optional[dist.ProcessGroup]] = {}
_GROUP_RANKS: Dict[str, List[List[int]]] = {}
_MY_GROUP_RANKS: Dict[str, List[int]] = {}
_SIZES: Dict[str, int] = {}

_LEAF_ORDER = ["h", "w", "fin", "fout"]  # slowest -> fastest inside the model block


def _env_int(*names, default=None):
    for n in names:
        if n in os.environ:
            return int(os.environ[n])
    return default


def get_size(name: str) -> int:
    if _WORLD_SIZE > 1 and name in _SIZES:
        return _SIZES[name]
    return 1


def get_rank(name: str) -> int:
    if _WORLD_SIZE > 1 and name in _MY_GROUP_RANKS:
        return _MY_GROUP_RANKS[name].index(_WORLD_RANK)
    return 0


def get_group(name: str):
    return _GROUPS.get(name, None)


def get_group_ranks(name: str) -> List[int]:
    """World ranks of this rank's group `name` (in group-rank order)."""
    return list(_MY_GROUP_RANKS.get(name, [_WORLD_RANK]))


def get_root(name: str) -> int:
    if _WORLD_SIZE > 1 and name in _MY_GROUP_RANKS:
        return min(_MY_GROUP_RANKS[name])
    return 0


def get_world_size() -> int:
    return _WORLD_SIZE


def get_world_rank() -> int:
    return _WORLD_RANK


def get_local_rank() -> int:
    return _LOCAL_RANK


def get_names() -> List[str]:
    return list(_GROUP_RANKS.keys())


def is_distributed(name: str) -> bool:
    return name in _GROUP_RANKS


def is_initialized() -> bool:
    return _INITIALIZED


def _coords(rank: int, sizes: Dict[str, int]):
    """world rank -> dict of coordinates for data, h, w, fin, fout."""
    c = {}
    r = rank
    for n in reversed(_LEAF_ORDER):
        c[n] = r % sizes[n]
        r //= sizes[n]
    c["data"] = r
    return c


def compute_group_ranks(world_size: int, sizes: Dict[str, int]) -> Dict[str, List[List[int]]]:
    """All groups of every kind as lists of world ranks (pure function, unit-testable)."""
    leaf = {n: int(sizes.get(n, 1)) for n in _LEAF_ORDER}
    model = math.prod(leaf.values())
    assert world_size % model == 0, f"world size {world_size} not divisible by model parallel size {model}"
    leaf["data"] = world_size // model
    coords = [_coords(r, leaf) for r in range(world_size)]

    def groups_varying(names):
        buckets: Dict[tuple, List[int]] = {}
        fixed = [n for n in ["data"] + _LEAF_ORDER if n not in names]
        for r, c in enumerate(coords):
            buckets.setdefault(tuple(c[n] for n in fixed), []).append(r)
        return [sorted(v) for _, v in sorted(buckets.items())]

    return {
        "world": [list(range(world_size))],
        "model": groups_varying(_LEAF_ORDER),
        "spatial": groups_varying(["h", "w"]),
        "matmul": groups_varying(["fin", "fout"]),
        "h": groups_varying(["h"]),
        "w": groups_varying(["w"]),
        "fin": groups_varying(["fin"]),
        "fout": groups_varying(["fout"]),
        "data": groups_varying(["data"]),
    }


def init(model_parallel_sizes=[1, 1, 1, 1], model_parallel_names=["h", "w", "fin", "fout"], verbose=False,
         timeout_s: Optional[float] = None, backend: Optional[str] = None) -> int:
    """Initialise torch.distributed (if launched with more than one process) and build all groups.

    Returns the model-parallel size (product of h, w, fin, fout)."""
    global _INITIALIZED, _WORLD_SIZE, _WORLD_RANK, _LOCAL_RANK
    world_size = _env_int("WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "SLURM_NTASKS", default=1)
    rank = _env_int("RANK", "OMPI_COMM_WORLD_RANK", "SLURM_PROCID", default=0)
    local_rank = _env_int("LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "SLURM_LOCALID", default=0)
    sizes = {n: int(s) for n, s in zip(model_parallel_names, model_parallel_sizes)}
    model_size = math.prod(sizes.values())

    _GROUPS.clear(); _GROUP_RANKS.clear(); _MY_GROUP_RANKS.clear(); _SIZES.clear()
    _WORLD_SIZE, _WORLD_RANK, _LOCAL_RANK = world_size, rank, local_rank

    if world_size > 1:
        if not dist.is_initialized():
            if backend is None:
                backend = "nccl" if torch.cuda.is_available() else "gloo"
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            kwargs = {}
            if timeout_s is not None:
                kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
            if backend == "nccl":
                torch.cuda.set_device(local_rank)
                kwargs["device_id"] = torch.device("cuda", local_rank)
            dist.init_process_group(backend=backend, rank=rank, world_size=world_size, **kwargs)
        all_groups = compute_group_ranks(world_size, sizes)
        for name, glist in all_groups.items():
            _GROUP_RANKS[name] = glist
            for ranks in glist:
                # every rank must take part in the creation of every group
                grp = dist.group.WORLD if name == "world" else dist.new_group(ranks=ranks)
                if rank in ranks:
                    _GROUPS[name] = grp
                    _MY_GROUP_RANKS[name] = ranks
                    _SIZES[name] = len(ranks)
        if verbose and rank == 0:
            for name, glist in all_groups.items():
                print(f"group {name}: {glist}")
    else:
        if model_size != 1:
            raise ValueError(f"model parallel size {model_size} requested but only one process was launched")
    _INITIALIZED = True
    return model_size


def cleanup():
    global _INITIALIZED, _WORLD_SIZE, _WORLD_RANK
    if dist.is_initialized():
        dist.destroy_process_group()
    _GROUPS.clear(); _GROUP_RANKS.clear(); _MY_GROUP_RANKS.clear(); _SIZES.clear()
    _INITIALIZED = False
    _WORLD_SIZE, _WORLD_RANK = 1, 0

"""Singleton that owns `torch.distributed` initialisation and the named process groups.

Layout rule: the children of a node partition the node's ranks as a grid; the first child takes contiguous ranks,
every following child lives in the complement of the ones before it (strided), so the first-listed leaf varies fastest."""

import os

import torch
import torch.distributed as dist


class DistributedManager:
    _shared = {}

    def __new__(cls):
        obj = super().__new__(cls)
        obj.__dict__ = cls._shared
        if not cls._shared:
            obj._rank, obj._world_size, obj._local_rank = 0, 1, 0
            obj._initialized = False
            obj._groups, obj._group_ranks, obj._group_names = {}, {}, []
            obj._distributed = False
        return obj

    # ---- basic properties
    @property
    def rank(self):
        return self._rank

    @property
    def local_rank(self):
        return self._local_rank

    @property
    def world_size(self):
        return self._world_size

    @property
    def distributed(self):
        return self._distributed

    @property
    def cuda(self):
        return torch.cuda.is_available()

    @property
    def device(self):
        return torch.device(f"cuda:{self._local_rank}") if torch.cuda.is_available() else torch.device("cpu")

    @property
    def group_names(self):
        return list(self._group_names)

    @classmethod
    def is_initialized(cls):
        return bool(cls._shared.get("_initialized", False))

    @classmethod
    def initialize(cls):
        m = cls()
        if m._initialized:
            return
        m._world_size = int(os.environ.get("WORLD_SIZE", os.environ.get("OMPI_COMM_WORLD_SIZE", os.environ.get("SLURM_NPROCS", "1"))))
        m._rank = int(os.environ.get("RANK", os.environ.get("OMPI_COMM_WORLD_RANK", os.environ.get("SLURM_PROCID", "0"))))
        m._local_rank = int(os.environ.get("LOCAL_RANK", os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", os.environ.get("SLURM_LOCALID", "0"))))
        m._distributed = m._world_size > 1
        if torch.cuda.is_available():
            torch.cuda.set_device(m._local_rank)
        if m._distributed and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            backend = "nccl" if torch.cuda.is_available() else "gloo"
            kwargs = {"device_id": m.device} if backend == "nccl" else {}
            dist.init_process_group(backend=backend, rank=m._rank, world_size=m._world_size, **kwargs)
        m._initialized = True

    # ---- named groups
    def group(self, name=None):
        if name is None:
            return None
        return self._groups.get(name, None)

    def group_size(self, name=None):
        if name is None:
            return self._world_size
        for grp in self._group_ranks.get(name, []):
            if self._rank in grp:
                return len(grp)
        return 1

    def group_rank(self, name=None):
        if name is None:
            return self._rank
        for grp in self._group_ranks.get(name, []):
            if self._rank in grp:
                return grp.index(self._rank)
        return 0

    def group_name(self, group=None):
        for n, g in self._groups.items():
            if g is group:
                return n
        return None

    def _register(self, name, rank_lists):
        self._group_names.append(name)
        self._group_ranks[name] = rank_lists
        mine = None
        for ranks in rank_lists:
            if self._distributed:
                g = dist.new_group(ranks=ranks) if len(ranks) != self._world_size else dist.group.WORLD
            else:
                g = None
            if self._rank in ranks:
                mine = g
        self._groups[name] = mine

    @staticmethod
    def create_groups_from_config(config, verbose=False):
        m = DistributedManager()

        def recurse(name, rank_lists):
            # rank_lists: the groups of node `name`; split each into the grid of the node's children
            kids = config.children[name]
            if not kids:
                return
            sizes = [config.nodes[k].size for k in kids]
            stride = 1
            for kid, size in zip(kids, sizes):
                kid_lists = []
                for grp in rank_lists:
                    n = len(grp)
                    block = stride * size
                    for base in range(0, n, block):
                        for off in range(stride):
                            kid_lists.append([grp[base + off + j * stride] for j in range(size)])
                m._register(kid, kid_lists)
                if verbose:
                    print(f"process group {kid}: {kid_lists}")
                recurse(kid, kid_lists)
                stride *= size

        root = config.root_id
        world = [list(range(m._world_size))]
        assert config.nodes[root].size in (None, m._world_size)
        recurse(root, world)

    @staticmethod
    def cleanup():
        if dist.is_initialized():
            dist.destroy_process_group()

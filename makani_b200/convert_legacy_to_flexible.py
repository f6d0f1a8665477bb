"""Convert per-rank legacy checkpoints of a model-parallel run into one flexible checkpoint (+ model package).

    python -m makani_b200.convert_legacy_to_flexible --yaml_config <file> --config <section> \
        --h_parallel_size H --w_parallel_size W --fin_parallel_size FI --fout_parallel_size FO \
        --input_path <dir with ckpt_mp{r}.tar> --output_path <dir>

The conversion needs no process group: every rank's `model_state` is read on the CPU and the shards of each
parameter are concatenated along the dimensions named in its `sharded_dims_mp`, using this framework's rank
order (h slowest, then w, fin, fout).  The reference spawns one NCCL process per model rank for the same job
(makani/convert_legacy_to_flexible.py:41-133).
"""

from __future__ import annotations

import argparse
import itertools
import os

import torch

from .utils.checkpoint import load_file

_ORDER = ["h", "w", "fin", "fout"]


def _rank_of(coord, sizes):
    r = 0
    for n in _ORDER:
        r = r * sizes[n] + coord[n]
    return r


def merge_states(states, sizes, sharded_dims):
    """states: list of per-rank state dicts (index = model rank); sharded_dims: name -> list of group names / None."""
    out = {}
    for name in states[0].keys():
        dims = sharded_dims.get(name)
        if not dims or all(d is None for d in dims):
            out[name] = states[0][name].clone()
            continue

        def gather(coord, dim_idx):
            # recursively concatenate along each sharded dimension
            while dim_idx < len(dims) and (dims[dim_idx] is None):
                dim_idx += 1
            if dim_idx >= len(dims):
                return states[_rank_of(coord, sizes)][name]
            g = dims[dim_idx]
            groups = {"matmul": ["fin", "fout"], "spatial": ["h", "w"]}.get(g, [g])
            parts = []
            for idx in itertools.product(*[range(sizes[a]) for a in groups]):
                c = dict(coord)
                c.update(dict(zip(groups, idx)))
                parts.append(gather(c, dim_idx + 1))
            return torch.cat(parts, dim=dim_idx)

        out[name] = gather({n: 0 for n in _ORDER}, 0)
    return out


def get_params(path):
    """The recipe a run wrote into its experiment directory (`<path>/config.json`), as a params object."""
    from .utils.YParams import ParamsBase

    return ParamsBase.from_json(os.path.join(path, "config.json"))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_path", required=True, type=str)
    ap.add_argument("--output_path", required=True, type=str)
    for n in _ORDER:
        ap.add_argument(f"--{n}_parallel_size", default=1, type=int)
    ap.add_argument("--yaml_config", default=None, type=str)
    ap.add_argument("--config", default=None, type=str)
    ap.add_argument("--prefix", default="ckpt", type=str, help="ckpt or best_ckpt")
    args = ap.parse_args(argv)
    sizes = {n: getattr(args, f"{n}_parallel_size") for n in _ORDER}
    nranks = 1
    for v in sizes.values():
        nranks *= v
    ckpts = [load_file(os.path.join(args.input_path, f"{args.prefix}_mp{r}.tar")) for r in range(nranks)]
    states = []
    for c in ckpts:
        st = c["model_state"]
        torch.nn.modules.utils.consume_prefix_in_state_dict_if_present(st, "module.")
        states.append(st)
    # sharding annotations come from a model instance built for rank 0 of a serial layout
    params = ckpts[0]["params"]
    from .models import model_registry
    model = model_registry.get_model(params)
    sharded = {k: list(getattr(v, "sharded_dims_mp", [])) for k, v in model.named_parameters()}
    full = merge_states(states, sizes, sharded)
    os.makedirs(args.output_path, exist_ok=True)
    store = {"iters": ckpts[0].get("iters", 0), "epoch": ckpts[0].get("epoch", 0), "model_state": full, "params": params}
    torch.save(store, os.path.join(args.output_path, f"{args.prefix}_mp0.tar"))
    try:
        from .models.model_package import save_model_package
        params.experiment_dir = args.output_path
        save_model_package(params)
    except Exception as e:
        print(f"model package not written: {e}")
    print(f"wrote {os.path.join(args.output_path, args.prefix + '_mp0.tar')}")


if __name__ == "__main__":
    main()

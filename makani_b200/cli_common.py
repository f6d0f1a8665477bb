"""Shared bootstrap of the command line entry points: flag parsing, recipe loading, topology, experiment directory.

Flag set and derived parameters follow makani/train.py:33-183, makani/inference.py:34-165 and
makani/train_profile.py (capture flags).
"""

from __future__ import annotations

import argparse
import logging
import os

import torch

from .utils import comm, logging_utils
from .utils.parse_dataset_metadata import parse_dataset_metadata
from .utils.YParams import YParams


def base_parser(description: str) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=description)
    p.add_argument("--fin_parallel_size", default=1, type=int, help="Input feature parallelization")
    p.add_argument("--fout_parallel_size", default=1, type=int, help="Output feature parallelization")
    p.add_argument("--h_parallel_size", default=1, type=int, help="Spatial parallelism dimension in h")
    p.add_argument("--w_parallel_size", default=1, type=int, help="Spatial parallelism dimension in w")
    p.add_argument("--parameters_reduction_buffer_count", default=1, type=int,
                   help="Number of buckets the gradient reduction is split into")
    p.add_argument("--run_num", default="00", type=str)
    p.add_argument("--exp_dir", default=None, type=str, help="Override of the recipe's experiment root directory")
    p.add_argument("--yaml_config", default="./config/sfnonet.yaml", type=str)
    p.add_argument("--config", default="base_73chq", type=str)
    p.add_argument("--batch_size", default=-1, type=int, help="Override of the global batch size of the recipe")
    p.add_argument("--enable_synthetic_data", action="store_true")
    p.add_argument("--amp_mode", default="none", type=str, choices=["none", "fp16", "bf16"])
    p.add_argument("--jit_mode", default="none", type=str, choices=["none", "script", "inductor"],
                   help="accepted for recipe compatibility; the hot path is hand-written kernels, nothing is traced")
    p.add_argument("--cuda_graph_mode", default="none", type=str, choices=["none", "fwdbwd", "step"])
    p.add_argument("--enable_odirect", action="store_true")
    p.add_argument("--checkpointing_level", default=0, type=int, help="How aggressively activation checkpointing is used")
    p.add_argument("--epsilon_factor", default=0, type=float)
    p.add_argument("--split_data_channels", action="store_true")
    p.add_argument("--print_timings_frequency", default=-1, type=int)
    p.add_argument("--skip_validation", action="store_true")
    p.add_argument("--save_checkpoint", default="legacy", choices=["none", "flexible", "legacy"], type=str)
    p.add_argument("--load_checkpoint", default="legacy", choices=["flexible", "legacy"], type=str)
    p.add_argument("--multistep_count", default=1, type=int, help="Number of autoregressive training steps (1 = conventional)")
    p.add_argument("--enable_benchy", action="store_true")
    p.add_argument("--disable_ddp", action="store_true")
    p.add_argument("--enable_grad_anomaly_detection", action="store_true")
    return p


def bootstrap(args, inference: bool = False):
    """Load the recipe, initialise the process topology and fill in every CLI-derived parameter."""
    params = YParams(os.path.abspath(args.yaml_config), args.config)
    params["epsilon_factor"] = args.epsilon_factor
    if getattr(args, "exp_dir", None):
        params["exp_dir"] = args.exp_dir
    for n in ("fin", "fout", "h", "w"):
        params[f"{n}_parallel_size"] = getattr(args, f"{n}_parallel_size")
    params["model_parallel_sizes"] = [args.h_parallel_size, args.w_parallel_size, args.fin_parallel_size, args.fout_parallel_size]
    params["model_parallel_names"] = ["h", "w", "fin", "fout"]
    params["parameters_reduction_buffer_count"] = args.parameters_reduction_buffer_count
    params["load_checkpoint"] = getattr(args, "checkpoint_format", None) or args.load_checkpoint
    params["save_checkpoint"] = args.save_checkpoint

    comm.init(model_parallel_sizes=params["model_parallel_sizes"], model_parallel_names=params["model_parallel_names"], verbose=False)
    world_rank = comm.get_world_rank()
    params["world_size"] = comm.get_world_size()
    if args.batch_size > 0:
        params.batch_size = args.batch_size
    params["global_batch_size"] = params.batch_size
    assert params["global_batch_size"] % comm.get_size("data") == 0, \
        f"Error, cannot evenly distribute {params['global_batch_size']} across {comm.get_size('data')} GPU."
    params["batch_size"] = int(params["global_batch_size"] // comm.get_size("data"))
    if "optimizer_max_grad_norm" not in params:
        params["optimizer_max_grad_norm"] = 1.0

    if torch.cuda.is_available():
        torch.cuda.set_device(comm.get_local_rank())
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
    if args.enable_grad_anomaly_detection:
        torch.autograd.set_detect_anomaly(True)

    exp_dir = os.path.join(params.exp_dir, args.config, str(args.run_num))
    if world_rank == 0:
        os.makedirs(os.path.join(exp_dir, "training_checkpoints"), exist_ok=True)
        os.makedirs(os.path.join(exp_dir, "wandb"), exist_ok=True)
    params["experiment_dir"] = os.path.abspath(exp_dir)
    ckpt_root = getattr(args, "checkpoint_path", None)
    if ckpt_root:
        params["checkpoint_path"] = os.path.join(ckpt_root, "ckpt_mp{mp_rank}.tar") if os.path.isdir(ckpt_root) else ckpt_root
        params["best_checkpoint_path"] = params["checkpoint_path"]
    else:
        params["checkpoint_path"] = os.path.join(exp_dir, "training_checkpoints/ckpt_mp{mp_rank}.tar")
        params["best_checkpoint_path"] = os.path.join(exp_dir, "training_checkpoints/best_ckpt_mp{mp_rank}.tar")

    resuming = True
    for mp_rank in range(comm.get_size("model")):
        if params["load_checkpoint"] == "legacy" or mp_rank < 1:
            resuming = resuming and os.path.isfile(params.checkpoint_path.format(mp_rank=mp_rank))
    params["resuming"] = resuming
    params["amp_mode"] = args.amp_mode
    params["jit_mode"] = args.jit_mode
    params["cuda_graph_mode"] = args.cuda_graph_mode
    params["skip_validation"] = args.skip_validation
    params["enable_odirect"] = args.enable_odirect
    params["checkpointing"] = args.checkpointing_level
    params["enable_synthetic_data"] = args.enable_synthetic_data
    params["split_data_channels"] = args.split_data_channels
    params["print_timings_frequency"] = args.print_timings_frequency
    params["multistep_count"] = args.multistep_count
    params["n_future"] = 0 if inference else args.multistep_count - 1
    params["enable_benchy"] = args.enable_benchy
    params["disable_ddp"] = args.disable_ddp
    params["enable_grad_anomaly_detection"] = args.enable_grad_anomaly_detection
    if params.get("wandb_dir") is None:
        params["wandb_dir"] = exp_dir

    if world_rank == 0:
        logging_utils.config_logger()
        logging_utils.log_to_file(logger_name=None, log_filename=os.path.join(exp_dir, "out.log"))
        logging_utils.log_versions()
        params.log(logging.getLogger())
    params["log_to_wandb"] = (world_rank == 0) and bool(params.get("log_to_wandb", False))
    params["log_to_screen"] = (world_rank == 0) and bool(params.get("log_to_screen", False))

    if params.get("metadata_json_path") is not None and os.path.exists(params["metadata_json_path"]):
        params, _ = parse_dataset_metadata(params["metadata_json_path"], params=params)
    elif not args.enable_synthetic_data:
        raise RuntimeError("Error, please specify a dataset descriptor file in json format (metadata_json_path) "
                           "or run with --enable_synthetic_data")
    else:
        # synthetic runs need no dataset: derive the channel lists from the recipe
        names = params.get("channel_names")
        n = len(names) if names is not None else params.get("N_out_channels", 2)
        params["in_channels"] = list(range(n))
        params["out_channels"] = list(range(n))
        if params.get("dhours") is None:
            params["dhours"] = 6
    return params, world_rank

"""Inference / scoring entry point: `python -m makani_b200.inference --yaml_config <file> --config <section>`.

Requires the checkpoints of the run (or `--checkpoint_path`).  `--mode score` rolls the model out over the
evaluation set and writes acc/rmse curves; `--mode ensemble` (declared but not implemented by the reference CLI,
makani/inference.py:55,161-165) runs an initial-condition ensemble from one sample and writes the RMSE of the ensemble
mean, the spread and their ratio per channel and lead time.
"""

from __future__ import annotations

import os

from .cli_common import base_parser, bootstrap
from .utils import comm


def main(argv=None):
    parser = base_parser("makani_b200 inference")
    parser.add_argument("--checkpoint_path", default=None, type=str)
    parser.add_argument("--enable_nhwc", action="store_true")
    parser.add_argument("--mode", default="score", type=str, choices=["score", "ensemble"])
    parser.add_argument("--checkpoint_format", default="legacy", choices=["flexible", "legacy"], type=str)
    parser.add_argument("--ensemble_size", default=8, type=int)
    parser.add_argument("--ensemble_noise_std", default=0.05, type=float, help="std of the initial-condition noise (normalised units)")
    parser.add_argument("--ensemble_ic", default=0, type=int, help="index of the evaluation sample used as initial condition")
    args = parser.parse_args(argv)
    params, world_rank = bootstrap(args, inference=True)
    if not args.enable_synthetic_data:
        for mp_rank in range(comm.get_size("model")):
            if params["load_checkpoint"] == "legacy" or mp_rank < 1:
                fname = params.checkpoint_path.format(mp_rank=mp_rank)
                assert os.path.isfile(fname), f"Error, checkpoint file {fname} not found"
    params["enable_nhwc"] = args.enable_nhwc
    params["n_future"] = 0
    from .utils.inferencer import Inferencer
    if args.mode == "score":
        inferencer = Inferencer(params, world_rank)
        inferencer.score_model()
        return inferencer
    inferencer = Inferencer(params, world_rank)
    inferencer.ensemble_result = inferencer.inference_ensemble(ic=args.ensemble_ic, n_members=args.ensemble_size,
                                                               noise_std=args.ensemble_noise_std)
    return inferencer


if __name__ == "__main__":
    main()

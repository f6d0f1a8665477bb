"""Training entry point: `python -m makani_b200.train --yaml_config <file> --config <section> [flags]`.

Launch one process per GPU with torchrun / mpirun / srun.  `--mode test` runs the autoregression self test with
the identity-like DebugNet.  Flag set: makani/train.py:33-183.
"""

from __future__ import annotations

from .cli_common import base_parser, bootstrap


def main(argv=None):
    parser = base_parser("makani_b200 training")
    parser.add_argument("--mode", default="train", type=str, choices=["train", "test"])
    args = parser.parse_args(argv)
    params, world_rank = bootstrap(args)
    from .utils.trainer import Trainer
    if args.mode == "train":
        trainer = Trainer(params, world_rank)
        trainer.train()
    else:
        params["nettype"] = "DebugNet"
        trainer = Trainer(params, world_rank)
        ok = trainer.test_autoregression_pipeline()
        if not ok:
            raise SystemExit(1)
    return trainer


if __name__ == "__main__":
    main()

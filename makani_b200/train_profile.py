"""Training entry point with a profiler capture window (see `makani_b200.utils.trainer_profile`).

    nsys profile --capture-range=cudaProfilerApi ... python -m makani_b200.train_profile --capture_mode training \
        --capture_range_start 10 --capture_range_stop 20 [training flags]
"""

from __future__ import annotations

from .cli_common import base_parser, bootstrap


def main(argv=None):
    parser = base_parser("makani_b200 profiling run")
    parser.add_argument("--capture_mode", default=[], nargs="+", type=str, choices=["training", "validation"],
                        help="which phases the capture window applies to")
    parser.add_argument("--capture_range_start", default=0, type=int, help="first captured step")
    parser.add_argument("--capture_range_stop", default=50, type=int, help="last captured step")
    parser.add_argument("--capture_ranks", default=[], nargs="+", type=int, help="ranks that toggle the profiler (default all)")
    parser.add_argument("--enable_anna", action="store_true", help="accepted for compatibility; layer hooks are not used")
    args = parser.parse_args(argv)
    params, world_rank = bootstrap(args)
    params["capture_mode"] = args.capture_mode
    params["capture_range_start"] = args.capture_range_start
    params["capture_range_stop"] = args.capture_range_stop
    params["capture_ranks"] = args.capture_ranks
    from .utils.trainer_profile import ProfilingTrainer
    trainer = ProfilingTrainer(params, world_rank)
    trainer.train()
    return trainer


if __name__ == "__main__":
    main()

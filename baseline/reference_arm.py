"""Reference arm of the benchmark: times the UNMODIFIED upstream `makani` package (installed under `baseline/_ref`).

What runs is upstream code only: `makani.utils.comm.init` (process groups), `makani.utils.YParams.YParams` (recipe),
`Trainer._update_parameters`, `makani.models.model_registry.get_model` (SFNO inside `SingleStepWrapper` /
`MultiStepWrapper` with `Preprocessor2D`), `makani.mpu.helpers.sync_params`, `makani.utils.losses.LossHandler`,
`torch.optim.AdamW(foreach=True)`, `makani.mpu.mappings.init_gradient_reduction_hooks` (DDP + reduction hook),
`Trainer._compile_model`, `Trainer._capture_model` (CUDA graph of forward + backward, `--cuda_graph_mode fwdbwd`) and
`Trainer.train_one_epoch` (the step loop: copy into the static buffers, graph replay, optimiser step).  The object is
assembled in the order of `Trainer.__init__` (makani/utils/trainer.py:280-589) minus the parts that need files on disk
(data loaders, model package, metrics climatology, visualiser): the data loader is a list of synthetic batches, as the
benchmark prescribes (the upstream synthetic loader itself cannot run, makani/utils/dataloaders/data_loader_dummy.py:73,
123-130).  Third-party packages this image lacks are replaced by the stock-torch stand-ins in `baseline/shims`.
Nothing of `makani_b200` is imported here.
"""

from __future__ import annotations

import contextlib
import json
import logging
import os
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SHIMS = os.path.join(HERE, "shims")
REF = os.path.join(HERE, "_ref")

SHIMMED = ["ruamel.yaml", "modulus", "torch_harmonics", "tensorly", "tltorch", "h5py", "jsbeautifier", "pytz", "moviepy"]


def _unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    sys.stdout.flush()
    return 0


class _SyntheticDataset:
    """The attributes `Trainer._update_parameters` reads from a dataset (makani/utils/trainer.py:184-201)."""

    def __init__(self, n_in, n_out, nlat, nlon, lat_shapes, lon_shapes, rh, rw):
        self.in_channels = list(range(n_in))
        self.out_channels = list(range(n_out))
        self.img_shape_x, self.img_shape_y = nlat, nlon
        self.img_crop_shape_x, self.img_crop_shape_y = nlat, nlon
        self.img_crop_offset_x, self.img_crop_offset_y = 0, 0
        self.img_local_shape_x, self.img_local_shape_y = lat_shapes[rh], lon_shapes[rw]
        self.img_local_offset_x, self.img_local_offset_y = sum(lat_shapes[:rh]), sum(lon_shapes[:rw])


def _bail_later(seconds=30.0):
    def _bail():
        time.sleep(seconds)
        os._exit(0)

    threading.Thread(target=_bail, daemon=True).start()


def run(args, clock_sampler_cls=None) -> int:
    if not os.path.isdir(os.path.join(REF, "makani")):
        return _unavailable("reference not installed under baseline/_ref")
    for p in (SHIMS, REF):
        if p not in sys.path:
            sys.path.insert(0, p)
    if any(m == "makani_b200" or m.startswith("makani_b200.") for m in sys.modules):
        return _unavailable("makani_b200 is loaded in this process; the reference arm must run without it")

    import torch
    import torch.distributed as dist
    from torch.cuda import amp

    cuda = torch.cuda.is_available()
    try:
        from makani.utils import comm
        from makani.utils.YParams import YParams
        from makani.utils.trainer import Trainer
        from makani.models import model_registry
        from makani.utils.losses import LossHandler
        from makani.mpu.mappings import init_gradient_reduction_hooks
        from makani.mpu.helpers import sync_params
        from makani.models.helpers import count_parameters
    except Exception as e:  # a stock line failed: name it
        import traceback
        tb = traceback.extract_tb(e.__traceback__)[-1]
        return _unavailable(f"reference import fails at {tb.filename.replace(ROOT + os.sep, '')}:{tb.lineno}: {type(e).__name__}: {e}")

    # -------------------------------------------------------------------------------- what makani/train.py does
    sizes = [args.h, args.w, args.fin, args.fout]
    comm.init(model_parallel_sizes=sizes, model_parallel_names=["h", "w", "fin", "fout"], verbose=False)
    world, rank, local_rank = comm.get_world_size(), comm.get_world_rank(), comm.get_local_rank()
    device = torch.device(f"cuda:{local_rank}") if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local_rank)
        torch.backends.cudnn.benchmark = True                    # makani/train.py:108-110
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True

    recipe = "sfno_tiny" if args.tiny else "sfno_linear_73chq_sc3_layers8_edim384_bench"
    params = YParams(os.path.join(ROOT, "config", "sfnonet.yaml"), recipe)
    nlat, nlon = params.img_shape_x, params.img_shape_y
    if args.small:
        nlat, nlon = 361, 720
    n_out = len(params.channel_names)
    n_in = n_out + (0 if args.tiny else 1)            # + the static cos(latitude) channel, delivered with the data
    dp = comm.get_size("data")
    batch = 1
    params["model_parallel_sizes"], params["model_parallel_names"] = sizes, ["h", "w", "fin", "fout"]
    params["parameters_reduction_buffer_count"] = 1   # makani/train.py:51 default
    params["world_size"] = world
    params["global_batch_size"] = batch * dp
    params["batch_size"] = batch
    params["optimizer_max_grad_norm"] = params.get("optimizer_max_grad_norm", 1.0)
    params["experiment_dir"] = "/tmp/makani_reference_arm"
    params["resuming"] = False
    params["amp_mode"] = "bf16" if cuda else "none"
    params["jit_mode"] = "none"
    params["cuda_graph_mode"] = args.ref_graph if cuda else "none"
    params["skip_validation"] = True
    params["enable_odirect"] = False
    params["checkpointing"] = 0
    params["enable_synthetic_data"] = True
    params["split_data_channels"] = False
    params["print_timings_frequency"] = 0
    params["multistep_count"] = args.multistep
    params["n_future"] = args.multistep - 1
    params["enable_benchy"] = False
    params["disable_ddp"] = False
    params["enable_grad_anomaly_detection"] = False
    params["log_to_wandb"] = False
    params["log_to_screen"] = (rank == 0)
    params["log_weights_and_grads"] = 0
    params["add_grid"] = params["add_zenith"] = params["add_orography"] = params["add_landmask"] = False
    params["img_shape_x"], params["img_shape_y"] = nlat, nlon

    # -------------------------------------------------------------------------------- Trainer.__init__, in its order
    from modulus.distributed.utils import compute_split_shapes  # the stand-in; same rule as the data loaders use

    tr = Trainer.__new__(Trainer)
    tr.params = None
    tr.world_rank = rank
    tr.data_parallel_rank = comm.get_rank("data")
    tr.device = device
    tr.logger = logging.getLogger()
    if dist.is_initialized():
        tens = torch.ones(1, device=device)
        dist.all_reduce(tens, group=comm.get_group("data"))
    tr.amp_enabled = params.amp_mode != "none"
    tr.amp_dtype = torch.bfloat16 if tr.amp_enabled else torch.float32
    lat_shapes = compute_split_shapes(nlat, comm.get_size("h"))
    lon_shapes = compute_split_shapes(nlon, comm.get_size("w"))
    tr.valid_dataset = _SyntheticDataset(n_in, n_out, nlat, nlon, lat_shapes, lon_shapes, comm.get_rank("h"), comm.get_rank("w"))
    params = tr._update_parameters(params)
    tr.params = params
    hl, wl = params.img_local_shape_x, params.img_local_shape_y

    torch.manual_seed(333 + comm.get_rank("model"))
    tr.model = model_registry.get_model(params).to(device)
    tr.preprocessor = tr.model.preprocessor
    sync_params(tr.model, mode="broadcast")
    tr.loss_obj = LossHandler(params).to(device)
    tr.capturable_optimizer = False
    betas = (params.optimizer_beta1, params.optimizer_beta2)
    tr.optimizer = torch.optim.AdamW(tr.model.parameters(), betas=betas, lr=params.lr, weight_decay=params.weight_decay, foreach=True)
    tr.scheduler = None
    tr.gscaler = amp.GradScaler(enabled=(tr.amp_dtype == torch.float16))

    capture_stream = None
    if dist.is_initialized() and not params.disable_ddp:
        if cuda:
            capture_stream = torch.cuda.Stream()
        parameter_size_mb = count_parameters(tr.model, device) * 4 / float(1024 * 1024)
        reduction_size_mb = max(1, int((parameter_size_mb / params.parameters_reduction_buffer_count) * 1.05))  # max: toy models only
        ctx = torch.cuda.stream(capture_stream) if cuda else contextlib.nullcontext()
        with ctx:
            tr.model = init_gradient_reduction_hooks(
                tr.model, device_ids=[device.index] if cuda else None, output_device=[device.index] if cuda else None,
                bucket_cap_mb=reduction_size_mb, broadcast_buffers=True, find_unused_parameters=False,
                gradient_as_bucket_view=True, static_graph=False)
        if capture_stream is not None:
            capture_stream.synchronize()

    tr._set_train()
    t_out = params.n_future + 1
    inp_shape = (batch, n_in, hl, wl)
    tar_shape = (batch, t_out * n_out, hl, wl)
    tr._compile_model(inp_shape)
    if not tr.loss_obj.is_distributed():
        try:
            tr.loss_obj = torch.jit.script(tr.loss_obj)       # makani/utils/trainer.py:527-528
        except Exception:
            pass
    tr.graph = None
    graph_mode = params.cuda_graph_mode
    if graph_mode != "none" and cuda:
        try:
            tr._capture_model(capture_stream, inp_shape, tar_shape, num_warmup_steps=20)
        except Exception as e:
            # keep the eager stock path if the capture is refused by the runtime
            tr.graph = None
            graph_mode = f"none (capture failed: {type(e).__name__})"
            torch.cuda.synchronize()
    tr.iters = 0
    tr.epoch = 0

    # -------------------------------------------------------------------------------- synthetic batches
    def make(seed, where):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(batch, 1, n_in, hl, wl, generator=g)
        y = torch.randn(batch, t_out, n_out, hl, wl, generator=g)
        if where == "pinned":
            return x.pin_memory(), y.pin_memory()
        return x.to(device), y.to(device)

    def barrier():
        if dist.is_initialized():
            dist.barrier(device_ids=[local_rank] if cuda else None)
        if cuda:
            torch.cuda.synchronize()

    def epoch(loader):
        # upstream prints progress and timings to stdout; the benchmark's stdout carries one JSON line only
        with contextlib.redirect_stdout(sys.stderr):
            return tr.train_one_epoch()

    def timed(loader_factory, steps, warmup):
        tr.train_dataloader = loader_factory(warmup)
        if warmup:
            epoch(tr.train_dataloader)
        tr.train_dataloader = loader_factory(steps)
        barrier()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        _, _, logs = epoch(tr.train_dataloader)
        if cuda:
            e1.record()
        barrier()
        ms = e0.elapsed_time(e1) if cuda else (time.perf_counter() - t0) * 1e3
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() / steps, logs

    # device-timed: the batches are resident on the device (the loop's `.to(device)` is then a no-op)
    resident = make(1234 + rank, "device")
    sampler = clock_sampler_cls(local_rank, None) if (clock_sampler_cls is not None and cuda) else None
    # untimed priming epoch so that allocator pools and cuDNN / cuFFT plans exist before the warm-up
    tr.train_dataloader = [resident] * 2
    epoch(tr.train_dataloader)
    if sampler is not None:
        sampler.start()
    ms_per_step, logs = timed(lambda n: [resident] * n, args.steps, args.warmup)
    clocks = sampler.stop() if sampler is not None else None
    value = batch * dp / (ms_per_step / 1e3)

    # end to end: every step's batch comes from pinned host memory through the loop's own `.to(device)`, and the loss
    # is read back every step by the loop's own timing print (`print_timings_frequency 1` -> `loss.item()`)
    e2e = None
    if not args.no_e2e:
        host = [make(100 + i + 17 * local_rank, "pinned" if cuda else "device") for i in range(2)]
        params.print_timings_frequency = 1
        ms_e2e, _ = timed(lambda n: [host[i % 2] for i in range(n)], args.steps, max(1, min(args.warmup, 2)))
        params.print_timings_frequency = 0
        h2d = sum(t.numel() * t.element_size() for t in host[0])
        e2e = {"value": batch * dp / (ms_e2e / 1e3), "unit": "samples/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4}

    if rank == 0:
        mp = args.h * args.w * args.fin * args.fout
        out = {
            "metric": "SFNO-73ch 721x1440 bf16 train samples/s", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 autocast (fp32 parameters and transforms, as upstream)",
            "data": "synthetic N(0,1), random-init weights", "impl": "reference",
            "config": {"model": recipe.replace("_bench", "") + ("_small" if args.small else ""), "global_batch": batch * dp,
                       "seq_len": f"{nlat}x{nlon}",
                       "parallelism": f"dp{dp}" + (f"xh{args.h}w{args.w}" if args.h * args.w > 1 else "")
                       + (f"xfin{args.fin}fout{args.fout}" if args.fin * args.fout > 1 else ""),
                       "l2_policy": "inputs+activations per step (>2 GB) exceed the 126 MB L2",
                       "loss": params.loss, "optimizer": "torch.optim.AdamW(foreach)", "cuda_graph": graph_mode,
                       "multistep_count": args.multistep, "final_loss": float(logs["loss"].detach() if hasattr(logs["loss"], "detach") else logs["loss"]),
                       "entry": "makani.utils.trainer.Trainer.train_one_epoch (unmodified upstream package)"},
            "clocks": clocks, "gpu_launches": 0, "shimmed_packages": SHIMMED,
        }
        if e2e is not None:
            out["e2e"] = e2e
        print(json.dumps(out))
    sys.stdout.flush()
    if dist.is_initialized():
        _bail_later()
        tr.graph = None
        import gc
        gc.collect()
        if cuda:
            torch.cuda.synchronize()
        dist.barrier(device_ids=[local_rank] if cuda else None)
        dist.destroy_process_group()
    return 0

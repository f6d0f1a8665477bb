"""Headline benchmark: SFNO-73ch 721x1440 bf16 training throughput (samples/s), weak scaling, pure data parallel.

    python bench.py --gpus N --steps K --warmup W [--impl native|reference|restated]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Model ("sfno_linear_73chq_sc3_layers8_edim384", reference recipe config/sfnonet.yaml:149-159): 721x1440
equiangular grid, 73 prognostic channels + 1 static cos(latitude) channel in, 73 out, embed_dim 384, 8 blocks,
scale_factor 3, dhconv spectral weights, MLP ratio 2, GELU, instance norm; random-init weights, synthetic
N(0,1) data, batch 1 per GPU; loss "absolute squared geometric l2"; AdamW.  One step = forward + backward +
gradient reduction + optimiser step, replayed from one CUDA graph after an eager warm-up (`--no-graph`: eager).
Prints one JSON line on rank 0: the device-timed value (CUDA events, max over ranks), the end-to-end value (every
step's batch copied from pinned host memory, every step's loss read back), clocks sampled during the timed region and
the number of this package's kernels launched in it.

Other configurations of the same harness: `--h/--w` (one sample split over latitude / longitude ranks with the fused
distributed transforms), `--fin/--fout` (channel parallelism), `--model afno`, `--mode rollout` (autoregressive
inference, ms per step), `--impl restated` (the reference's op sequence on stock PyTorch kernels and NCCL),
`--impl reference` (the unmodified upstream package, if importable).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BASELINE_VALUE = None  # the reference publishes no throughput number


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="native", choices=["native", "reference", "restated"],
                    help="native: this framework; reference: the unmodified upstream package from baseline/_ref; restated: the "
                         "reference's op sequence on stock PyTorch kernels and NCCL, through this package's model code")
    ap.add_argument("--small", action="store_true", help="reduced grid for profiling captures (not a bench value)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--mode", default="train", choices=["train", "rollout"],
                    help="train: samples/s of the optimisation step (headline); rollout: ms per autoregressive inference step")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--model", default="sfno", choices=["sfno", "afno"], help="sfno: the headline model; afno: FourCastNet v1 (720x1440x20)")
    ap.add_argument("--fin", type=int, default=1, help="input-feature parallel ranks (channel parallelism)")
    ap.add_argument("--fout", type=int, default=1, help="output-feature parallel ranks")
    ap.add_argument("--h", type=int, default=1, help="latitude-parallel ranks per model instance (default: pure data parallel)")
    ap.add_argument("--w", type=int, default=1, help="longitude-parallel ranks per model instance")
    ap.add_argument("--multistep", type=int, default=1, help="multistep_count: autoregressive steps per training sample (loss over all of them)")
    ap.add_argument("--ref-graph", default="fwdbwd", choices=["none", "fwdbwd"], help="reference arm: its --cuda_graph_mode")
    ap.add_argument("--tiny", action="store_true", help="32x64 plumbing configuration (CPU friendly; not a bench value)")
    ap.add_argument("--via", default="harness", choices=["harness", "trainer"],
                    help="harness: network + loss + optimiser assembled by utils/bench_harness.py; trainer: the step of the "
                         "product's entry point (cli_common.bootstrap -> Trainer with the recipe of config/sfnonet.yaml, synthetic "
                         "data, --amp_mode bf16 --cuda_graph_mode step), i.e. what `python -m makani_b200.train` runs")
    return ap.parse_args()


def reference_arm(args):
    """Times the unmodified upstream package from baseline/_ref (see baseline/reference_arm.py)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm as arm
    except Exception as e:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"baseline/reference_arm.py not importable: {type(e).__name__}: {e}"}))
        return 0
    return arm.run(args, clock_sampler_cls=ClockSampler)


class ClockSampler:
    """Samples SM clocks / throttle reasons of this rank's GPU while the timed region runs.

    Primary: an NVML polling thread (read-only queries, 50 ms period, exactly between `start` and `stop`);
    fallback: an `nvidia-smi --query-gpu ... -lms 200` child process."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, uuid: str = None):
        self.gpu_index, self.uuid = gpu_index, uuid
        self.proc = None
        self.thread = None
        self.samples = []
        self.path = os.path.join("/tmp", f"bench_clocks_{os.getpid()}.csv")

    # ---- NVML
    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        if self.uuid:
            try:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(self.uuid if self.uuid.startswith("GPU-") else "GPU-" + self.uuid)
            except Exception:
                pass
        vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        idx = self.gpu_index
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.gpu_index < len(ids) and ids[self.gpu_index].isdigit():
                idx = int(ids[self.gpu_index])
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(idx)

    def _poll(self):
        nv, h = self._nv, self._h
        bits = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.samples.append((float(sm), [n for n, b in bits.items() if mask & b]))
            except Exception:
                pass
            self._stop.wait(0.05)

    def start(self):
        import threading
        try:
            self._nv, self._h = self._nvml_handle()
            self._max = float(self._nv.nvmlDeviceGetMaxClockInfo(self._h, self._nv.NVML_CLOCK_SM))
            self._stop = threading.Event()
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2.0)
            if self.samples:
                sm = sorted(s[0] for s in self.samples)
                out["sm_mhz"] = sm[len(sm) // 2]
                out["sm_max_mhz"] = self._max
                out["reasons"] = sorted({r for s in self.samples for r in s[1]})
                out["samples"] = len(sm)
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for n, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out["sm_mhz"] = sm[len(sm) // 2]
            out["sm_max_mhz"] = max(mx)
        out["reasons"] = sorted(reasons)
        return out


def _gpu_uuid(torch, index):
    try:
        return str(torch.cuda.get_device_properties(index).uuid)
    except Exception:
        return None


def via_trainer(args):
    """The headline step through the training entry point: the same flags a user passes to `python -m makani_b200.train`
    go through `cli_common.bootstrap`, the `Trainer` builds model (registry + stepper + preprocessor), loss, reducer and
    optimiser from the recipe, and its own `_prepare_batch` / `_train_step` are timed on synthetic batches."""
    import tempfile

    import torch
    import torch.distributed as dist

    from makani_b200 import cli_common
    from makani_b200.ops import _ext
    from makani_b200.utils import comm
    from makani_b200.utils.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = torch.cuda.is_available()      # without a GPU only the plumbing runs (--tiny): not a bench value
    if on_gpu:
        torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank) if on_gpu else torch.device("cpu")
    mp = args.h * args.w * args.fin * args.fout
    dp = max(1, world // mp)
    recipe = "sfno_tiny" if args.tiny else "sfno_linear_73chq_sc3_layers8_edim384_bench"
    argv = ["--yaml_config", os.path.join(ROOT, "config", "sfnonet.yaml"), "--config", recipe, "--enable_synthetic_data",
            "--amp_mode", "bf16", "--cuda_graph_mode", "none" if args.no_graph else "step", "--batch_size", str(dp),
            "--skip_validation", "--save_checkpoint", "none", "--multistep_count", str(args.multistep),
            "--h_parallel_size", str(args.h), "--w_parallel_size", str(args.w), "--fin_parallel_size", str(args.fin),
            "--fout_parallel_size", str(args.fout), "--exp_dir", tempfile.mkdtemp(prefix="makani_b200_bench_")]
    cargs = cli_common.base_parser("bench").parse_args(argv)
    params, world_rank = cli_common.bootstrap(cargs)
    params["log_to_screen"] = False
    # the 74th input channel of the headline model is the cosine of the solar zenith angle: the loader delivers it per
    # time step and the preprocessor appends it to every (autoregressive) input, as in the reference's recipe
    params["add_zenith"] = True
    params["n_train_samples_per_epoch"] = params["batch_size"] * dp * 2
    if on_gpu:
        _ext.require()
    trainer = Trainer(params, world_rank)
    trainer._set_train()
    data = next(iter(trainer.train_dataloader))
    inp, tar = trainer._prepare_batch(data)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank] if on_gpu else None)
        if on_gpu:
            torch.cuda.synchronize()

    for _ in range(5 + args.warmup):
        loss = trainer._train_step(inp, tar)
    barrier()
    sampler = ClockSampler(local_rank, _gpu_uuid(torch, local_rank)) if on_gpu else None
    if sampler is not None:
        sampler.start()
    l0 = _ext.launch_count() if on_gpu else 0
    if on_gpu:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    if on_gpu:
        ev0.record()
    for _ in range(args.steps):
        loss = trainer._train_step(inp, tar)
    if on_gpu:
        ev1.record()
    barrier()
    launches = (_ext.launch_count() - l0) if on_gpu else 0
    clocks = sampler.stop() if sampler is not None else None
    t = torch.tensor([ev0.elapsed_time(ev1) if on_gpu else (time.perf_counter() - t0) * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / args.steps
    if on_gpu:
        _ext.check_device_errors(dev)
    if world_rank == 0:
        print(json.dumps({
            "metric": "SFNO-73ch 721x1440 bf16 train samples/s", "value": params["batch_size"] * dp / (ms / 1e3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic N(0,1), random-init weights", "impl": "native",
            "config": {"model": recipe.replace("_bench", ""), "global_batch": params["batch_size"] * dp,
                       "seq_len": f"{params.img_shape_x}x{params.img_shape_y}",
                       "parallelism": f"dp{dp}" + (f"xh{args.h}w{args.w}" if args.h * args.w > 1 else ""),
                       "l2_policy": "inputs+activations per step (>2 GB) exceed the 126 MB L2", "loss": params.loss,
                       "optimizer": type(trainer.optimizer).__name__, "cuda_graph": trainer.graph_mode,
                       "multistep_count": args.multistep, "final_loss": float(loss),
                       "entry": "cli_common.bootstrap -> Trainer._prepare_batch / _train_step (python -m makani_b200.train)"},
            "clocks": clocks, "gpu_launches": launches}))
    sys.stdout.flush()
    if world > 1:
        import threading

        def _bail():
            time.sleep(30.0)
            os._exit(0)

        threading.Thread(target=_bail, daemon=True).start()
        trainer.graph = None
        import gc
        gc.collect()
        if on_gpu:
            torch.cuda.synchronize()
            from makani_b200.parallel import peer
            peer.release_slots()
        dist.barrier(device_ids=[local_rank] if on_gpu else None)
        dist.destroy_process_group()
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    if args.via == "trainer":
        return via_trainer(args)

    import torch
    import torch.distributed as dist

    from makani_b200.ops import _ext
    from makani_b200.utils import comm
    from makani_b200.utils.bench_harness import build_flagship, FlagshipConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus or world == 1, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm.init(model_parallel_sizes=[args.h, args.w, args.fin, args.fout])
    native = args.impl == "native"
    if native:
        _ext.require()
    else:
        _ext.set_native(False)
        torch.backends.cuda.matmul.allow_tf32 = True      # as makani/train.py:109-110
        torch.backends.cudnn.allow_tf32 = True

    cfg = FlagshipConfig(small=args.small, h=args.h, w=args.w, graph=(not args.no_graph) and native, native=native, model=args.model)
    runner = build_flagship(cfg, dev)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    if args.mode == "rollout":
        sampler = ClockSampler(local_rank, _gpu_uuid(torch, local_rank))
        sampler.start()
        ms, launches, finite = runner.rollout(args.steps, args.warmup, world, local_rank, graph=not args.no_graph)
        clocks = sampler.stop()
        _ext.check_device_errors(dev)
        if rank == 0:
            print(json.dumps({
                "metric": "SFNO-73ch 721x1440 bf16 rollout ms/step", "value": ms, "unit": "ms/step", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic N(0,1), random-init weights", "impl": "native",
                "config": {"model": cfg.name, "global_batch": 1, "seq_len": f"{cfg.nlat}x{cfg.nlon}",
                           "parallelism": f"h{args.h}w{args.w}", "cuda_graph": not args.no_graph, "state_finite": finite},
                "clocks": clocks, "gpu_launches": launches}))
        sys.stdout.flush()
        if world > 1:
            import threading

            def _bail():
                time.sleep(30.0)
                os._exit(0)

            threading.Thread(target=_bail, daemon=True).start()
            runner._rollout_graph = None
            import gc
            gc.collect()
            torch.cuda.synchronize()
            from makani_b200.parallel import peer
            peer.release_slots()
            dist.barrier(device_ids=[local_rank])
            dist.destroy_process_group()
        return 0

    # ---------------------------------------------------------------- device-timed steps (inputs resident)
    inp, tgt = runner.synthetic_batch(seed=1234 + rank)
    # untimed priming: the eager steps that size the allocator pools and peer buffers, then the graph capture, so that
    # the W warm-up steps and the K timed steps below are all replays
    for _ in range(5 if cfg.graph else 0):
        runner.step(inp, tgt)
    for _ in range(args.warmup):
        runner.step(inp, tgt)
    barrier()
    sampler = ClockSampler(local_rank, _gpu_uuid(torch, local_rank))
    sampler.start()
    l0 = _ext.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    torch.cuda.profiler.start()     # lets `ncu --profile-from-start off` capture exactly the timed steps
    for _ in range(args.steps):
        loss = runner.step(inp, tgt)
    torch.cuda.profiler.stop()
    ev1.record()
    barrier()
    launches = _ext.launch_count() - l0
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t.item() / args.steps
    mp = args.h * args.w * args.fin * args.fout
    dp = world // mp
    global_batch = cfg.batch_per_gpu * dp
    value = global_batch / (ms_per_step / 1e3)
    if native:
        _ext.check_device_errors(dev)
    final_loss = float(loss)
    if "timeline" in os.environ.get("MAKANI_B200_DP_DIAG", "") and getattr(runner, "reducer", None) is not None:
        rep = runner.reducer.timeline_report()
        if rep is not None and rank == 0:
            print("timeline " + json.dumps(rep), file=sys.stderr)

    # ---------------------------------------------------------------- end to end through the public API
    e2e = None
    if not args.no_e2e:
        e2e = runner.end_to_end(steps=args.steps, warmup=max(1, min(args.warmup, 2)), world=world, local_rank=local_rank)

    if rank == 0:
        out = {
            "metric": ("SFNO-73ch 721x1440 bf16 train samples/s" if args.model == "sfno" else "AFNO-20ch 720x1440 bf16 train samples/s"),
            "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": (value / BASELINE_VALUE) if BASELINE_VALUE else None, "dtype": "bf16" if native else "bf16 autocast (fp32 transforms, as the reference)",
            "data": "synthetic N(0,1), random-init weights", "impl": "native" if native else "restated-torch",
            "config": {"model": cfg.name, "global_batch": global_batch, "seq_len": f"{cfg.nlat}x{cfg.nlon}",
                       "parallelism": f"dp{dp}" + (f"xh{args.h}w{args.w}" if args.h * args.w > 1 else "")
                       + (f"xfin{args.fin}fout{args.fout}" if args.fin * args.fout > 1 else ""), "l2_policy": "inputs+activations per step (>2 GB) exceed the 126 MB L2",
                       "loss": cfg.loss, "optimizer": "AdamW (fused)" if native else "torch.optim.AdamW(foreach)",
                       "cuda_graph": bool(cfg.graph), "final_loss": final_loss,
                       **({"diag": os.environ["MAKANI_B200_DP_DIAG"] + " (not a bench value)"} if os.environ.get("MAKANI_B200_DP_DIAG") else {})},
            "clocks": clocks, "gpu_launches": launches,
        }
        if e2e is not None:
            out["e2e"] = e2e
        print(json.dumps(out))
    # Teardown.  CUDA graphs that hold NCCL kernels must be gone before the communicators are destroyed; a helper
    # thread ends the process if the teardown of the communication libraries stalls, so that a finished measurement
    # can never turn into a hung job.
    sys.stdout.flush()
    if world > 1:
        import gc
        import threading

        def _bail():
            time.sleep(30.0)
            os._exit(0)

        threading.Thread(target=_bail, daemon=True).start()
        torch.cuda.synchronize()
        if getattr(runner.train_step, "graph", None) is not None:
            runner.train_step.graph = None
        gc.collect()
        torch.cuda.synchronize()
        from makani_b200.parallel import peer
        peer.release_slots()
        dist.barrier(device_ids=[local_rank])
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Command-line entry points on the tiny synthetic recipes: training writes checkpoints, a second launch resumes, the
inference entry point scores the trained model, the self-test mode checks the autoregression plumbing."""

import os
import shutil

import pytest
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture()
def recipe(tmp_path):
    cfg = yaml.safe_load(open(os.path.join(ROOT, "config", "debug.yaml")))
    for sec in cfg.values():
        sec["exp_dir"] = str(tmp_path / "runs")
        sec["log_to_screen"] = False
    path = tmp_path / "debug.yaml"
    path.write_text(yaml.safe_dump(cfg))
    return str(path), tmp_path


def _args(path, config, *extra):
    return ["--yaml_config", path, "--config", config, "--enable_synthetic_data", "--run_num", "t0", *extra]


@pytest.mark.parametrize("config", ["tiny_sfno", "tiny_afno", "tiny_vit"])
def test_train_cli_writes_checkpoints(recipe, config):
    from makani_b200 import train
    path, tmp = recipe
    trainer = train.main(_args(path, config))
    exp = tmp / "runs" / config / "t0"
    assert (exp / "training_checkpoints" / "ckpt_mp0.tar").is_file()
    assert (exp / "out.log").is_file()
    assert trainer.iters == 4          # 8 samples per epoch at batch size 2


def test_train_cli_resumes_and_inference_scores(recipe):
    from makani_b200 import inference, train
    path, tmp = recipe
    train.main(_args(path, "tiny_sfno"))
    again = train.main(_args(path, "tiny_sfno"))
    assert again.params.resuming and again.startEpoch >= 1
    inf = inference.main(_args(path, "tiny_sfno"))
    assert inf is not None
    ens = inference.main(_args(path, "tiny_sfno", "--mode", "ensemble", "--ensemble_size", "4", "--ensemble_noise_std", "0.1"))
    res = ens.ensemble_result
    assert res["rmse"].shape == (4, 3) and res["spread"].shape == (4, 3)        # 4 channels, 2 rollout steps + 1
    assert (res["spread"] > 0).all() and (res["rmse"] > 0).all()
    assert os.path.isfile(os.path.join(ens.params.experiment_dir, "ensemble_spread_skill_ratio.npy"))
    one = ens.inference_ensemble(ic=0, n_members=1, noise_std=0.0)
    assert float(one["spread"].abs().sum()) == 0.0


def test_self_test_mode(recipe):
    from makani_b200 import train
    path, _ = recipe
    train.main(_args(path, "tiny_sfno", "--mode", "test"))


def test_quickstart_example_runs(tmp_path):
    import importlib.util
    spec = importlib.util.spec_from_file_location("quickstart", os.path.join(ROOT, "examples", "quickstart.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = mod.main(["--workdir", str(tmp_path)])
    assert out["acc"].shape == (4, 5) and out["pred"].shape[0] == 5
    assert out["scores"]["base"]["validation steps"] > 0


def test_profile_cli_runs_with_a_capture_window(recipe):
    """The profiling entry point trains like the normal one; on CPU the profiler toggles are no-ops but the window
    bookkeeping (start / stop step, ranks, modes) is exercised."""
    from makani_b200 import train_profile
    path, tmp = recipe
    trainer = train_profile.main(_args(path, "tiny_sfno", "--capture_mode", "training", "validation", "--capture_range_start", "1",
                                       "--capture_range_stop", "3", "--capture_ranks", "0"))
    assert trainer.iters == 4
    assert (tmp / "runs" / "tiny_sfno" / "t0" / "training_checkpoints" / "ckpt_mp0.tar").is_file()


def test_makani_alias_package_resolves_to_this_framework():
    """`makani.*` imports give the very module objects of `makani_b200.*` (and `makani.mpu` the parallel layer); the
    upstream command name `python -m makani.train` reaches the same CLI."""
    import subprocess
    import sys
    import os
    import makani
    import makani.utils.comm as c1
    import makani_b200.utils.comm as c2
    import makani.mpu.helpers as h1
    import makani_b200.parallel.helpers as h2
    from makani.models import model_registry
    assert c1 is c2 and h1 is h2
    assert makani.Trainer.__module__ == "makani_b200.utils.trainer"
    assert "SFNO" in model_registry.list_models()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-m", "makani.train", "--help"], cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "--yaml_config" in out.stdout and "--cuda_graph_mode" in out.stdout


def test_package_level_names_of_the_upstream_layout():
    """What the upstream `__init__` files export is importable from the same places here (and through the alias)."""
    import makani
    from makani import Inferencer, Trainer  # noqa: F401
    from makani.models import MultiStepWrapper, Preprocessor2D, SingleStepWrapper, model_registry  # noqa: F401
    from makani.models.common import (MLP, ComplexActivation, ComplexReLU, DropPath, EncoderDecoder,  # noqa: F401
                                      FactorizedSpectralConv, InverseRealFFT2, PatchEmbed, RealFFT2, SpectralAttention, SpectralConv)
    from makani.utils.dataloaders.data_loader_dummy import DummyLoader  # noqa: F401
    from makani.utils.parse_dataset_metada import parse_dataset_metadata  # noqa: F401
    from makani.mpu.mappings import init_gradient_reduction_hooks  # noqa: F401
    from makani.third_party.climt.zenith_angle import cos_zenith_angle

    assert isinstance(makani.__version__, str)
    import datetime

    import numpy as np
    lon, lat = np.meshgrid(np.linspace(0, 360, 8, endpoint=False), np.linspace(90, -90, 5))
    cz = cos_zenith_angle(datetime.datetime(2020, 6, 21, 12, tzinfo=datetime.timezone.utc), lon, lat)
    assert cz.shape == (1, 5, 8) and cz.dtype == np.float32 and abs(float(cz[0, 2, 0]) - 1.0) < 0.1      # noon at 0E on the equator in June
    assert Trainer.__module__ == "makani_b200.utils.trainer"

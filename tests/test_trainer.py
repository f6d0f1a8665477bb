"""End-to-end CPU runs of the Trainer / Inferencer on a tiny on-disk dataset and on synthetic data,
checkpoint round trips (legacy <-> flexible) and the autoregression self test."""

import os

import numpy as np
import pytest
import torch

from makani_b200.utils import checkpoint as ckpt
from makani_b200.utils.inferencer import Inferencer
from makani_b200.utils.trainer import Trainer
from testutils import get_default_parameters, init_dataset


def _params(tmp_path, **over):
    paths = init_dataset(str(tmp_path))
    exp = os.path.join(str(tmp_path), "runs", "cfg", "00")
    os.makedirs(os.path.join(exp, "training_checkpoints"), exist_ok=True)
    p = get_default_parameters(experiment_dir=exp, exp_dir=os.path.join(str(tmp_path), "runs"),
                               checkpoint_path=os.path.join(exp, "training_checkpoints/ckpt_mp{mp_rank}.tar"),
                               best_checkpoint_path=os.path.join(exp, "training_checkpoints/best_ckpt_mp{mp_rank}.tar"),
                               **paths)
    p.update_params(over)
    return p


def test_train_one_epoch_on_files(tmp_path):
    p = _params(tmp_path, n_future=0, valid_autoreg_steps=2)
    trainer = Trainer(p, 0)
    trainer.train()
    assert os.path.isfile(p.checkpoint_path.format(mp_rank=0))
    assert os.path.isfile(p.best_checkpoint_path.format(mp_rank=0))
    logs = trainer.metrics.logs
    assert logs["base"]["validation steps"] > 0
    assert np.isfinite(logs["base"]["validation loss"])
    assert "validation z500" in logs["metrics"] and "ACC AUC t2m" in logs["metrics"]


def test_multistep_history_zenith_and_resume(tmp_path):
    p = _params(tmp_path, n_future=1, n_history=1, add_zenith=True, add_grid=True, grid_num_frequencies=2,
                save_checkpoint="flexible", load_checkpoint="flexible", load_optimizer=False)
    trainer = Trainer(p, 0)
    assert p.N_in_channels == (4 + 1) * 2 + 4
    trainer.train()
    w_before = {k: v.detach().clone() for k, v in trainer.model.named_parameters()}
    p2 = _params(tmp_path, n_future=1, n_history=1, add_zenith=True, add_grid=True, grid_num_frequencies=2,
                 save_checkpoint="flexible", load_checkpoint="flexible", load_optimizer=False, resuming=True, max_epochs=1)
    t2 = Trainer(p2, 0)
    for k, v in t2.model.named_parameters():
        assert torch.equal(v, w_before[k]), k
    assert t2.startEpoch == trainer.epoch


def test_seed_reproducible_synthetic_step():
    def run():
        torch.manual_seed(0)
        p = get_default_parameters(enable_synthetic_data=True, img_shape_x=32, img_shape_y=64, scale_factor=1,
                                   n_train_samples_per_epoch=4, n_eval_samples_per_epoch=2, skip_validation=True,
                                   save_checkpoint="none", train_data_path=None, valid_data_path=None)
        t = Trainer(p, 0)
        _, _, logs = t.train_one_epoch()
        return logs["loss"], [q.detach().clone() for q in t.model.parameters()]
    l1, w1 = run()
    l2, w2 = run()
    assert np.isfinite(l1) and l1 == l2
    for a, b in zip(w1, w2):
        assert torch.equal(a, b)


def test_legacy_and_flexible_checkpoints_are_interchangeable(tmp_path):
    p = _params(tmp_path, skip_validation=True, save_checkpoint="none")
    t = Trainer(p, 0)
    leg = os.path.join(str(tmp_path), "leg_mp{mp_rank}.tar")
    flx = os.path.join(str(tmp_path), "flx_mp{mp_rank}.tar")
    t.save_checkpoint(leg, checkpoint_mode="legacy")
    t.save_checkpoint(flx, checkpoint_mode="flexible")
    ref = {k: v.detach().clone() for k, v in t.model.named_parameters()}
    for path, mode in ((leg, "legacy"), (flx, "flexible"), (leg, "flexible"), (flx, "legacy")):
        with torch.no_grad():
            for v in t.model.parameters():
                v.zero_()
        t.restore_checkpoint(path, checkpoint_mode=mode)
        for k, v in t.model.named_parameters():
            assert torch.equal(v, ref[k]), (mode, k)
    # a checkpoint written from a DDP-wrapped model carries the "module." prefix
    d = ckpt.load_file(leg.format(mp_rank=0))
    d["model_state"] = {"module." + k: v for k, v in d["model_state"].items()}
    torch.save(d, leg.format(mp_rank=0))
    t.restore_checkpoint(leg, checkpoint_mode="legacy")


def test_inferencer_scores_and_single_rollout(tmp_path):
    p = _params(tmp_path, skip_validation=True)
    t = Trainer(p, 0)
    t.save_checkpoint(p.checkpoint_path, checkpoint_mode="legacy")
    pi = _params(tmp_path, n_future=0, valid_autoreg_steps=3)
    inf = Inferencer(pi, 0)
    logs = inf.score_model()
    assert os.path.isfile(os.path.join(pi.experiment_dir, "acc_curves.npy"))
    acc = np.load(os.path.join(pi.experiment_dir, "acc_curves.npy"))
    assert acc.shape == (4, 4)
    targ, pred, logs1, acc1, rmse1 = inf.inference_single(ic=0, compute_metrics=True, output_data=True, output_channels=[0, 1])
    assert pred.shape == targ.shape == (4, 1, 2, 33, 64)
    # the rollout helper reproduces the eager predictions
    data = [x.unsqueeze(0) for x in inf.valid_dataset[0]]
    state, outs = inf.rollout(data[0][:, 0], steps=2, keep_outputs=True)
    assert torch.allclose(outs[0][:, [0, 1]], pred[0], atol=1e-5)


def test_autoregression_self_test_with_debugnet(tmp_path):
    p = _params(tmp_path, nettype="DebugNet", n_history=1, valid_autoreg_steps=2, skip_validation=True, save_checkpoint="none")
    t = Trainer(p, 0)
    assert t.test_autoregression_pipeline()


def test_model_package_round_trip(tmp_path):
    """A finished run can be reloaded from its experiment directory alone and reproduces the trained model's output."""
    import datetime
    from makani_b200.models.model_package import LocalPackage, load_model_package
    p = _params(tmp_path, add_zenith=True)
    trainer = Trainer(p, 0)
    trainer.train()
    exp = p.experiment_dir
    for name in ("config.json", "metadata.json", "global_means.npy", "global_stds.npy"):
        assert os.path.isfile(os.path.join(exp, name)), name
    wrapped = load_model_package(LocalPackage(exp), pretrained=True, device="cpu")
    torch.manual_seed(0)
    x = torch.randn(1, len(p.in_channels), p.img_shape_x, p.img_shape_y)
    t = datetime.datetime(2018, 3, 1, 6, tzinfo=datetime.timezone.utc)
    with torch.no_grad():
        y = wrapped(x, t)
    assert y.shape == (1, len(p.out_channels), p.img_shape_x, p.img_shape_y) and torch.isfinite(y).all()
    # same weights as the trainer's best checkpoint
    best = ckpt.load_file(p.best_checkpoint_path.format(mp_rank=0))["model_state"]
    for k, v in wrapped.model.state_dict().items():
        assert torch.equal(v, best[k.replace("module.", "")]), k


def test_validation_video_is_written(tmp_path):
    """`log_video` renders the first validation rollout (prediction vs target per step) into a GIF."""
    pytest.importorskip("PIL")
    p = _params(tmp_path, log_video=1)
    trainer = Trainer(p, 0)
    assert trainer.visualizer is not None
    trainer.train()
    gifs = [f for f in os.listdir(p.experiment_dir) if f.endswith(".gif")]
    assert gifs, os.listdir(p.experiment_dir)

"""Drop-in parity with the unmodified upstream package: for every network family, the same constructor arguments give
the same state-dict keys and shapes, an upstream state dict loads strictly, and forward output, input gradient and every
parameter gradient agree on CPU in fp32.  Needs the upstream package under `baseline/_ref` (installed offline, not
tracked); skipped when it is absent.  The comparison runs in a child process (`tests/reference_parity_worker.py`)."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASES = ["sfno_dhconv_instance_norm", "sfno_dhconv_scale2_layer_norm", "sfno_diagonal", "sfno_three_layers_frequency_embedding",
         "sfno_coarser_output_grid", "fno", "afno_v1", "afno_v1_thresholded", "afno_v2", "vit", "vit_qkv_bias"]


@pytest.fixture(scope="module")
def results():
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "makani")):
        pytest.skip("upstream package not installed under baseline/_ref")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="4")
    env.pop("PYTHONPATH", None)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "reference_parity_worker.py")] + CASES + ["losses", "metrics", "wrapped1", "wrapped2", "wrapped_features", "reshape_fields", "mpu_layers", "common_layers", "grids", "training_steps", "metrics_handler", "initialisation", "history_and_residual", "checkpoints"],
                          cwd="/tmp", env=env,
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = {}
    for line in proc.stdout.splitlines():
        if line.startswith("{"):
            r = json.loads(line)
            out[r["case"]] = r
    return out


@pytest.mark.parametrize("case", CASES)
def test_network_matches_upstream(results, case):
    r = results[case]
    assert "upstream_error" not in r, r
    assert r["only_upstream"] == [] and r["only_here"] == [] and r["shape_mismatch"] == [], r
    assert r["grad_presence_differs"] == [], r
    assert r["forward"] < 1e-5 and r["input_grad"] < 1e-4 and r["worst_param_grad"] < 1e-4, r


def test_loss_handler_matches_upstream(results):
    r = results["losses"]
    assert len(r["value"]) == 16
    for k, v in r["value"].items():
        assert v < 1e-6, (k, v)
    for k, v in r["grad"].items():
        assert v < 1e-5, (k, v)


@pytest.mark.parametrize("multistep", [1, 2])
def test_wrapped_model_matches_upstream(results, multistep):
    """Registry + preprocessor (sinusoidal grid features) + single- / multi-step wrapper: same state-dict keys as upstream
    (so its checkpoints load), same outputs in evaluation and training mode."""
    r = results[f"wrapped_multistep{multistep}"]
    assert r["wrapper"] == ("SingleStepWrapper" if multistep == 1 else "MultiStepWrapper")
    assert r["only_upstream"] == [] and r["only_here"] == [] and r["shape_mismatch"] == [], r
    assert r["train_shape"][0] == r["train_shape"][1]
    assert r["eval_forward"] < 1e-5 and r["train_forward"] < 1e-5, r


def test_metric_functions_match_upstream(results):
    """GeometricL1 / RMSE / ACC under the three quadrature rules and every reduction mode, and the time quadratures."""
    r = results["metrics"]
    assert len(r["err"]) == 75
    for k, v in r["err"].items():
        assert isinstance(v, float) and v < 1e-5, (k, v)


def test_checkpoints_are_interchangeable_with_upstream(results):
    """Legacy and flexible checkpoints written by the upstream trainer restore here (model, AdamW state, scheduler,
    counters), and checkpoints written here restore in the upstream trainer."""
    r = results["checkpoints"]
    for mode in ("legacy", "flexible"):
        assert r[f"{mode}_forward"] < 1e-6, r
        assert r[f"{mode}_counters"] == [7, 2] and r[f"{mode}_scheduler_epoch"] == 1, r
        assert r[f"upstream_reads_{mode}"] < 1e-6 and r[f"upstream_reads_{mode}_counters"] == [11, 3], r
    assert r["legacy_optimizer_lr"] == 1.0 and r["legacy_optimizer_state"] < 1e-7, r


def test_zenith_history_and_multistep_match_upstream(results):
    r = results["wrapped_features"]
    assert len(r["err"]) == 12
    for k, v in r["err"].items():
        assert isinstance(v, float) and v < 1e-5, (k, v)


def test_reshape_fields_matches_upstream(results):
    """Sample preparation of the numpy data path; upstream itself fails on inputs with grid channels (it reshapes by the
    channel count without them), those combinations are checked for their shape only."""
    r = results["reshape_fields"]
    assert len(r["err"]) == 18 and len(r.get("upstream_failed", [])) == 8
    for k, v in r["err"].items():
        assert isinstance(v, float) and v < 1e-6, (k, v)


def test_channel_parallel_layers_match_upstream_on_one_rank(results):
    r = results["mpu_layers"]
    assert len(r["err"]) == 9
    for k, v in r["err"].items():
        assert isinstance(v, float) and v < 1e-5, (k, v)


def test_common_building_blocks_match_upstream(results):
    r = results["common_layers"]
    assert len(r["err"]) == 13
    for k, v in r["err"].items():
        assert isinstance(v, float) and v < 1e-5, (k, v)


def test_grids_quadrature_and_feature_names_match_upstream(results):
    r = results["grids"]
    assert len(r["err"]) == 14
    for k, v in r["err"].items():
        assert isinstance(v, float) and v < 1e-5, (k, v)


def test_five_training_steps_track_upstream(results):
    """Same model, data, loss and AdamW hyper-parameters on both stacks: loss curve and weights (where the gradient is not
    rounding noise) stay together; the model has complex spectral weights, so this pins the optimiser's complex
    convention to the one of the upstream trainer (stock `torch.optim.AdamW`)."""
    r = results["training_steps"]
    assert r["has_complex"] and r["compared"] >= 20
    assert max(r["loss"]) < 1e-5, r
    assert r["weights"] < 1e-4, r


def test_metrics_handler_matches_upstream(results):
    r = results["metrics_handler"]
    assert r["table_rows"] == 24 and len(r["err"]) == 14
    for k, v in r["err"].items():
        assert isinstance(v, float) and v < 1e-5, (k, v)


def test_parameter_initialisation_matches_upstream(results):
    r = results["initialisation"]
    assert r["off"] == [], r["off"]
    assert r["identical"] > 250 and r["identical"] > 10 * r["same_statistics"], r


def test_history_normalisation_and_residual_targets(results):
    r = results["history_and_residual"]
    assert len(r["err"]) == 5
    for k, v in r["err"].items():
        assert isinstance(v, float) and v < 1e-5, (k, v)

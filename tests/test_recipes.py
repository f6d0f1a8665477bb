"""Every recipe of the shipped configuration files parses and builds its network (on a reduced grid, with a reduced
width where the recipe's own would take minutes on a CPU), and the recipe names of the upstream configuration files
are all present."""

import os

import pytest
import torch
import yaml

from makani_b200.models import model_registry
from makani_b200.utils.YParams import YParams

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FILES = ["sfnonet.yaml", "afnonet.yaml", "vit.yaml", "icml_models.yaml", "debug.yaml"]

UPSTREAM_NAMES = {
    "sfnonet.yaml": ["base_config", "base_73chq", "base_73chq_finetune", "sfno_linear_73chq_sc3_layers8_edim384_wstgl2",
                     "sfno_linear_73chq_sc3_layers8_edim384_asgl2"],
    "afnonet.yaml": ["full_field", "afno_26ch_arxiv_network", "afno_26ch_arxiv_network_finetune", "afno_26ch_arxiv_network_test_config",
                     "afno_26ch_optimized_network", "afno_26ch_optimized_network_finetune"],
    "vit.yaml": ["full_field", "vit_73ch", "vit_73ch_big"],
    "icml_models.yaml": ["base_config", "sfno_dhealy", "sfno_dhealy_26ch_edim128", "sfno_dhealy_26ch_finetune", "sfno_dhealy_26ch",
                         "sfno_dhealy_26ch_2step", "sfno_dhealy_26ch_filterskip", "sfno_dhealy_26ch_nobigskip", "sfno_nonlinear_26ch",
                         "sfno_nonlinear_26ch_2step", "fno_linear_26ch", "fno_linear_26ch_2step", "fno_nonlinear_26ch",
                         "fno_nonlinear_26ch_2step", "sfno_dhealy_73ch", "sfno_dhealy_73ch_2step", "sfno_nonlinear_73ch",
                         "sfno_nonlinear_73ch_2step", "fno_linear_73ch", "fno_linear_73ch_2step", "fno_nonlinear_73ch",
                         "fno_nonlinear_73ch_2step", "sfno_dhealy_73ch_layers12_edim256", "sfno_dhealy_73ch_edim768",
                         "sfno_dhealy_73ch_edim768_debug"],
}


def _recipes():
    out = []
    for f in FILES:
        with open(os.path.join(ROOT, "config", f)) as fh:
            out += [(f, name) for name in yaml.safe_load(fh)]
    return out


@pytest.mark.parametrize("fname", sorted(UPSTREAM_NAMES))
def test_upstream_recipe_names_are_present(fname):
    with open(os.path.join(ROOT, "config", fname)) as fh:
        have = set(yaml.safe_load(fh))
    assert [n for n in UPSTREAM_NAMES[fname] if n not in have] == []


@pytest.mark.parametrize("fname,recipe", _recipes())
def test_recipe_builds_its_network(fname, recipe):
    p = YParams(os.path.join(ROOT, "config", fname), recipe)
    if p.get("nettype") is None:
        pytest.skip("a base section without a network")
    patch = p.get("patch_size", None)
    ph, pw = (patch if isinstance(patch, (list, tuple)) else (patch, patch)) if patch else (1, 1)
    H, W = (4 * ph, 8 * pw) if patch else (32, 64)
    nch = 3
    p.update_params(dict(img_shape_x=H, img_shape_y=W, img_crop_shape_x=H, img_crop_shape_y=W, img_local_shape_x=H, img_local_shape_y=W,
                         img_crop_offset_x=0, img_crop_offset_y=0, img_local_offset_x=0, img_local_offset_y=0,
                         N_in_channels=nch, N_out_channels=nch, in_channels=list(range(nch)), out_channels=list(range(nch)),
                         channel_names=["u10m", "v10m", "t2m"], n_history=0, n_future=0, add_zenith=False, add_grid=False,
                         add_orography=False, add_landmask=False, embed_dim=min(int(p.get("embed_dim", 32)), 32),
                         num_layers=min(int(p.get("num_layers", 2)), 2), depth=min(int(p.get("depth", 2)), 2),
                         num_heads=4, num_blocks=min(int(p.get("num_blocks", 4)), 4), scale_factor=min(int(p.get("scale_factor", 1)), 2),
                         history_normalization_mode="none"))
    torch.manual_seed(0)
    model = model_registry.get_model(p)
    model.eval()
    with torch.no_grad():
        y = model(torch.randn(1, nch, H, W))
    assert tuple(y.shape) == (1, nch, H, W) and torch.isfinite(y).all()

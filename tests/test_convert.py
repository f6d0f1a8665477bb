"""Legacy -> flexible conversion: shards written by a (h, w, fin, fout) layout are re-assembled in rank order."""

import itertools
import os

import torch

from makani_b200.convert_legacy_to_flexible import _rank_of, main, merge_states
from makani_b200.parallel.helpers import compute_split_shapes


def _split(t, dim, n, i):
    return torch.split(t, compute_split_shapes(t.shape[dim], n), dim=dim)[i]


def test_merge_states_inverts_the_sharding():
    torch.manual_seed(0)
    sizes = dict(h=2, w=3, fin=2, fout=1)
    full = {"spec": torch.randn(4, 5, 7, 9), "dh": torch.randn(4, 5, 7), "mlp": torch.randn(6, 10, 1, 1), "rep": torch.randn(3)}
    dims = {"spec": [None, None, "h", "w"], "dh": [None, None, "h"], "mlp": ["fout", "fin", None, None], "rep": [None]}
    nranks = 2 * 3 * 2 * 1
    states = [None] * nranks
    for h, w, fi, fo in itertools.product(range(2), range(3), range(2), range(1)):
        st = {"spec": _split(_split(full["spec"], 2, 2, h), 3, 3, w).clone(), "dh": _split(full["dh"], 2, 2, h).clone(),
              "mlp": _split(_split(full["mlp"], 0, 1, fo), 1, 2, fi).clone(), "rep": full["rep"].clone()}
        states[_rank_of(dict(h=h, w=w, fin=fi, fout=fo), sizes)] = st
    merged = merge_states(states, sizes, dims)
    for k, v in full.items():
        assert torch.equal(merged[k], v), k


def test_converter_cli_on_a_serial_run(tmp_path):
    """With all sizes 1 the converter is a re-packaging of the legacy file plus a model package."""
    from makani_b200.utils import checkpoint as ckpt
    from makani_b200.models import model_registry
    from testutils import get_default_parameters
    p = get_default_parameters(img_shape_x=17, img_shape_y=32, img_crop_shape_x=17, img_crop_shape_y=32, img_crop_offset_x=0,
                               img_crop_offset_y=0, img_local_shape_x=17, img_local_shape_y=32, img_local_offset_x=0,
                               img_local_offset_y=0, N_in_channels=4, N_out_channels=4, experiment_dir=str(tmp_path))
    model = model_registry.get_model(p)
    src = tmp_path / "in"
    src.mkdir()
    torch.save({"iters": 7, "epoch": 2, "model_state": model.state_dict(), "params": p}, src / "ckpt_mp0.tar")
    out = tmp_path / "out"
    main(["--input_path", str(src), "--output_path", str(out)])
    got = ckpt.load_file(str(out / "ckpt_mp0.tar"))
    assert got["iters"] == 7 and got["epoch"] == 2
    for k, v in model.state_dict().items():
        assert torch.equal(got["model_state"][k], v), k
    assert os.path.isfile(out / "config.json")

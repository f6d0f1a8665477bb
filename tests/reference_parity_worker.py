"""Worker of tests/test_reference_parity.py: builds a network of the unmodified upstream package (installed under
`baseline/_ref`, third-party packages stood in for by `baseline/shims`) and the same network of this framework from the
same keyword arguments, loads the upstream state dict into this framework's network (strictly) and compares forward
output and every gradient on CPU in fp32.  Runs in a process of its own because the repository also ships an alias
package named `makani`.  Prints one JSON line per case."""

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))

import importlib
import warnings

warnings.filterwarnings("ignore")

import torch

SFNO = dict(inp_shape=(32, 64), out_shape=(32, 64), scale_factor=1, inp_chans=4, out_chans=3, embed_dim=16, num_layers=2,
            model_grid_type="equiangular", sht_grid_type="legendre-gauss", hard_thresholding_fraction=1.0, use_mlp=True,
            activation_function="gelu", encoder_layers=1, pos_embed="none", big_skip=True)

CASES = {
    "sfno_dhconv_instance_norm": ("sfnonet", "SphericalFourierNeuralOperatorNet", dict(SFNO, operator_type="dhconv", normalization_layer="instance_norm"), (32, 64), 4),
    "sfno_dhconv_scale2_layer_norm": ("sfnonet", "SphericalFourierNeuralOperatorNet",
                                      dict(SFNO, operator_type="dhconv", normalization_layer="layer_norm", scale_factor=2, pos_embed="direct"), (32, 64), 4),
    # 33 latitudes: the upstream diagonal operator can only be built when the two mode counts agree
    "sfno_diagonal": ("sfnonet", "SphericalFourierNeuralOperatorNet",
                      dict(SFNO, inp_shape=(33, 64), out_shape=(33, 64), operator_type="diagonal", normalization_layer="none"), (33, 64), 4),
    "sfno_three_layers_frequency_embedding": ("sfnonet", "SphericalFourierNeuralOperatorNet",
                                              dict(SFNO, operator_type="dhconv", normalization_layer="instance_norm", bias=True, mlp_ratio=3.0,
                                                   num_layers=3, big_skip=False, pos_embed="frequency", encoder_layers=2), (32, 64), 4),
    "sfno_coarser_output_grid": ("sfnonet", "SphericalFourierNeuralOperatorNet",
                                 dict(SFNO, operator_type="dhconv", normalization_layer="instance_norm", out_shape=(16, 32)), (32, 64), 4),
    "fno": ("sfnonet", "FourierNeuralOperatorNet", dict(SFNO, operator_type="dhconv", normalization_layer="instance_norm"), (32, 64), 4),
    "afno_v1": ("afnonet", "AdaptiveFourierNeuralOperatorNet",
                dict(inp_shape=(32, 64), patch_size=(4, 4), inp_chans=4, out_chans=3, embed_dim=32, num_layers=2, num_blocks=4), (32, 64), 4),
    "afno_v1_thresholded": ("afnonet", "AdaptiveFourierNeuralOperatorNet",
                            dict(inp_shape=(32, 64), patch_size=(8, 8), inp_chans=4, out_chans=3, embed_dim=32, num_layers=2, num_blocks=4,
                                 hard_thresholding_fraction=0.5, sparsity_threshold=0.05, mlp_ratio=2.0), (32, 64), 4),
    "afno_v2": ("afnonet_v2", "AdaptiveFourierNeuralOperatorNet",
                dict(inp_shape=(32, 64), patch_size=(4, 4), inp_chans=4, out_chans=3, embed_dim=32, num_layers=2, num_blocks=4), (32, 64), 4),
    "vit": ("vit", "VisionTransformer",
            dict(inp_shape=(32, 64), patch_size=(4, 4), inp_chans=4, out_chans=3, embed_dim=32, depth=2, num_heads=4), (32, 64), 4),
    "vit_qkv_bias": ("vit", "VisionTransformer",
                     dict(inp_shape=(32, 64), patch_size=(8, 8), inp_chans=4, out_chans=3, embed_dim=48, depth=3, num_heads=6, mlp_ratio=2.0,
                          qkv_bias=True), (32, 64), 4),
}


def rel(a, b):
    if a.is_complex():
        a, b = torch.view_as_real(a), torch.view_as_real(b)
    return ((a.double() - b.double()).norm() / (b.double().norm() + 1e-30)).item()


def run(name):
    mod, cls, kw, hw, cin = CASES[name]
    out = {"case": name}
    try:
        ref_cls = getattr(importlib.import_module(f"makani.models.networks.{mod}"), cls)
        torch.manual_seed(0)
        ref = ref_cls(**kw)
    except Exception as e:      # an upstream network that cannot be built with stock arguments is reported, not compared
        out["upstream_error"] = f"{type(e).__name__}: {e}"[:200]
        return out
    if ROOT not in sys.path:
        sys.path.append(ROOT)
    my_cls = getattr(importlib.import_module(f"makani_b200.models.networks.{mod}"), cls)
    mine = my_cls(**kw)
    sr, sm = ref.state_dict(), mine.state_dict()
    out["only_upstream"] = sorted(set(sr) - set(sm))
    out["only_here"] = sorted(set(sm) - set(sr))
    out["shape_mismatch"] = [k for k in sr if k in sm and tuple(sr[k].shape) != tuple(sm[k].shape)]
    if out["only_upstream"] or out["only_here"] or out["shape_mismatch"]:
        return out
    # random values everywhere (biases, norm weights, position embeddings start from constants, which would hide a
    # re-ordering), scaled so that activations stay of order one
    with torch.no_grad():
        for prm in ref.parameters():
            prm.add_(torch.randn_like(prm) * 0.05)
    sr = ref.state_dict()
    mine.load_state_dict(sr, strict=True)
    torch.manual_seed(1)
    x = torch.randn(2, cin, *hw)
    ref.eval()
    mine.eval()
    try:
        with torch.no_grad():
            yr = ref(x)
    except Exception as e:
        out["upstream_error"] = f"forward: {type(e).__name__}: {e}"[:200]
        return out
    with torch.no_grad():
        ym = mine(x)
    out["forward"] = rel(ym, yr)
    ref.train()
    mine.train()
    xr, xm = x.clone().requires_grad_(), x.clone().requires_grad_()
    ref(xr).square().mean().backward()
    mine(xm).square().mean().backward()
    out["input_grad"] = rel(xm.grad, xr.grad)
    gm = dict(mine.named_parameters())
    worst, missing = 0.0, []
    largest = max((p.grad.abs().max().item() for p in ref.parameters() if p.grad is not None), default=0.0)
    for n, p in ref.named_parameters():
        g, h = p.grad, gm[n].grad
        if (g is None) != (h is None):
            missing.append(n)
            continue
        if g is None or g.abs().max().item() < 1e-5 * largest:
            # a gradient that is zero in exact arithmetic (a bias in front of an instance norm): rounding noise on both sides
            if h is not None and h.abs().max().item() > 1e-4 * largest:
                worst = max(worst, 1.0)
            continue
        worst = max(worst, rel(h, g))
    out["worst_param_grad"] = worst
    out["grad_presence_differs"] = missing
    return out


LOSSES = ["l2", "geometric l2", "absolute squared geometric l2", "weighted geometric l2", "geometric l1",
          "absolute squared weighted geometric l2"]

_LOSS_YAML = """
base: &B
    img_shape_x: 33
    img_shape_y: 64
    img_crop_shape_x: 33
    img_crop_shape_y: 64
    img_crop_offset_x: 0
    img_crop_offset_y: 0
    img_local_shape_x: 33
    img_local_shape_y: 64
    img_local_offset_x: 0
    img_local_offset_y: 0
    N_out_channels: 5
    N_in_channels: 5
    n_future: 0
    channel_names: ["u10m", "v10m", "t2m", "z500", "t850"]
    channel_weights: "auto"
    model_grid_type: "equiangular"
    loss: "l2"
    pole_mask: 0
    batch_size: 2
    out_channels: [0, 1, 2, 3, 4]
    in_channels: [0, 1, 2, 3, 4]
"""


def run_losses():
    """`LossHandler(params)` of both packages on the same prediction / target: value and gradient."""
    import tempfile

    from makani.utils.losses import LossHandler as RefLoss
    from makani.utils.YParams import YParams as RefY

    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.utils.losses import LossHandler as MyLoss
    from makani_b200.utils.YParams import YParams as MyY

    path = os.path.join(tempfile.mkdtemp(prefix="parity_"), "c.yaml")
    with open(path, "w") as f:
        f.write(_LOSS_YAML)
    out = {"case": "losses", "value": {}, "grad": {}}
    for grid in ("equiangular", "legendre_gauss"):
        for name in LOSSES:
            pr, pm = RefY(path, "base"), MyY(path, "base")
            for q in (pr, pm):
                q["loss"], q["model_grid_type"] = name, grid
            lr, lm = RefLoss(pr), MyLoss(pm)
            torch.manual_seed(0)
            a = torch.randn(2, 5, 33, 64, requires_grad=True)
            b, i = torch.randn(2, 5, 33, 64), torch.randn(2, 5, 33, 64)
            a2 = a.detach().clone().requires_grad_()
            vr, vm = lr(a, b, i), lm(a2, b, i)
            vr.backward()
            vm.backward()
            out["value"][f"{grid}:{name}"] = abs(float(vr) - float(vm)) / abs(float(vr))
            out["grad"][f"{grid}:{name}"] = rel(a2.grad, a.grad)
    # multistep training: predictions and targets of all steps stacked along the channels, per-step weights
    for nf in (1, 2):
        for name in ("absolute squared geometric l2", "weighted geometric l1"):
            pr, pm = RefY(path, "base"), MyY(path, "base")
            for q in (pr, pm):
                q["loss"], q["n_future"] = name, nf
            lr, lm = RefLoss(pr).train(), MyLoss(pm).train()
            torch.manual_seed(nf)
            a = torch.randn(2, 5 * (nf + 1), 33, 64, requires_grad=True)
            b, i = torch.randn(2, 5 * (nf + 1), 33, 64), torch.randn(2, 5, 33, 64)
            a2 = a.detach().clone().requires_grad_()
            vr, vm = lr(a, b, i), lm(a2, b, i)
            vr.backward()
            vm.backward()
            out["value"][f"multistep{nf + 1}:{name}"] = abs(float(vr) - float(vm)) / abs(float(vr))
            out["grad"][f"multistep{nf + 1}:{name}"] = rel(a2.grad, a.grad)
    return out


def run_metrics():
    """The geometric metric functions and the time quadratures of both packages on the same fields."""
    from makani.utils.metrics import functions as RF

    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.utils.metrics import functions as MF

    out = {"case": "metrics", "err": {}}
    torch.manual_seed(0)
    x, y = torch.randn(3, 5, 33, 64), torch.randn(3, 5, 33, 64)
    for grid in ("naive", "legendre-gauss", "clenshaw-curtiss"):      # the first argument is the quadrature rule
        for name in ("GeometricL1", "GeometricRMSE", "GeometricACC"):
            for cr, br in (("mean", "mean"), ("none", "mean"), ("none", "none"), ("sum", "sum")):
                for norm in (False, True):
                    kw = dict(grid_type=grid, img_shape=(33, 64), crop_shape=(33, 64), crop_offset=(0, 0), normalize=norm,
                              channel_reduction=cr, batch_reduction=br)
                    a, b = getattr(RF, name)(**kw)(x, y), getattr(MF, name)(**kw)(x, y)
                    key = f"{grid}:{name}:{cr}:{br}:{int(norm)}"
                    out["err"][key] = rel(b, a) if tuple(a.shape) == tuple(b.shape) else f"shape {tuple(a.shape)} vs {tuple(b.shape)}"
    t = torch.randn(4, 9, 3)
    for name, n in (("SimpsonQuadrature", 8), ("TrapezoidQuadrature", 8), ("Quadrature", 8)):
        a = getattr(RF, name)(n, 0.25, torch.device("cpu"))(t, dim=1)
        b = getattr(MF, name)(n, 0.25, torch.device("cpu"))(t, dim=1)
        out["err"][name] = rel(b, a) if tuple(a.shape) == tuple(b.shape) else f"shape {tuple(a.shape)} vs {tuple(b.shape)}"
    return out


def run_wrapped(multistep):
    """`model_registry.get_model(params)` (network inside the single- / multi-step wrapper with its preprocessor) of
    both packages from the same recipe: state dict, evaluation forward, training forward (all autoregressive steps)."""
    import logging

    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as RA
    from makani.models import model_registry
    from makani.utils import comm
    from makani.utils.trainer import Trainer
    from makani.utils.YParams import YParams

    sizes = [1, 1, 1, 1]
    comm.init(model_parallel_sizes=sizes, model_parallel_names=["h", "w", "fin", "fout"], verbose=False)
    recipe = os.path.join(ROOT, "config", "sfnonet.yaml")
    params = YParams(recipe, "sfno_tiny")
    nlat, nlon, n_out = params.img_shape_x, params.img_shape_y, len(params.channel_names)
    for k, v in dict(model_parallel_sizes=sizes, model_parallel_names=["h", "w", "fin", "fout"], world_size=1, global_batch_size=2,
                     batch_size=2, experiment_dir="/tmp/parity", resuming=False, amp_mode="none", jit_mode="none",
                     cuda_graph_mode="none", skip_validation=True, enable_odirect=False, checkpointing=0,
                     enable_synthetic_data=True, split_data_channels=False, multistep_count=multistep, n_future=multistep - 1,
                     add_grid=True, add_zenith=False, add_orography=False, add_landmask=False, gridtype="sinusoidal",
                     grid_num_frequencies=2).items():
        params[k] = v
    tr = Trainer.__new__(Trainer)
    tr.params, tr.world_rank, tr.data_parallel_rank = None, 0, 0
    tr.device, tr.logger = torch.device("cpu"), logging.getLogger()
    tr.valid_dataset = RA._SyntheticDataset(n_out, n_out, nlat, nlon, [nlat], [nlon], 0, 0)
    params = tr._update_parameters(params)      # upstream derives the channel counts etc.
    torch.manual_seed(0)
    ref = model_registry.get_model(params)
    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.models import model_registry as my_registry
    from makani_b200.utils.YParams import YParams as MyY

    mp = MyY(recipe, "sfno_tiny")
    for k, v in params.to_dict().items():
        mp[k] = v
    mine = my_registry.get_model(mp)
    sr, sm = ref.state_dict(), mine.state_dict()
    out = {"case": f"wrapped_multistep{multistep}", "wrapper": type(ref).__name__,
           "only_upstream": sorted(set(sr) - set(sm)), "only_here": sorted(set(sm) - set(sr)),
           "shape_mismatch": [k for k in sr if k in sm and tuple(sr[k].shape) != tuple(sm[k].shape)]}
    if out["only_upstream"] or out["only_here"] or out["shape_mismatch"]:
        return out
    mine.load_state_dict(sr, strict=True)
    x = torch.randn(2, n_out, nlat, nlon)
    ref.eval()
    mine.eval()
    with torch.no_grad():
        out["eval_forward"] = rel(mine(x), ref(x))
    ref.train()
    mine.train()
    yr, ym = ref(x), mine(x)
    out["train_shape"] = [list(yr.shape), list(ym.shape)]
    out["train_forward"] = rel(ym, yr)
    return out


def _upstream_trainer(multistep=1, extra=None):
    """An upstream Trainer object assembled far enough to build the model and to save / restore checkpoints."""
    import logging

    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as RA
    from makani.models import model_registry
    from makani.utils import comm
    from makani.utils.trainer import Trainer
    from makani.utils.YParams import YParams

    sizes = [1, 1, 1, 1]
    comm.init(model_parallel_sizes=sizes, model_parallel_names=["h", "w", "fin", "fout"], verbose=False)
    recipe = os.path.join(ROOT, "config", "sfnonet.yaml")
    params = YParams(recipe, "sfno_tiny")
    nlat, nlon, n_out = params.img_shape_x, params.img_shape_y, len(params.channel_names)
    for k, v in dict(model_parallel_sizes=sizes, model_parallel_names=["h", "w", "fin", "fout"], world_size=1, global_batch_size=2,
                     batch_size=2, experiment_dir="/tmp/parity", resuming=False, amp_mode="none", jit_mode="none",
                     cuda_graph_mode="none", skip_validation=True, enable_odirect=False, checkpointing=0,
                     enable_synthetic_data=True, split_data_channels=False, multistep_count=multistep, n_future=multistep - 1,
                     add_grid=True, add_zenith=False, add_orography=False, add_landmask=False, gridtype="sinusoidal",
                     grid_num_frequencies=2, log_to_screen=False).items():
        params[k] = v
    for k, v in (extra or {}).items():
        params[k] = v
    tr = Trainer.__new__(Trainer)
    tr.params, tr.world_rank, tr.data_parallel_rank = None, 0, 0
    tr.device, tr.logger = torch.device("cpu"), logging.getLogger()
    tr.valid_dataset = RA._SyntheticDataset(n_out, n_out, nlat, nlon, [nlat], [nlon], 0, 0)
    params = tr._update_parameters(params)
    tr.params = params
    torch.manual_seed(0)
    tr.model = model_registry.get_model(params)
    return tr, params, recipe


def run_wrapped_features():
    """Zenith-angle channels (cached per step), input history and multistep training through the wrappers of both
    packages: training-mode and evaluation-mode forward for every combination."""
    if ROOT not in sys.path:
        sys.path.append(ROOT)
    out = {"case": "wrapped_features", "err": {}}
    for ms, zen, nh in [(1, True, 0), (2, True, 0), (2, False, 1), (1, True, 1), (2, True, 1), (3, True, 2)]:
        tr, params, recipe = _upstream_trainer(ms, dict(add_zenith=zen, n_history=nh, add_grid=False))
        from makani_b200.models import model_registry as my_registry
        from makani_b200.utils.YParams import YParams as MyY

        mp = MyY(recipe, "sfno_tiny")
        for k, v in params.to_dict().items():
            mp[k] = v
        ref, mine = tr.model, my_registry.get_model(mp)
        mine.load_state_dict(ref.state_dict(), strict=True)
        nlat, nlon, C = params.img_shape_x, params.img_shape_y, len(params.channel_names)
        torch.manual_seed(ms * 10 + nh)
        inp, tar = torch.randn(2, (nh + 1) * C, nlat, nlon), torch.randn(2, ms * C, nlat, nlon)
        izen = torch.rand(2, nh + 1, 1, nlat, nlon) if zen else None
        tzen = torch.rand(2, ms, 1, nlat, nlon) if zen else None
        for mode in ("train", "eval"):
            outs = []
            for m in (ref, mine):
                m.train() if mode == "train" else m.eval()
                with torch.no_grad():
                    # every model gets its own copies: the upstream preprocessor keeps (and later overwrites) the caller's tensors
                    ip, _ = m.preprocessor.cache_unpredicted_features(inp.clone(), tar.clone(), None if izen is None else izen.clone(),
                                                                      None if tzen is None else tzen.clone())
                    outs.append(m(m.preprocessor.flatten_history(ip)))
            same = tuple(outs[0].shape) == tuple(outs[1].shape)
            out["err"][f"multistep{ms}_zenith{int(zen)}_history{nh}_{mode}"] = rel(outs[1], outs[0]) if same else "shape"
    return out


def run_reshape_fields():
    """`utils.img_utils.reshape_fields` (sample preparation of the numpy data path) of both packages."""
    import tempfile
    import types

    import numpy as np
    from makani.utils.img_utils import reshape_fields as ref_fn

    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.utils.img_utils import reshape_fields as my_fn

    d = tempfile.mkdtemp(prefix="parity_fields_")
    rng = np.random.default_rng(0)
    C = 6
    stats = {}
    for name, arr in (("min", rng.normal(size=(1, C, 1, 1)) - 3), ("max", rng.normal(size=(1, C, 1, 1)) + 3),
                      ("mean", rng.normal(size=(1, C, 1, 1))), ("std", rng.uniform(0.5, 2.0, size=(1, C, 1, 1)))):
        stats[name] = os.path.join(d, name + ".npy")
        np.save(stats[name], arr.astype(np.float32))
    out = {"case": "reshape_fields", "err": {}}
    for norm in ("zscore", "minmax"):
        for grid in (None, "linear", "sinusoidal"):
            for which, nhist, train in (("inp", 1, True), ("inp", 0, False), ("tar", 0, True)):
                chans = [0, 2, 3, 5]
                p = types.SimpleNamespace(in_channels=chans, out_channels=chans, min_path=stats["min"], max_path=stats["max"],
                                          global_means_path=stats["mean"], global_stds_path=stats["std"], normalization=norm,
                                          add_grid=grid is not None, gridtype=grid, n_grid_channels={None: 0, "linear": 2, "sinusoidal": 4}[grid],
                                          roll=True)
                img = rng.normal(size=(nhist + 1, len(chans), 24, 48)).astype(np.float32)
                # evaluation samples are not cropped: the window is the whole field there
                args = (which, 16, 32, 3, 5, p, 7, train) if train else (which, 24, 48, 0, 0, p, 7, train)
                key = f"{norm}:{grid}:{which}:{nhist}:{int(train)}"
                b = my_fn(img.copy(), *args)
                try:
                    a = ref_fn(img.copy(), *args)
                except ValueError:
                    # upstream reshapes an input with grid channels by the channel count without them and fails;
                    # checked here instead: data channels first, then the grid channels, per history step
                    n_grid = p.n_grid_channels
                    ok = which == "inp" and n_grid > 0 and b.shape[0] == (nhist + 1) * (len(chans) + n_grid)
                    out["err"][key] = 0.0 if ok else "upstream failed and the shape here is unexpected"
                    out.setdefault("upstream_failed", []).append(key)
                    continue
                out["err"][key] = rel(b.double(), a.double()) if tuple(a.shape) == tuple(b.shape) else f"shape {tuple(a.shape)} vs {tuple(b.shape)}"
    return out


def run_mpu_layers():
    """The channel-parallel layer classes of `makani.mpu` against `makani_b200.parallel` on one rank: same state dict,
    and with the same (random) weights the same output, input gradient and parameter gradients."""
    from makani.mpu import layer_norm as RN
    from makani.mpu import layers as RL
    from makani.utils import comm

    sizes, names = [1, 1, 1, 1], ["h", "w", "fin", "fout"]
    comm.init(model_parallel_sizes=sizes, model_parallel_names=names, verbose=False)
    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.parallel import layer_norm as MN
    from makani_b200.parallel import layers as ML
    from makani_b200.utils import comm as my_comm

    my_comm.init(model_parallel_sizes=sizes, model_parallel_names=names)
    gelu = torch.nn.GELU
    cases = [
        ("matmul_nchw", "DistributedMatmul", RL, ML, dict(inp_dim=6, out_dim=5, input_format="nchw", bias=True), (2, 6, 8, 16)),
        ("matmul_tokens", "DistributedMatmul", RL, ML, dict(inp_dim=6, out_dim=5, input_format="traditional", bias=True), (2, 7, 6)),
        ("mlp_nchw", "DistributedMLP", RL, ML, dict(in_features=6, hidden_features=12, out_features=6, input_format="nchw", act_layer=gelu), (2, 6, 8, 16)),
        ("mlp_tokens", "DistributedMLP", RL, ML, dict(in_features=6, hidden_features=12, out_features=6, input_format="traditional", act_layer=gelu), (2, 9, 6)),
        ("patch_embed", "DistributedPatchEmbed", RL, ML, dict(img_size=(16, 32), patch_size=(4, 4), in_chans=3, embed_dim=8,
                                                              input_is_matmul_parallel=False, output_is_matmul_parallel=True), (2, 3, 16, 32)),
        ("attention_bias", "DistributedAttention", RL, ML, dict(dim=16, input_format="traditional", num_heads=4, qkv_bias=True), (2, 9, 16)),
        ("attention_qk_norm", "DistributedAttention", RL, ML, dict(dim=16, input_format="traditional", num_heads=4, qk_norm=True), (2, 9, 16)),
        ("layer_norm", "DistributedLayerNorm", RN, MN, dict(normalized_shape=5, elementwise_affine=True), (2, 5, 8, 16)),
        ("real_fft2", "DistributedRealFFT2", RL, ML, dict(nlat=8, nlon=16), (2, 3, 8, 16)),
    ]
    out = {"case": "mpu_layers", "err": {}}
    for tag, name, R, M, kw, shape in cases:
        torch.manual_seed(0)
        r, m = getattr(R, name)(**kw), getattr(M, name)(**kw)
        sr, sm = r.state_dict(), m.state_dict()
        if set(sr) != set(sm) or any(tuple(sr[k].shape) != tuple(sm[k].shape) for k in sr):
            out["err"][tag] = f"state dict differs: {sorted(set(sr) ^ set(sm))}"
            continue
        with torch.no_grad():
            for prm in r.parameters():       # the upstream classes start from all-ones weights: that hides any re-ordering
                prm.copy_(torch.randn_like(prm) * 0.3)
        m.load_state_dict(r.state_dict())
        x = torch.randn(*shape)
        xr, xm = x.clone().requires_grad_(), x.clone().requires_grad_()
        yr, ym = r(xr), m(xm)
        if tuple(yr.shape) != tuple(ym.shape):
            out["err"][tag] = f"output shape {tuple(yr.shape)} vs {tuple(ym.shape)}"
            continue
        worst = rel(ym, yr)
        yr.abs().square().sum().backward()
        ym.abs().square().sum().backward()
        worst = max(worst, rel(xm.grad, xr.grad))
        gm = dict(m.named_parameters())
        for n, prm in r.named_parameters():
            if prm.grad is not None:
                worst = max(worst, rel(gm[n].grad, prm.grad))
        out["err"][tag] = worst
    return out


def run_common_layers():
    """Building blocks of `makani.models.common` against this framework's, one by one, with random weights: MLP,
    EncoderDecoder, the FFT wrappers, the complex activations and the spectral convolution (SHT and FFT flavours)."""
    import torch_harmonics as th
    from makani.models.common import activations as RA
    from makani.models.common import layers as RL
    from makani.models.common import spectral_convolution as RS
    from makani.utils import comm

    sizes, names = [1, 1, 1, 1], ["h", "w", "fin", "fout"]
    comm.init(model_parallel_sizes=sizes, model_parallel_names=names, verbose=False)
    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.models.common import activations as MA
    from makani_b200.models.common import layers as ML
    from makani_b200.models.common import spectral_convolution as MS
    from makani_b200.sht import sht as my_sht
    from makani_b200.utils import comm as my_comm

    my_comm.init(model_parallel_sizes=sizes, model_parallel_names=names)
    gelu, nlat, nlon = torch.nn.GELU, 16, 32
    real, cplx, spec = (2, 6, 8, 16), "complex", "spectral"

    def build(tag):
        if tag == "spectral_conv_sht":
            kw = dict(operator_type="dhconv", bias=True)
            return (RS.SpectralConv(th.RealSHT(nlat, nlon, grid="legendre-gauss").float(), th.InverseRealSHT(nlat, nlon, grid="legendre-gauss").float(), 6, 6, **kw),
                    MS.SpectralConv(my_sht.RealSHT(nlat, nlon, grid="legendre-gauss"), my_sht.InverseRealSHT(nlat, nlon, grid="legendre-gauss"), 6, 6, **kw))
        if tag == "spectral_conv_fft":
            kw = dict(operator_type="dhconv", bias=False)
            return (RS.SpectralConv(RL.RealFFT2(nlat, nlon), RL.InverseRealFFT2(nlat, nlon), 6, 6, **kw),
                    MS.SpectralConv(ML.RealFFT2(nlat, nlon), ML.InverseRealFFT2(nlat, nlon), 6, 6, **kw))
        raise KeyError(tag)

    cases = [
        ("mlp_nchw", "MLP", RL, ML, dict(in_features=6, hidden_features=12, out_features=5, act_layer=gelu, output_bias=True, input_format="nchw"), real),
        ("mlp_tokens", "MLP", RL, ML, dict(in_features=6, hidden_features=12, out_features=5, act_layer=gelu, output_bias=False, input_format="traditional"), (2, 9, 6)),
        ("encoder_nchw", "EncoderDecoder", RL, ML, dict(num_layers=2, input_dim=6, output_dim=5, hidden_dim=8, act_layer=gelu, input_format="nchw"), real),
        ("encoder_tokens", "EncoderDecoder", RL, ML, dict(num_layers=1, input_dim=6, output_dim=5, hidden_dim=8, act_layer=gelu, input_format="traditional"), (2, 9, 6)),
        ("rfft2", "RealFFT2", RL, ML, dict(nlat=8, nlon=16, lmax=6, mmax=5), real),
        ("irfft2", "InverseRealFFT2", RL, ML, dict(nlat=8, nlon=16, lmax=6, mmax=5), spec),
        ("crelu_cartesian", "ComplexReLU", RA, MA, dict(negative_slope=0.1, mode="cartesian", bias_shape=(3, 1, 1)), cplx),
        ("crelu_modulus", "ComplexReLU", RA, MA, dict(negative_slope=0.0, mode="modulus", bias_shape=(3, 1, 1), scale=2.0), cplx),
        ("crelu_real", "ComplexReLU", RA, MA, dict(negative_slope=0.0, mode="real"), cplx),
        ("cact_cartesian", "ComplexActivation", RA, MA, dict(activation=torch.nn.Tanh(), mode="cartesian", bias_shape=(3, 1, 1)), cplx),
        ("cact_modulus", "ComplexActivation", RA, MA, dict(activation=torch.nn.Tanh(), mode="modulus", bias_shape=(3, 1, 1)), cplx),
        ("spectral_conv_sht", None, None, None, None, (2, 6, nlat, nlon)),
        ("spectral_conv_fft", None, None, None, None, (2, 6, nlat, nlon)),
    ]
    out = {"case": "common_layers", "err": {}}
    for tag, name, R, M, kw, shape in cases:
        torch.manual_seed(0)
        r, m = build(tag) if name is None else (getattr(R, name)(**kw), getattr(M, name)(**kw))
        sr, sm = r.state_dict(), m.state_dict()
        if set(sr) != set(sm) or any(tuple(sr[k].shape) != tuple(sm[k].shape) for k in sr):
            out["err"][tag] = f"state dict differs: {sorted(set(sr) ^ set(sm))}"
            continue
        with torch.no_grad():
            for prm in r.parameters():
                prm.copy_(torch.randn_like(prm) * 0.3)
        m.load_state_dict(r.state_dict())
        x = (torch.randn(2, 3, 8, 9, dtype=torch.complex64) if shape == cplx
             else torch.randn(2, 3, 6, 5, dtype=torch.complex64) if shape == spec else torch.randn(*shape))
        xr, xm = x.clone().requires_grad_(), x.clone().requires_grad_()
        yr, ym = r(xr), m(xm)
        worst = 0.0
        if isinstance(yr, tuple):                      # spectral convolutions also return the (regridded) residual
            worst = rel(ym[1], yr[1])
            yr, ym = yr[0], ym[0]
        if tuple(yr.shape) != tuple(ym.shape):
            out["err"][tag] = f"output shape {tuple(yr.shape)} vs {tuple(ym.shape)}"
            continue
        worst = max(worst, rel(ym, yr))
        yr.abs().square().sum().backward()
        ym.abs().square().sum().backward()
        worst = max(worst, rel(xm.grad, xr.grad))
        gm = dict(m.named_parameters())
        for n, prm in r.named_parameters():
            if prm.grad is not None:
                worst = max(worst, rel(gm[n].grad, prm.grad))
        out["err"][tag] = worst
    return out


def run_grids():
    """Grid conversion, quadrature weights (three rules, cropped and normalised) and the auxiliary channel names."""
    import numpy as np
    from makani.utils import features as RF
    from makani.utils import grids as RG

    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.utils import features as MF
    from makani_b200.utils import grids as MG

    out = {"case": "grids", "err": {}}
    lat = torch.linspace(np.pi / 2, -np.pi / 2, 17).double()
    lon = torch.linspace(0, 2 * np.pi, 33)[:-1].double()
    torch.manual_seed(0)
    x = torch.randn(2, 3, 17, 32)
    for src, dst in (("equiangular", "legendre-gauss"), ("equiangular", "equiangular")):
        r, m = RG.GridConverter(src, dst, lat, lon), MG.GridConverter(src, dst, lat, lon)
        out["err"][f"converter:{src}:{dst}"] = max(rel(m(x), r(x)), rel(torch.as_tensor(m.get_dst_coords()[0]), torch.as_tensor(r.get_dst_coords()[0])))
    for rule in ("naive", "clenshaw-curtiss", "legendre-gauss"):
        for tag, kw in (("full", {}), ("crop", dict(crop_shape=(8, 16), crop_offset=(4, 8))), ("normalized", dict(normalize=True))):
            r, m = RG.GridQuadrature(rule, (17, 32), **kw), MG.GridQuadrature(rule, (17, 32), **kw)
            xx = x[..., :8, :16] if tag == "crop" else x
            out["err"][f"quadrature:{rule}:{tag}"] = rel(m(xx), r(xx))
    for i, kw in enumerate((dict(add_zenith=True, add_grid=True, grid_type="sinusoidal", grid_num_frequencies=2, add_orography=True, add_landmask=True),
                            dict(add_grid=True, grid_type="linear", add_landmask=True), dict(add_zenith=True))):
        out["err"][f"aux_channels:{i}"] = 0.0 if RF.get_auxiliary_channels(**kw) == MF.get_auxiliary_channels(**kw) else 1.0
    return out


def run_training_steps():
    """Five optimisation steps of the two stacks side by side (wrapped SFNO with two-step training, LossHandler, AdamW
    with weight decay; the upstream side uses what its trainer instantiates, this side the fused optimiser's CPU path):
    the loss curves and the final weights, complex spectral weights included, stay together."""
    from makani.utils.losses import LossHandler as RefLoss

    tr, params, recipe = _upstream_trainer(2, dict(add_grid=False))
    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.models import model_registry as my_registry
    from makani_b200.ops.optim import FusedAdamW
    from makani_b200.utils.losses import LossHandler as MyLoss
    from makani_b200.utils.YParams import YParams as MyY

    mp = MyY(recipe, "sfno_tiny")
    for k, v in params.to_dict().items():
        mp[k] = v
    ref, mine = tr.model, my_registry.get_model(mp)
    mine.load_state_dict(ref.state_dict(), strict=True)
    lr_, lm_ = RefLoss(params), MyLoss(mp)
    betas = (params.optimizer_beta1, params.optimizer_beta2)
    opt_r = torch.optim.AdamW(ref.parameters(), betas=betas, lr=1e-2, weight_decay=0.05, foreach=True)
    opt_m = FusedAdamW(mine.parameters(), betas=betas, lr=1e-2, weight_decay=0.05)
    nlat, nlon, C = params.img_shape_x, params.img_shape_y, len(params.channel_names)
    out = {"case": "training_steps", "loss": [], "has_complex": any(p.is_complex() for p in ref.parameters())}
    ref.train()
    mine.train()
    lr_.train()
    lm_.train()
    for step in range(5):
        g = torch.Generator().manual_seed(step)
        inp, tar = torch.randn(2, C, nlat, nlon, generator=g), torch.randn(2, 2 * C, nlat, nlon, generator=g)
        losses = []
        for model, loss_fn, opt in ((ref, lr_, opt_r), (mine, lm_, opt_m)):
            opt.zero_grad(set_to_none=True)
            loss = loss_fn(model(inp.clone()), tar.clone(), inp.clone())
            loss.backward()
            opt.step()
            losses.append(float(loss))
        out["loss"].append(abs(losses[1] - losses[0]) / abs(losses[0]))
    # Adam turns a gradient that is zero in exact arithmetic (a bias in front of an instance norm) into steps of +-lr
    # whose sign is rounding noise: such parameters are left out of the comparison
    pm = dict(mine.named_parameters())
    largest = max(p.grad.abs().max().item() for p in ref.parameters() if p.grad is not None)
    live = [n for n, p in ref.named_parameters() if p.grad is not None and p.grad.abs().max().item() > 1e-4 * largest]
    out["compared"], out["left_out"] = len(live), len(pm) - len(live)
    pr = dict(ref.named_parameters())

    def masked_rel(n):
        # the same holds element by element inside a tensor (e.g. spectral weights of modes that carry no signal)
        a, b, g = pm[n].detach(), pr[n].detach(), pr[n].grad
        if a.is_complex():
            a, b, g = torch.view_as_real(a), torch.view_as_real(b), torch.view_as_real(g)
        keep = g.abs() > 1e-3 * g.abs().max()
        return ((a - b)[keep].double().norm() / (b[keep].double().norm() + 1e-30)).item()

    out["weights"] = max(masked_rel(n) for n in live)
    return out


def run_metrics_handler():
    """`MetricsHandler` of both packages fed with the same rollout: scalar logs, ACC / RMSE curves and the rollout table."""
    os.environ["TORCHDYNAMO_DISABLE"] = "1"       # upstream wraps its metric handles in torch.compile
    import numpy as np

    tr, params, recipe = _upstream_trainer(1, dict(add_grid=False, dhours=6, dt=1))
    from makani.utils.metric import MetricsHandler as RefHandler

    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.utils.metric import MetricsHandler as MyHandler
    from makani_b200.utils.YParams import YParams as MyY

    mp = MyY(recipe, "sfno_tiny")
    for k, v in params.to_dict().items():
        mp[k] = v
    names = list(params.channel_names)
    C, H, W = len(names), params.img_shape_x, params.img_shape_y
    torch.manual_seed(0)
    mult, clim, dev = torch.rand(C) + 0.5, torch.randn(C, H, W) * 0.1, torch.device("cpu")
    kw = dict(rmse_var_names=names, acc_vars_names=names, acc_auc_var_names=names)
    r, m = RefHandler(params, mult, clim, dev, **kw), MyHandler(mp, mult.clone(), clim.clone(), dev, **kw)
    for h in (r, m):
        h.initialize_buffers()
        h.zero_buffers()
    for it in range(3):
        for idt in range(params.valid_autoreg_steps + 1):
            p, t = torch.randn(2, C, H, W), torch.randn(2, C, H, W)
            loss = torch.tensor(1.0 + 0.1 * (it + idt))
            r.update(p.clone(), t.clone(), loss.clone(), idt)
            m.update(p.clone(), t.clone(), loss.clone(), idt)
    (lr, acc_r, rmse_r), (lm, acc_m, rmse_m) = r.finalize(final_inference=True), m.finalize(final_inference=True)
    out = {"case": "metrics_handler", "err": {"acc_curve": rel(acc_m, acc_r), "rmse_curve": rel(rmse_m, rmse_r)}}
    for sec in ("base", "metrics"):
        for k, v in lr[sec].items():
            if k == "rollouts":
                continue
            out["err"][f"{sec}/{k}"] = (abs(float(lm[sec][k]) - float(v)) / (abs(float(v)) + 1e-30)) if k in lm[sec] else "missing here"
    rows_r = [list(row) for row in lr["metrics"]["rollouts"].data]
    tab = lm["metrics"]["rollouts"]
    rows_m = [list(row) for row in (tab["data"] if isinstance(tab, dict) else tab.data)]
    same_labels = [x[:3] for x in rows_r] == [x[:3] for x in rows_m]
    vals = max(abs(float(a[3]) - float(b[3])) / (abs(float(a[3])) + 1e-30) for a, b in zip(rows_r, rows_m)) if same_labels else 1.0
    out["err"]["rollout_table"] = vals if same_labels and len(rows_r) == len(rows_m) else "labels differ"
    out["table_rows"] = len(rows_r)
    return out


def run_initialisation():
    """Constructed from the same seed, most parameter tensors of the two packages are bit-identical; the rest (drawn in
    another order) must at least have the same spread and mean."""
    if ROOT not in sys.path:
        sys.path.append(ROOT)
    out = {"case": "initialisation", "identical": 0, "same_statistics": 0, "off": []}
    for name, (mod, cls, kw, hw, cin) in CASES.items():
        ref_cls = getattr(importlib.import_module(f"makani.models.networks.{mod}"), cls)
        my_cls = getattr(importlib.import_module(f"makani_b200.models.networks.{mod}"), cls)
        torch.manual_seed(0)
        sr = ref_cls(**kw).state_dict()
        torch.manual_seed(0)
        sm = my_cls(**kw).state_dict()
        for k, a in sr.items():
            b = sm[k]
            if a.is_complex():
                a, b = torch.view_as_real(a), torch.view_as_real(b)
            a, b = a.float(), b.float()
            if torch.equal(a, b):
                out["identical"] += 1
                continue
            sa, sb = a.std().item(), b.std().item()
            tol_mean = 4.0 * sa / (a.numel() ** 0.5) + 1e-6
            if abs(sa - sb) <= 0.1 * sa + 1e-8 and abs(a.mean().item() - b.mean().item()) <= 2 * tol_mean:
                out["same_statistics"] += 1
            else:
                out["off"].append(f"{name}:{k}: std {sa:.4g} vs {sb:.4g}, mean {a.mean().item():.3g} vs {b.mean().item():.3g}")
    return out


def run_history_and_residual():
    """Exponential history normalisation through the wrappers, and residual targets: with `target: residual` the
    upstream multistep wrapper adds the increment in place to its own input, so its first-step output is overwritten by
    the second step; the check here is against its evaluation-mode steps chained by hand."""
    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.models import model_registry as my_registry
    from makani_b200.utils.YParams import YParams as MyY

    def pair(extra):
        tr, params, recipe = _upstream_trainer(2, dict(add_grid=False, **extra))
        mp = MyY(recipe, "sfno_tiny")
        for k, v in params.to_dict().items():
            mp[k] = v
        mine = my_registry.get_model(mp)
        mine.load_state_dict(tr.model.state_dict(), strict=True)
        return tr.model, mine, params

    out = {"case": "history_and_residual", "err": {}}
    ref, mine, params = pair(dict(n_history=2, history_normalization_mode="exponential", history_normalization_decay=0.5))
    C, H, W = len(params.channel_names), params.img_shape_x, params.img_shape_y
    torch.manual_seed(0)
    inp = torch.randn(2, 3 * C, H, W)
    for mode in ("train", "eval"):
        outs = []
        for m in (ref, mine):
            m.train() if mode == "train" else m.eval()
            with torch.no_grad():
                outs.append(m(inp.clone()))
        out["err"][f"exponential_{mode}"] = rel(outs[1], outs[0])
    ref, mine, params = pair(dict(n_history=0, target="residual"))
    inp = torch.randn(2, C, H, W)
    ref.eval()
    mine.train()
    with torch.no_grad():
        s1 = ref(inp.clone())
        s2 = ref(s1.clone())
        ym = mine(inp.clone())
    out["err"]["residual_step1"], out["err"]["residual_step2"] = rel(ym[:, :C], s1), rel(ym[:, C:], s2)
    mine.eval()
    with torch.no_grad():
        out["err"]["residual_eval"] = rel(mine(inp.clone()), s1)
    return out


def run_checkpoints():
    """A checkpoint written by the upstream trainer (legacy and flexible format) restores into this framework's model
    and optimiser, and a checkpoint written here restores into the upstream trainer."""
    import tempfile

    tr, params, recipe = _upstream_trainer()
    nlat, nlon, n_out = params.img_shape_x, params.img_shape_y, len(params.channel_names)
    tr.optimizer = torch.optim.AdamW(tr.model.parameters(), lr=1e-3)
    tr.scheduler = torch.optim.lr_scheduler.StepLR(tr.optimizer, step_size=3)
    x = torch.randn(2, n_out, nlat, nlon)
    tr.model.train()
    tr.model(x).square().mean().backward()
    tr.optimizer.step()
    tr.scheduler.step()
    tr.iters, tr.epoch = 7, 2
    d = tempfile.mkdtemp(prefix="parity_ckpt_")
    legacy, flexible = os.path.join(d, "legacy_mp{mp_rank}.tar"), os.path.join(d, "flexible_mp{mp_rank}.tar")
    tr.save_checkpoint(legacy, checkpoint_mode="legacy")
    tr.save_checkpoint(flexible, checkpoint_mode="flexible")

    if ROOT not in sys.path:
        sys.path.append(ROOT)
    from makani_b200.models import model_registry as my_registry
    from makani_b200.utils import checkpoint as my_ckpt
    from makani_b200.utils.YParams import YParams as MyY

    mp = MyY(recipe, "sfno_tiny")
    for k, v in params.to_dict().items():
        mp[k] = v
    out = {"case": "checkpoints"}
    tr.model.eval()
    with torch.no_grad():
        y_ref = tr.model(x)
    for mode, path in (("legacy", legacy), ("flexible", flexible)):
        torch.manual_seed(123)
        mine = my_registry.get_model(mp)
        opt = torch.optim.AdamW(mine.parameters(), lr=5e-2)
        sch = torch.optim.lr_scheduler.StepLR(opt, step_size=3)
        iters, epoch = my_ckpt.restore_checkpoint(path, mine, optimizer=opt, scheduler=sch, mode=mode,
                                                  load_optimizer=(mode == "legacy"), load_scheduler=True, load_counters=True)
        mine.eval()
        with torch.no_grad():
            out[f"{mode}_forward"] = rel(mine(x), y_ref)
        out[f"{mode}_counters"] = [iters, epoch]
        out[f"{mode}_scheduler_epoch"] = sch.last_epoch
        if mode == "legacy":
            so, sm = tr.optimizer.state_dict(), opt.state_dict()
            out["legacy_optimizer_lr"] = sm["param_groups"][0]["lr"] / so["param_groups"][0]["lr"]
            out["legacy_optimizer_state"] = max(rel(sm["state"][k]["exp_avg"], so["state"][k]["exp_avg"]) for k in so["state"])
    # the other direction: written here, restored by the upstream trainer (its plain `torch.load` of a file that holds
    # the recipe object needs the opt-out of weights-only loading on this version of torch, also for its own files)
    os.environ["TORCH_FORCE_NO_WEIGHTS_ONLY_LOAD"] = "1"
    torch.manual_seed(5)
    mine = my_registry.get_model(mp)
    mine.eval()
    with torch.no_grad():
        y_mine = mine(x)
    for mode in ("legacy", "flexible"):
        path = os.path.join(d, "here_" + mode + "_mp{mp_rank}.tar")
        my_ckpt.save_checkpoint(path, mine, optimizer=None, scheduler=None, params=mp, iters=11, epoch=3, mode=mode)
        try:
            tr.restore_checkpoint(path, checkpoint_mode=mode, load_counters=True)
            tr.model.eval()
            with torch.no_grad():
                out[f"upstream_reads_{mode}"] = rel(tr.model(x), y_mine)
            out[f"upstream_reads_{mode}_counters"] = [tr.iters, tr.startEpoch]
        except Exception as e:
            out[f"upstream_reads_{mode}"] = f"{type(e).__name__}: {e}"[:300]
    return out


if __name__ == "__main__":
    import makani

    assert os.path.realpath(makani.__file__).startswith(os.path.realpath(os.path.join(ROOT, "baseline", "_ref"))), makani.__file__
    for name in (sys.argv[1:] or list(CASES) + ["losses", "metrics", "wrapped1", "wrapped2", "wrapped_features", "reshape_fields", "mpu_layers", "common_layers", "grids", "training_steps", "metrics_handler", "initialisation", "history_and_residual", "checkpoints"]):
        if name == "losses":
            res = run_losses()
        elif name == "metrics":
            res = run_metrics()
        elif name == "checkpoints":
            res = run_checkpoints()
        elif name == "wrapped_features":
            res = run_wrapped_features()
        elif name == "reshape_fields":
            res = run_reshape_fields()
        elif name == "mpu_layers":
            res = run_mpu_layers()
        elif name == "common_layers":
            res = run_common_layers()
        elif name == "grids":
            res = run_grids()
        elif name == "training_steps":
            res = run_training_steps()
        elif name == "metrics_handler":
            res = run_metrics_handler()
        elif name == "initialisation":
            res = run_initialisation()
        elif name == "history_and_residual":
            res = run_history_and_residual()
        elif name.startswith("wrapped"):
            res = run_wrapped(int(name[len("wrapped"):]))
        else:
            res = run(name)
        print(json.dumps(res))
        sys.stdout.flush()
